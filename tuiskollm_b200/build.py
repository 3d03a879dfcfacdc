"""Builds ``libtuisko_sm100.so`` in-tree with nvcc for sm_100a (the only target)."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libtuisko_sm100.so")
SOURCES = ["norm_quant.cu", "fp8_proj.cu", "fp8_pair.cu", "fp8_pair_persist.cu", "fp8_mlp.cu", "gdn.cu", "materialize.cu", "nvfp4.cu", "nvfp4_pair.cu", "nvfp4_persist.cu", "peer_reduce.cu", "sampler.cu", "ops.cu", "static_entry.cu"]
HEADERS = ["common.cuh", "ptx.cuh", "kernels.h", "ops.hpp", "../../include/tuisko_sm100.h"]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; tuisko-kernels-sm100 has no prebuilt or CPU fallback")


def is_stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles the library when it is absent or older than its sources.  Several processes may
    call this at once (one rank per GPU): an exclusive file lock lets one of them compile, into a
    temporary file that is renamed into place, and the others then find the library fresh."""
    if not force and not is_stale():
        return LIB
    import fcntl

    with open(LIB + ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and not is_stale():  # another process built it while this one waited
                return LIB
            return _compile(verbose)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _compile(verbose: bool) -> str:
    """TK100_EXPERIMENT=1 in the environment of the build adds -DTK100_EXPERIMENT: the library
    then honours the TK100_DEBUG performance-experiment bits (which make results wrong); the
    default build has no such code."""
    tmp = "%s.%d.tmp" % (LIB, os.getpid())
    cmd = [
        nvcc_path(), "-std=c++17", "-O3", "-lineinfo",
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-Xcompiler", "-fPIC,-fvisibility=hidden", "-shared",
        "-Xptxas", "-v" if verbose else "-warn-spills",
        "-o", tmp,
    ] + (["-DTK100_EXPERIMENT"] if os.environ.get("TK100_EXPERIMENT") == "1" else []) \
      + [os.path.join(CSRC, s) for s in SOURCES] + ["-lcudart_static", "-ldl", "-lrt", "-lpthread"]
    env = dict(os.environ)
    # the image exports CC/CXX pointing at a private gcc; nvcc wants the system one
    if os.path.exists("/usr/bin/g++"):
        cmd[1:1] = ["-ccbin", "/usr/bin/g++"]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        if os.path.exists(tmp):
            os.unlink(tmp)
        raise RuntimeError("nvcc failed building libtuisko_sm100.so")
    os.replace(tmp, LIB)  # atomic: a concurrent loader sees the old file or the new one, whole
    return LIB


if __name__ == "__main__":
    print(build(force=True, verbose="-v" in sys.argv))
