//! Compiles the hand-written CUDA sources for sm_100a with nvcc and links the result.
//!
//! `TUISKO_SM100_CSRC` points at the directory holding the `.cu` files
//! (`tuiskollm_b200/csrc` of the kernel repository, next to `include/tuisko_sm100.h`);
//! the default assumes that repository is checked out as `vendor/tuisko-sm100`.
//! The source list is the one `tuiskollm_b200/build.py` compiles (`SOURCES`): keep them equal.

use std::path::PathBuf;
use std::process::Command;

const SOURCES: &[&str] = &[
    "norm_quant.cu",
    "fp8_proj.cu",
    "fp8_pair.cu",
    "fp8_pair_persist.cu",
    "fp8_mlp.cu",
    "gdn.cu",
    "materialize.cu",
    "nvfp4.cu",
    "nvfp4_pair.cu",
    "nvfp4_persist.cu",
    "peer_reduce.cu",
    "sampler.cu",
    "ops.cu",
    "static_entry.cu",
];

fn main() {
    let out = PathBuf::from(std::env::var("OUT_DIR").expect("OUT_DIR"));
    let csrc = std::env::var("TUISKO_SM100_CSRC")
        .map(PathBuf::from)
        .unwrap_or_else(|_| PathBuf::from("../../vendor/tuisko-sm100/tuiskollm_b200/csrc"));
    let nvcc = std::env::var("NVCC").unwrap_or_else(|_| "nvcc".to_string());
    let library = out.join("libtuisko_sm100.so");

    // Always the explicit -gencode form: plain -arch=sm_100a rejects tcgen05.*.
    let status = Command::new(&nvcc)
        .args(["-std=c++17", "-O3", "-lineinfo"])
        .args(["-gencode", "arch=compute_100a,code=sm_100a"])
        .args(["-Xcompiler", "-fPIC,-fvisibility=hidden", "-shared"])
        .args(["-Xptxas", "-warn-spills"])
        .arg("-o")
        .arg(&library)
        .args(SOURCES.iter().map(|source| csrc.join(source)))
        .args(["-lcudart_static", "-ldl", "-lrt", "-lpthread"])
        .status()
        .expect("running nvcc");
    assert!(status.success(), "nvcc failed building libtuisko_sm100.so");

    for source in SOURCES {
        println!("cargo:rerun-if-changed={}", csrc.join(source).display());
    }
    println!("cargo:rerun-if-env-changed=TUISKO_SM100_CSRC");
    println!("cargo:rustc-link-search=native={}", out.display());
    println!("cargo:rustc-link-lib=dylib=tuisko_sm100");
}
