"""GPU tests of the peer-memory sum (tk100_peer_sum_bf16) that one GPU can run: world = 1 (the
rank's own buffer is its only peer) for both forms, graph replay over many steps, the bounded
wait for a peer that never arrives, and rejected arguments.  The multi-rank arithmetic runs in
`bench.py --gpus N`, which checks the result against an NCCL all-reduce before timing it."""
import numpy as np
import pytest
import torch

from gpu_util import graph_replay, host

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tk():
    import tuiskollm_b200 as tk
    return tk


def bf16_rne(x: torch.Tensor) -> np.ndarray:
    return host(x.to(torch.bfloat16).view(torch.int16)).view(np.uint16)


@pytest.mark.parametrize("values", [8, 5120, 16384, 16392, 256 * 5120])
def test_single_rank_sum_is_the_rounded_partial(tk, values):
    """With one rank the sum is the partial itself: the output must be its nearest-even BF16
    rounding in the one-shot form (<= 16 384 values) and in the two-shot form, step after step
    (the parities alternate) and with a buffer sized for more than the call uses."""
    from tuiskollm_b200 import ops

    ctx = tk.Context(device=0)
    capacity = 512 * 5120
    buf = torch.zeros(ops.peer_sum_bytes(capacity, 1) // 8, dtype=torch.int64, device="cuda")
    out = torch.empty(values + 8, dtype=torch.int16, device="cuda")
    gen = torch.Generator(device="cuda").manual_seed(values)
    for step in range(4):
        partial = torch.randn(values, generator=gen, device="cuda", dtype=torch.float32) * (step + 1)
        out.fill_(0x5A5A)
        ops.peer_sum_bf16(ctx, None, values, capacity, 1, 0, partial, [buf.data_ptr()], out)
        torch.cuda.synchronize()
        got = host(out).view(np.uint16)
        assert np.array_equal(got[:values], bf16_rne(partial)), step
        assert np.all(got[values:] == 0x5A5A), "wrote past the end of the output"
    assert ctx.device_status() == 0


def test_graph_replay_advances_the_step_on_the_device(tk):
    """A captured launch is replayed: the step number lives on the device, so every replay uses
    fresh flags and the other parity."""
    from tuiskollm_b200 import ops

    ctx = tk.Context(device=0)
    values = 64 * 5120
    buf = torch.zeros(ops.peer_sum_bytes(values, 1) // 8, dtype=torch.int64, device="cuda")
    partial = torch.randn(values, device="cuda", dtype=torch.float32)
    out = torch.zeros(values, dtype=torch.int16, device="cuda")
    ops.peer_sum_bf16(ctx, None, values, values, 1, 0, partial, [buf.data_ptr()], out)
    graph = graph_replay(lambda: ops.peer_sum_bf16(ctx, None, values, values, 1, 0, partial,
                                                    [buf.data_ptr()], out))
    for i in range(5):
        partial.mul_(1.5)
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert np.array_equal(host(out).view(np.uint16), bf16_rne(partial)), i
    assert ctx.device_status() == 0


@pytest.mark.parametrize("values", [5120, 64 * 5120])
def test_missing_peer_runs_into_the_bounded_wait(tk, values):
    """world = 2 on one GPU: rank 1 does not exist, so its flag never comes; the kernel gives up
    after its limit and reports TK100_DEVICE_WAIT_TIMEOUT instead of hanging."""
    from tuiskollm_b200 import _lib, ops

    ctx = tk.Context(device=0)
    words = ops.peer_sum_bytes(values, 2) // 8
    bufs = torch.zeros((2, (words + 31) // 32 * 32), dtype=torch.int64, device="cuda")
    partial = torch.randn(values, device="cuda", dtype=torch.float32)
    out = torch.zeros(values, dtype=torch.int16, device="cuda")
    ops.peer_sum_bf16(ctx, None, values, values, 2, 0, partial,
                      [bufs[0].data_ptr(), bufs[1].data_ptr()], out)
    torch.cuda.synchronize()
    assert ctx.device_status() & _lib.DEVICE_WAIT_TIMEOUT


def test_rejected_arguments(tk):
    from tuiskollm_b200 import ops

    ctx = tk.Context(device=0)
    buf = torch.zeros(ops.peer_sum_bytes(1024, 1) // 8, dtype=torch.int64, device="cuda")
    partial = torch.zeros(2048, device="cuda", dtype=torch.float32)
    out = torch.zeros(2048, dtype=torch.int16, device="cuda")
    with pytest.raises(tk.GpuError):  # not a multiple of 8
        ops.peer_sum_bf16(ctx, None, 12, 1024, 1, 0, partial, [buf.data_ptr()], out)
    with pytest.raises(tk.GpuError):  # beyond the capacity the buffer was sized for
        ops.peer_sum_bf16(ctx, None, 2048, 1024, 1, 0, partial, [buf.data_ptr()], out)
    with pytest.raises(tk.GpuError):  # rank outside the world
        ops.peer_sum_bf16(ctx, None, 1024, 1024, 1, 1, partial, [buf.data_ptr()], out)
    with pytest.raises(tk.GpuError):  # misaligned buffer
        ops.peer_sum_bf16(ctx, None, 1024, 1024, 1, 0, partial, [buf.data_ptr() + 8], out)
    assert ops.peer_sum_bytes(0, 1) == 0 and ops.peer_sum_bytes(1024, 9) == 0
