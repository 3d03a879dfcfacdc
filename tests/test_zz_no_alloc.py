"""The context-free FP8 projection for hosts that may not allocate device memory (engines
with a fixed arena and a no-allocation gate; guest code in a process whose CUDA allocator
it does not own).  Its scratch is a fixed array inside the library, so the checks here are:
same output as the context entry point, on two calls in a row that share that array, no
device allocation across the calls, and clear refusals beyond the array's capacity.

Collected last on purpose (file name): a failure here cannot hide another test's result."""
import numpy as np
import pytest
import torch

from gpu_util import assert_inactive_untouched, dev, host, max_relative_error, sentinel_plane

pytestmark = pytest.mark.gpu


def _u16(t):
    return host(t.view(torch.int16)).view(np.uint16)


@pytest.mark.parametrize("rows,out_rows", [(3, 2064), (32, 8192), (64, 8192), (100, 2048), (200, 16384), (256, 16384)])
def test_static_entry_matches_context_entry_on_two_calls(oracle, rows, out_rows):
    import tuiskollm_b200 as tk
    from tuiskollm_b200 import ops, synth

    hidden = 5120
    ctx = tk.Context(device=0)
    w, s = synth.torch_fp8_weights(31, out_rows, out_rows, hidden, "cuda")  # drawn on the device
    s = s.view(torch.int16)
    outs = []
    for call in range(2):  # second call: new activations, same shared scratch
        xb = synth.normal_bf16(31, 100 + call, (rows, hidden))
        codes = torch.empty((rows, hidden), dtype=torch.uint8, device="cuda")
        scales = torch.empty((rows,), dtype=torch.float32, device="cuda")
        ref = sentinel_plane((rows + 1, out_rows), torch.int16)
        got = sentinel_plane((rows + 1, out_rows), torch.int16)
        tk.Fp8ProjectionOp(ctx).launch(None, rows, out_rows, hidden, dev(xb.view(np.int16)), codes,
                                       scales, w, s, ref)
        torch.cuda.synchronize()
        route = ctx.last_kernel
        free_before, _ = torch.cuda.mem_get_info()
        ops.fp8_projection_static(None, rows, out_rows, hidden, codes, scales, w, s, got)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        if call == 1:  # the first call may load lazily-bound code; after that nothing moves
            assert free_after == free_before, "the static entry point changed free device memory"
        a, b = _u16(got)[:rows], _u16(ref)[:rows]
        exp = (b.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        # same tolerance as the projection parity tests: max relative error 1e-2 (floor 0.25)
        assert max_relative_error(a, exp, 0.25) <= 1e-2
        # wherever the context route runs the same kernel (it moves to CTA pairs from 256 rows),
        # both pick the same tile and split and add the partials in the same order: equal bits
        if route.startswith("fp8_projection_kernel"):
            assert np.array_equal(a, b)
        assert_inactive_untouched(got, rows)
        oc, os_ = oracle.quantize_e4m3(xb)
        assert max_relative_error(a, oracle.fp8_projection(oc, os_, host(w), host(s).view(np.uint16)), 0.25) <= 1e-2
        outs.append(a.copy())
    assert not np.array_equal(outs[0], outs[1])
    assert ctx.device_status() == 0
    # no bounded wait gave up on the static route either; reading clears the word
    assert ops.fp8_projection_static_status() == 0
    assert ops.fp8_projection_static_status() == 0


def test_static_entry_refuses_what_its_scratch_cannot_hold():
    import tuiskollm_b200 as tk
    from tuiskollm_b200 import ops

    hidden = 5120
    codes = torch.zeros((300, hidden), dtype=torch.uint8, device="cuda")
    scales = torch.ones((300,), dtype=torch.float32, device="cuda")
    w = torch.zeros((4096, hidden), dtype=torch.uint8, device="cuda")
    s = torch.zeros((4096,), dtype=torch.int16, device="cuda")
    out = torch.zeros((300, 4096), dtype=torch.int16, device="cuda")
    with pytest.raises(tk.GpuError) as info:
        ops.fp8_projection_static(None, ops.STATIC_MAX_ROWS + 1, 4096, hidden, codes, scales, w, s, out)
    assert info.value.code == "gpu.launch" and "row count" in str(info.value)
    # 256 rows x 4096 outputs would split K four ways: 16 MiB of partial tiles > 8 MiB
    with pytest.raises(tk.GpuError) as info:
        ops.fp8_projection_static(None, 256, 4096, hidden, codes, scales, w, s, out)
    assert info.value.code == "gpu.arena" and "static scratch holds" in str(info.value)
    with pytest.raises(tk.GpuError) as info:
        ops.fp8_projection_static(None, 1, 4096, hidden, codes, scales, w.data_ptr() + 16, s, out)
    assert info.value.code == "gpu.launch" and "misaligned" in str(info.value)
    torch.cuda.synchronize()
