"""Multi-rank GPU tests of the two kernels that talk to peers over NVLink: the fused argmax
exchange (tk100_argmax_exchange) and the peer-memory sum (tk100_peer_sum_bf16).  Two ranks, one
process per GPU, run several steps eagerly and as graph replays; every result is compared with a
host restatement computed from data gathered with NCCL: the first-maximum merge
(tuisko-engine/src/sampling.rs:162-173 applied across shards) and a rank-ordered fp32 sum rounded
to BF16 once.  Skipped on a box with fewer than two GPUs.

No rank leaves early, every wait in the kernels is bounded, NVLS stays off and the kernels use
plain peer loads and stores."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORLD = 2


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _setup(rank, port):
    for p in (ROOT, os.path.join(ROOT, "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=WORLD, device_id=torch.device("cuda", rank))
    return dist


def _merge(gathered):
    """[world, rows, 2] int32 (value bits, global index) -> [rows, 2] by the first-maximum rule."""
    world, rows, _ = gathered.shape
    out = np.zeros((rows, 2), np.int32)
    for t in range(rows):
        best = None
        for r in range(world):
            bits, idx = int(gathered[r, t, 0]) & 0xFFFFFFFF, int(gathered[r, t, 1])
            if idx < 0:
                continue
            key = bits ^ (0xFFFFFFFF if bits & 0x80000000 else 0x80000000)
            if best is None or (key, -idx) > (best[0], -best[1]):
                best = (key, idx, int(gathered[r, t, 0]))
        out[t] = (best[2], best[1])
    return out


def _exchange_worker(rank, port):
    dist = _setup(rank, port)
    import time

    import tuiskollm_b200 as tk
    from oracle import tuisko_oracle as O
    from tuiskollm_b200 import dist as tkd, synth

    hidden, rows = 1024, 3
    vocab = WORLD * (128 * 3 + 64)  # shards that end in a 64-row tail tile
    shard = tkd.vocab_shard(vocab, WORLD, rank)
    ctx = tk.Context(device=rank, hidden=hidden)
    wc, ws = synth.fp8_weights(61, 1, vocab, hidden)  # every rank draws the same full plane
    up = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    _buf, _hdl, peers = tkd.alloc_exchange(rows, WORLD, torch.device("cuda", rank))
    op = tk.LmHeadOp(ctx, shard.rows, shard.offset)
    x = torch.zeros((rows, hidden), dtype=torch.int16, device="cuda")
    codes = torch.empty((rows, hidden), dtype=torch.uint8, device="cuda")
    scales = torch.empty((rows,), dtype=torch.float32, device="cuda")
    logits = torch.empty((rows, shard.rows), dtype=torch.int16, device="cuda")
    scratch = torch.zeros((rows,), dtype=torch.int64, device="cuda")
    pairs = torch.zeros((rows, 2), dtype=torch.int32, device="cuda")
    merged = torch.zeros((rows, 2), dtype=torch.int32, device="cuda")

    def set_weights(full_codes, full_scales):
        sl = slice(shard.offset, shard.offset + shard.rows)
        return up(full_codes[sl]), up(full_scales[sl].view(np.int16))

    w, s = set_weights(wc, ws)

    state = {"one_launch": False}

    def step():
        if state["one_launch"]:  # projection, argmax, exchange and merge in one kernel
            op.launch_sharded(None, rows, x, codes, scales, w, s, logits, None, scratch, WORLD, rank,
                              peers, merged)
            return
        op.launch(None, rows, x, codes, scales, w, s, logits, None, scratch, None)
        op.exchange(None, rows, WORLD, rank, scratch, peers, merged)

    def check(tag, xb, full_codes, full_scales):
        got = merged.cpu().numpy().copy()
        op.launch(None, rows, x, codes, scales, w, s, logits, None, scratch, pairs)  # finalize route
        torch.cuda.synchronize()
        gathered = torch.zeros((WORLD, rows, 2), dtype=torch.int32, device="cuda")
        dist.all_gather_into_tensor(gathered.view(-1), pairs.view(-1))
        expect = _merge(gathered.cpu().numpy())
        assert np.array_equal(got, expect), f"{tag}: rank {rank}: {got.tolist()} != {expect.tolist()}"
        # ... and equal to greedy_index over the whole vocabulary's BF16 logits as the two
        # shards wrote them (the selection rule the host sampler applies to that plane), which in
        # turn lie within tolerance of the CPU oracle's projection
        parts = [torch.empty_like(logits).view(torch.uint8) for _ in range(WORLD)]
        dist.all_gather(parts, logits.view(torch.uint8))  # NCCL has no 16-bit integer type
        plane = np.concatenate([p.cpu().numpy().view(np.uint16) for p in parts], axis=1)
        for t in range(rows):
            assert int(got[t, 1]) == O.greedy_index(plane[t]), f"{tag}: token {t}"
        oc, os_ = O.quantize_e4m3(xb)
        exp = O.fp8_projection(oc, os_, full_codes, full_scales)
        val = O.bf16_to_f32(plane).astype(np.float64)
        assert (np.abs(val - exp) / np.maximum(np.abs(exp), 0.1)).max() <= 1e-2, tag
        return got

    winners = set()
    for i in range(8):  # eager steps, fresh hidden rows every step, rank 1 late on odd steps;
        # the two forms of the exchange (own launch / inside the projection) alternate in pairs and
        # share the device step counter
        state["one_launch"] = (i // 2) % 2 == 1
        xb = synth.normal_bf16(61, 10 + i, (rows, hidden))
        x.copy_(up(xb.view(np.int16)))
        if rank == 1 and i % 2 == 1:
            time.sleep(0.05)
        step()
        torch.cuda.synchronize()
        got = check(f"eager step {i}", xb, wc, ws)
        winners.update(int(v) // shard.rows for v in got[:, 1])
    assert winners == {0, 1}, f"both shards should win some token, saw {winners}"

    # an exact cross-shard tie: the winning row of token 0 duplicated in the other shard
    xb = synth.normal_bf16(61, 20, (rows, hidden))
    oc, os_ = O.quantize_e4m3(xb)
    full = O.fp8_projection(oc, os_, wc, ws)
    best = int(np.argmax(full[0]))
    other = (best + vocab // 2) % vocab
    wc2, ws2 = wc.copy(), ws.copy()
    wc2[other], ws2[other] = wc[best], ws[best]
    w, s = set_weights(wc2, ws2)
    x.copy_(up(xb.view(np.int16)))
    step()
    torch.cuda.synchronize()
    got = check("cross-shard tie", xb, wc2, ws2)
    assert int(got[0, 1]) == min(best, other)

    # graph replay of the one-launch form: the step number lives on the device, the parities alternate
    state["one_launch"] = True
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    dist.barrier()
    with torch.cuda.graph(graph):
        step()
    for i in range(3):
        xb = synth.normal_bf16(61, 30 + i, (rows, hidden))
        x.copy_(up(xb.view(np.int16)))
        merged.fill_(-7)
        graph.replay()
        torch.cuda.synchronize()
        check(f"graph replay {i}", xb, wc2, ws2)
    assert ctx.device_status() == 0
    dist.barrier()
    torch.cuda.synchronize()
    dist.destroy_process_group()


def _peer_sum_worker(rank, port):
    dist = _setup(rank, port)
    import time

    import tuiskollm_b200 as tk
    from tuiskollm_b200 import dist as tkd, ops

    ctx = tk.Context(device=rank)
    capacity = 64 * 5120
    _buf, _hdl, peers = tkd.alloc_peer_sum(capacity, WORLD, torch.device("cuda", rank))
    gen = torch.Generator(device="cuda").manual_seed(100 + rank)

    def expected(partial):
        parts = [torch.empty_like(partial) for _ in range(WORLD)]
        dist.all_gather(parts, partial)
        acc = parts[0].clone()
        for p in parts[1:]:
            acc = acc + p  # fp32, rank order
        return acc.to(torch.bfloat16).view(torch.int16).cpu().numpy()

    # sizes alternate between the one-shot form (<= 16 384 values) and the two-shot form, and
    # between small and large calls of each, on one buffer; rank 1 is late on some steps so that
    # rank 0 runs a step ahead into the next form
    sizes = [5120, 64 * 5120, 5120, 16384, 16392, 8, 32 * 5120, 64 * 5120, 5120, 5120]
    for i, values in enumerate(sizes):
        partial = torch.randn(values, generator=gen, device="cuda", dtype=torch.float32) * (1 + i)
        out = torch.full((values + 8,), 0x5A5A, dtype=torch.int16, device="cuda")
        want = expected(partial)
        if rank == 1 and i % 3 == 1:
            time.sleep(0.05)
        ops.peer_sum_bf16(ctx, None, values, capacity, WORLD, rank, partial, peers, out)
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        assert np.array_equal(got[:values], want), f"step {i} ({values} values), rank {rank}"
        assert np.all(got[values:] == 0x5A5A), "wrote past the end of the output"
    # back-to-back launches without a host sync in between (a fast rank runs ahead on the device)
    outs, wants = [], []
    for i, values in enumerate([5120, 64 * 5120, 5120, 64 * 5120]):
        partial = torch.randn(values, generator=gen, device="cuda", dtype=torch.float32)
        wants.append(expected(partial))
        outs.append((torch.zeros(values, dtype=torch.int16, device="cuda"), partial))
    torch.cuda.synchronize()
    dist.barrier()
    for (out, partial) in outs:
        ops.peer_sum_bf16(ctx, None, partial.numel(), capacity, WORLD, rank, partial, peers, out)
    torch.cuda.synchronize()
    for i, ((out, _p), want) in enumerate(zip(outs, wants)):
        assert np.array_equal(out.cpu().numpy(), want), f"back-to-back launch {i}, rank {rank}"
    # graph replay of both forms
    for values in (5120, 48 * 5120):
        partial = torch.randn(values, generator=gen, device="cuda", dtype=torch.float32)
        out = torch.zeros(values, dtype=torch.int16, device="cuda")
        fn = lambda: ops.peer_sum_bf16(ctx, None, values, capacity, WORLD, rank, partial, peers, out)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        for i in range(3):
            partial.mul_(1.25).add_(float(rank))
            want = expected(partial)
            out.zero_()
            graph.replay()
            torch.cuda.synchronize()
            assert np.array_equal(out.cpu().numpy(), want), f"graph replay {i} of {values} values"
    assert ctx.device_status() == 0
    dist.barrier()
    torch.cuda.synchronize()
    dist.destroy_process_group()


def _spawn(worker):
    import torch.multiprocessing as mp

    mp.spawn(worker, args=(_free_port(),), nprocs=WORLD, join=True)


needs_two = pytest.mark.skipif(torch.cuda.device_count() < WORLD, reason="needs two GPUs")


@needs_two
def test_argmax_exchange_two_ranks_equals_host_merge():
    _spawn(_exchange_worker)


@needs_two
def test_peer_sum_two_ranks_mixed_sizes_equals_rank_ordered_sum():
    _spawn(_peer_sum_worker)
