"""Host-side multi-rank logic on CPU: two gloo ranks shard a vocabulary, compute their
per-shard (max, index) pairs with the oracle, gather them with the package's own helper and
merge with the first-maximum rule; the result must equal greedy_index over the whole row."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def merge_rule(gathered: np.ndarray) -> np.ndarray:
    """[world, rows, 2] int32 (value bits, global index) -> [rows, 2]: greater value in IEEE
    total order wins, equal values go to the lowest global index (sampling.rs:162-173)."""
    world, rows, _ = gathered.shape
    out = np.zeros((rows, 2), np.int32)
    for t in range(rows):
        best = None
        for r in range(world):
            bits, idx = int(gathered[r, t, 0]) & 0xFFFFFFFF, int(gathered[r, t, 1])
            key = bits ^ (0xFFFFFFFF if bits & 0x80000000 else 0x80000000)
            if best is None or (key, -idx) > (best[0], -best[1]):
                best = (key, idx, gathered[r, t, 0])
        out[t] = (best[2], best[1])
    return out


def _worker(rank, world, port, vocab, rows, queue):
    import sys
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import tuisko_oracle as O
    from tuiskollm_b200 import dist as tkd, synth

    hidden = 1024
    shard = tkd.vocab_shard(vocab, world, rank)
    # every rank builds the same full plane from the seed and keeps only its rows
    wc, ws = synth.fp8_weights(5, 1, vocab, hidden)
    wc[vocab - 3], ws[vocab - 3] = wc[7], ws[7]  # a cross-shard duplicate row -> tie
    x = synth.normal_bf16(5, 2, (rows, hidden))
    codes, scales = O.quantize_e4m3(x)
    mine = O.fp8_projection(codes, scales, wc[shard.offset:shard.offset + shard.rows],
                            ws[shard.offset:shard.offset + shard.rows])
    bits = O.f32_to_bf16(mine.astype(np.float32))
    pairs = np.zeros((rows, 2), np.int32)
    for t in range(rows):
        i = O.greedy_index(bits[t])
        pairs[t] = (np.array([int(bits[t, i]) << 16], np.uint32).view(np.int32)[0], shard.offset + i)
    gathered = torch.zeros((world, rows, 2), dtype=torch.int32)
    tkd.gather_pairs(torch.from_numpy(pairs), gathered)
    merged = merge_rule(gathered.numpy())
    if rank == 0:
        full = O.f32_to_bf16(O.fp8_projection(codes, scales, wc, ws).astype(np.float32))
        expect = [O.greedy_index(full[t]) for t in range(rows)]
        queue.put((merged[:, 1].tolist(), expect, gathered.numpy()[:, :, 1].tolist()))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_vocab_shard_gather_merge():
    world, vocab, rows = 2, 2048, 3
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, vocab, rows, queue)) for r in range(world)]
    for p in procs:
        p.start()
    merged, expect, per_rank = queue.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert merged == expect
    # both ranks contributed candidates from their own index ranges
    assert all(0 <= i < vocab // 2 for i in per_rank[0]) and all(vocab // 2 <= i < vocab for i in per_rank[1])


def test_shard_arithmetic():
    import sys
    sys.path.insert(0, ROOT)
    from tuiskollm_b200 import dist as tkd

    assert tkd.vocab_shard(248320, 8, 7) == tkd.Shard(31040, 217280)
    assert [tkd.vocab_shard(248320, p, 0).rows for p in (1, 2, 4, 8)] == [248320, 124160, 62080, 31040]
    assert tkd.column_shard(17408, 8, 3) == tkd.Shard(2176, 6528)
    assert tkd.reduction_shard(17408, 8, 1) == tkd.Shard(2176, 2176)
    assert tkd.column_shard(8192, 8, 0).rows == 1024 and tkd.column_shard(12288, 8, 0).rows == 1536
    with pytest.raises(ValueError):
        tkd.vocab_shard(248320, 3, 0)
    with pytest.raises(ValueError):
        tkd.vocab_shard(248320, 2, 2)
    with pytest.raises(ValueError):
        tkd.column_shard(17408, 16, 0)
