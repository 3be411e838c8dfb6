"""Multi-rank host logic on CPU: two gloo ranks shard the heads of one attention layer, each computes its column
block (here with the CPU oracle standing in for the device kernels), and the all-gather rebuilds the full output."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tscale_b200 import shard


def test_split_range_is_a_partition():
    for n in (1, 7, 12, 32, 192):
        for world in (1, 2, 3, 4, 8):
            covered = []
            for r in range(world):
                b, e = shard.split_range(n, world, r)
                assert 0 <= b <= e <= n
                covered += list(range(b, e))
            assert covered == list(range(n))
            sizes = [shard.split_range(n, world, r)[1] - shard.split_range(n, world, r)[0] for r in range(world)]
            assert max(sizes) - min(sizes) <= 1


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, heads, d, result_path):
    from oracle import oracle as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(0)  # every rank generates the same inputs and keeps its own heads
    frag_lens = [70, 58]
    ln = sum(frag_lens)
    q = rng.standard_normal((ln, heads * d)).astype(np.float32)
    k = rng.standard_normal((ln, heads * d)).astype(np.float32)
    v = rng.standard_normal((ln, heads * d)).astype(np.float32)
    spans, ptr = O.window_spans(frag_lens, 16)
    O.set_threads(1)
    b, e = shard.head_shard(heads, world, rank)
    cols = slice(b * d, e * d)
    local = O.att_fwd(q[:, cols], k[:, cols], v[:, cols], spans, ptr, e - b, 0.5)["out"]
    full = shard.gather_head_blocks(torch.from_numpy(local), heads, d, world)
    want = O.att_fwd(q, k, v, spans, ptr, heads, 0.5)["out"]
    ok = np.array_equal(full.numpy(), want)
    # max over ranks of a per-rank time, the way bench.py reports it
    t = torch.tensor([float(rank + 1)])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ok = ok and float(t.item()) == world
    with open(result_path + str(rank), "w") as f:
        f.write("ok" if ok else "mismatch")
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_shard_heads_and_gather(tmp_path):
    world, heads, d = 2, 3, 16   # uneven: 2 heads + 1 head
    port = _free_port()
    path = str(tmp_path / "res")
    mp.spawn(_worker, args=(world, port, heads, d, path), nprocs=world, join=True)
    for r in range(world):
        assert open(path + str(r)).read() == "ok"


def test_unit_rects_cover_the_range_exactly():
    """tsa_shard_range + tsa_shard_rects: every (fragment, head) unit lands in exactly one rectangle of exactly one rank."""
    for frags, heads in ((4, 32), (16, 12), (3, 5), (1, 7)):
        for world in (1, 2, 3, 4, 8):
            seen = np.zeros((frags, heads), dtype=np.int32)
            for r in range(world):
                rects = shard.rank_rects(frags, heads, world, r)
                assert len(rects) <= 3
                b, e = shard.split_range(frags * heads, world, r)
                units = []
                for (f0, f1, h0, h1) in rects:
                    assert 0 <= f0 < f1 <= frags and 0 <= h0 < h1 <= heads
                    assert f1 - f0 == 1 or (h0 == 0 and h1 == heads)   # several fragments only with all heads
                    seen[f0:f1, h0:h1] += 1
                    units += [f * heads + h for f in range(f0, f1) for h in range(h0, h1)]
                assert units == list(range(b, e))                       # in unit order
            assert (seen == 1).all()
    # the long-context prefill: 4 fragments x 32 heads over 8 ranks = half the heads of one fragment each
    assert shard.rank_rects(4, 32, 8, 5) == [(2, 3, 16, 32)]
    assert shard.rank_rects(4, 32, 2, 1) == [(2, 4, 0, 32)]


def _worker_units(rank, world, port, frags, heads, d, seq, result_path):
    """Strong-scaling split of one batch: each rank computes its rectangle of (fragment, head) units into a compact
    block, the blocks are all-gathered, and the per-unit checksums of the gathered result equal those of the whole
    batch computed in one piece."""
    from oracle import oracle as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(1)
    ln = frags * seq
    q = rng.standard_normal((ln, heads * d)).astype(np.float32)
    k = rng.standard_normal((ln, heads * d)).astype(np.float32)
    v = rng.standard_normal((ln, heads * d)).astype(np.float32)
    O.set_threads(1)
    spans_all, ptr_all = O.window_spans([seq] * frags, 0)
    want = torch.from_numpy(O.att_fwd(q, k, v, spans_all, ptr_all, heads, 0.0)["out"]).to(torch.bfloat16)
    want_sums = shard.unit_checksums(want, frags, seq, heads, d)
    rects = shard.rank_rects(frags, heads, world, rank)
    assert len(rects) == 1
    f0, f1, h0, h1 = rects[0]
    rows, cols = slice(f0 * seq, f1 * seq), slice(h0 * d, h1 * d)
    spans, ptr = O.window_spans([seq] * (f1 - f0), 0)
    local = O.att_fwd(q[rows, cols], k[rows, cols], v[rows, cols], spans, ptr, h1 - h0, 0.0)["out"]
    local = torch.from_numpy(np.ascontiguousarray(local)).to(torch.bfloat16)
    gathered = torch.empty((world,) + tuple(local.shape), dtype=torch.bfloat16)
    shard.gather_blocks(local, gathered)
    ok = True
    for r in range(world):
        (g0, g1, k0, k1), = shard.rank_rects(frags, heads, world, r)
        sums = shard.unit_checksums(gathered[r], g1 - g0, seq, k1 - k0, d)
        ok = ok and torch.equal(sums, want_sums[g0:g1, k0:k1])
    with open(result_path + str(rank), "w") as f:
        f.write("ok" if ok else "mismatch")
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_split_units_and_gather_blocks(tmp_path):
    world = 2
    port = _free_port()
    path = str(tmp_path / "units")
    mp.spawn(_worker_units, args=(world, port, 2, 3, 16, 48, path), nprocs=world, join=True)
    for r in range(world):
        assert open(path + str(r)).read() == "ok"
