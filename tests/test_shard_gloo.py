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
