"""Decode workload of bench.py: int8 KV-cache attention step over 64 sequences (context lengths uniform in
[1024, 8192], 16 heads x 128, fp16 scale per (token, head)), one new token appended per step.

A step = tsa_kv_append + tsa_att_decode for all sequences.  The metric is algorithmic HBM traffic per second:
per step sum over sequences of keys * H * (2 * D bytes of int8 K and V + two fp16 scales).
"""
import json
import os
import time

import numpy as np

from .util import ClockSampler, load_peaks

N_SEQ, HEADS, D = 64, 16, 128
CTX_LO, CTX_HI = 1024, 8192
SEED = 3


def step_bytes(ctx_lens, heads, d, scale_bytes):
    # after the append a sequence of length n attends n - 1 keys (the new token itself is excluded)
    return float(sum((n - 1) * heads * (2 * d + 2 * scale_bytes) for n in ctx_lens))


def cpu_decode_sample(n_seq_sample, threads):
    """The reference's CPU decode (oracle/_ref, else the oracle port) on a few sequences of the same shape."""
    from concurrent.futures import ThreadPoolExecutor
    from oracle import oracle as O
    rng = np.random.default_rng(SEED)
    ctx = rng.integers(CTX_LO, CTX_HI + 1, N_SEQ)[:n_seq_sample]
    use_ref = O.ref() is not None
    jobs = []
    for n in ctx:
        kc = rng.integers(-127, 128, (n, HEADS * D)).astype(np.int8)
        vc = rng.integers(-127, 128, (n, HEADS * D)).astype(np.int8)
        ks = (rng.random((n, HEADS)) * 2e-4 + 1e-4).astype(np.float32)
        vs = np.full((n, HEADS), 1 / 24.0, dtype=np.float32)
        q8 = rng.integers(-127, 128, (HEADS * D,)).astype(np.int8)
        qs = np.full((HEADS,), 1 / 24.0, dtype=np.float32)
        jobs.append((kc, ks, vc, vs, q8, qs))

    def one(job):
        kc, ks, vc, vs, q8, qs = job
        O.decode_step(kc, ks, vc, vs, q8, qs, HEADS, 1 << 30, 0.0, exp_mode="poly", use_ref=use_ref)

    reps = 3
    t0 = time.perf_counter()
    with ThreadPoolExecutor(max_workers=threads) as ex:
        for _ in range(reps):
            list(ex.map(one, jobs))
    sec = (time.perf_counter() - t0) / reps
    nbytes = step_bytes([int(n) for n in ctx], HEADS, D, 4)  # the reference keeps f32 key scales
    return nbytes / sec / 1e9, "reference" if use_ref else "port", \
        "%d sequences of the same length distribution, one step, %d repetitions" % (n_seq_sample, reps), sec


def config(args):
    return {"workload": "decode", "sequences": N_SEQ, "context": "uniform[%d,%d]" % (CTX_LO, CTX_HI), "heads": HEADS,
            "head_dim": D, "kv_dtype": "i8", "scale_dtype": "f16", "window": "full", "append_per_step": 1,
            "l2": "KV cache (about 1.2 GB per step) is larger than L2", "sharding": "sequences, per-GPU work fixed"}


def run(args, rank, world, local_rank, emit=True, quick=False):
    """emit=False: return the line instead of printing it; quick: no end-to-end leg and no CPU baseline (the short run
    bench.py adds to its default line)."""
    if args.impl == "reference":
        if rank != 0:
            return
        threads = os.cpu_count() or 1
        vals = []
        for i in range(args.warmup + args.steps):
            gbs, kind, sample, sec = cpu_decode_sample(8, threads)
            if i >= args.warmup:
                vals.append((gbs, sec))
        gbs = float(np.mean([v[0] for v in vals]))
        print(json.dumps({
            "impl": "reference", "metric": "decode_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1000.0 * float(np.mean([v[1] for v in vals])), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "i8", "data": "synthetic", "config": config(args),
            "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": kind, "sample": sample},
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}))
        return

    import torch
    import torch.distributed as dist
    from tscale_b200 import ops

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    steps, warmup = args.steps, max(args.warmup, 3)
    rng = np.random.default_rng(SEED + 1000 * rank)
    ctx0 = [int(x) for x in rng.integers(CTX_LO, CTX_HI + 1, N_SEQ)]
    cap = CTX_HI + steps + warmup + 8 + 2 * steps
    cache = ops.KVCache(N_SEQ, cap, HEADS, D, dev, scale_dtype=torch.float16, out_dtype=torch.float32)
    gen = torch.Generator(device=dev)
    gen.manual_seed(SEED + 1000 * rank)
    cache.k.copy_(torch.randint(-127, 128, cache.k.shape, generator=gen, device=dev, dtype=torch.int8))
    cache.v.copy_(torch.randint(-127, 128, cache.v.shape, generator=gen, device=dev, dtype=torch.int8))
    cache.k_scale.copy_((torch.rand(cache.k_scale.shape, generator=gen, device=dev) * 2e-4 + 1e-4).half())
    cache.v_scale.copy_((torch.rand(cache.v_scale.shape, generator=gen, device=dev) * 0.02 + 0.01).half())
    cache.ctx_lens.copy_(torch.tensor(ctx0, dtype=torch.int32))
    cache.max_ctx = max(ctx0)
    row = HEADS * D
    k_new = torch.randint(-127, 128, (N_SEQ, row), generator=gen, device=dev, dtype=torch.int8)
    v_new = torch.randint(-127, 128, (N_SEQ, row), generator=gen, device=dev, dtype=torch.int8)
    ks_new = (torch.rand((N_SEQ, HEADS), generator=gen, device=dev) * 2e-4 + 1e-4).half()
    vs_new = (torch.rand((N_SEQ, HEADS), generator=gen, device=dev) * 0.02 + 0.01).half()
    q = torch.randint(-127, 128, (N_SEQ, row), generator=gen, device=dev, dtype=torch.int8)
    qs = torch.full((N_SEQ, HEADS), 1 / 24.0, device=dev)
    out = torch.empty((N_SEQ, row), dtype=torch.float32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    launches = [0]
    lens = list(ctx0)

    def step():
        cache.append(k_new, ks_new, v_new, vs_new, status=status)
        cache.decode(q, qs, 1 << 30, 0.0, out=out, status=status)
        launches[0] += 3  # append, per-chunk partials, merge

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        step()
        lens = [n + 1 for n in lens]
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    launches[0] = 0
    nbytes = 0.0
    barrier()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        step()
        lens = [n + 1 for n in lens]
        nbytes += step_bytes(lens, HEADS, D, 2)
    t1.record()
    barrier()
    ms_total = t0.elapsed_time(t1)
    timed_launches = launches[0]
    clocks = sampler.stop() if rank == 0 else None
    assert int(status.item()) == 0
    tt = torch.tensor([ms_total], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    ms_step = float(tt.item()) / steps
    value = nbytes / steps * world / (ms_step * 1e-3) / 1e9

    # the dominant kernel alone (partials + merge), events around each launch
    evs = []
    for _ in range(min(steps, 20)):
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        cache.decode(q, qs, 1 << 30, 0.0, out=out, status=status)
        e1.record()
        evs.append((e0, e1))
    torch.cuda.synchronize()
    k_ms = float(np.mean([a.elapsed_time(b) for a, b in evs]))
    k_bytes = step_bytes(lens, HEADS, D, 2)

    e2e = None
    if not quick and not getattr(args, "no_e2e", False):
        # end to end: the step's host inputs (query, new K/V rows and scales) come from pinned memory, the result goes back
        host = {n: t.cpu().pin_memory() for n, t in (("q", q), ("qs", qs), ("k", k_new), ("v", v_new), ("ks", ks_new), ("vs", vs_new))}
        host_out = torch.empty(out.shape, dtype=out.dtype).pin_memory()
        h2d = sum(t.numel() * t.element_size() for t in host.values())
        d2h = host_out.numel() * host_out.element_size()
        e_steps = min(steps, 50)

        def e2e_step():
            q.copy_(host["q"], non_blocking=True)
            qs.copy_(host["qs"], non_blocking=True)
            k_new.copy_(host["k"], non_blocking=True)
            v_new.copy_(host["v"], non_blocking=True)
            ks_new.copy_(host["ks"], non_blocking=True)
            vs_new.copy_(host["vs"], non_blocking=True)
            step()
            host_out.copy_(out, non_blocking=True)

        e2e_step()
        lens = [n + 1 for n in lens]
        barrier()
        e_bytes = 0.0
        t0.record()
        for _ in range(e_steps):
            e2e_step()
            lens = [n + 1 for n in lens]
            e_bytes += step_bytes(lens, HEADS, D, 2)
        t1.record()
        barrier()
        tt = torch.tensor([t0.elapsed_time(t1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e_ms = float(tt.item()) / e_steps
        e2e = {"value": e_bytes / e_steps * world / (e_ms * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": e_ms, "steps": e_steps}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peaks = load_peaks()
    achieved = k_bytes / (k_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": "DecodePartialKernel<128> + DecodeCombineKernel<128>", "achieved": achieved,
                "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                "peak_source": "MEASURED_PEAKS.json copy bandwidth (%s)" % peaks["_source"], "frac_of_8tbs_nominal": achieved / 8000.0,
                "ms_per_launch": k_ms, "algorithmic_bytes_per_launch": k_bytes,
                # not measured in this run: the ratio comes from the ncu capture of this workload at this size
                # (profiles/decode_partial_i8_d128_64seq.md: 1.1588 GB of DRAM traffic for 1.166 GB algorithmic)
                "traffic": 0.994 * k_bytes, "traffic_source": "algorithmic bytes x 0.994, the dram/algorithmic ratio of the committed ncu capture "
                                                                "profiles/decode_partial_i8_d128_64seq.md (same workload and size); not re-measured per run"}
    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline and not quick:
        threads = os.cpu_count() or 1
        gbs, kind, sample, sec = cpu_decode_sample(8, threads)
        cpu_baseline = {"value": gbs, "unit": "GB/s", "cores": threads, "kind": kind, "sample": sample, "seconds": sec}
    line = {
        "metric": "decode_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "i8", "data": "synthetic",
        "config": config(args), "clocks": clocks, "e2e": e2e, "gpu_launches": timed_launches, "roofline": roofline,
        "cpu_baseline": cpu_baseline}
    if not emit:
        return line
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
