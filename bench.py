#!/usr/bin/env python
"""Benchmark of the quantized attention path on B200.

    python bench.py --gpus N --steps K --warmup W [--workload longctx|prefill125m|train15b|decode|infer|neighbours] [--impl reference]

Default workload `longctx` is the long-context prefill, the largest single-GPU configuration of the path:
4 fragments x 32768 tokens, 32 heads x 128, full causal, e4m3 Q/K/V with per-row f32 scales, bf16 output.
Inputs are seeded synthetic N(0,1)*0.5, quantised on the GPU by the library's abs-max quantiser.  The metric is
algorithmic attention TFLOP/s: 4 * D * (attended pairs) per (fragment, head), masked-out work inside partially
filled tiles not counted.

One process per GPU.  With N > 1 the 128 (fragment, head) units of the ONE batch are split contiguously over the
ranks (tsa_shard_range / tsa_shard_rects), every rank runs the forward on its units only, and every rank ends
the step with the whole bf16 output: the attention kernel itself stores its rows into all ranks' buffers
(tsa_att_fwd_to over symmetric memory, one cross-rank barrier per step); `--gather nccl` all-gathers the blocks over
NCCL slice by slice instead, `--gather scatter` uses the library's copy kernel.  Strong scaling, `value` = the whole batch's flops / the slowest rank's step.
At N = 1 the line also carries short runs of the other workloads (`also`: prefill125m, train15b, decode).

The other workloads (`--workload prefill125m|train15b|decode|infer`) keep per-GPU work fixed (weak scaling).

`--impl reference` times the reference's own CPU attention (oracle/_ref, else the oracle port) on the host
cores, on a bounded sample of the same workload.
"""
import argparse
import json
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from benchlib.util import ClockSampler, load_peaks  # noqa: E402


# ----------------------------------------------------------------------------------------------------
# workloads
def pairs_window(seq, window):
    """attended (query, key) pairs of one fragment: row i sees min(i, window) keys (all i keys if window <= 0)"""
    if window <= 0 or window >= seq:
        return seq * (seq - 1) // 2
    return window * (window - 1) // 2 + (seq - window) * window


WORKLOADS = {
    # name: fragments, seq, heads, head_dim, qk dtype, layers [(window, slope)], backward?
    "prefill125m": dict(frags=16, seq=4096, heads=12, d=64, qk="e4m3", v="e4m3",
                        layers=[(64, 0.5), (64, 0.5), (64, 0.5), (0, 0.0)], bwd=False, seed=1),
    "train15b": dict(frags=8, seq=4096, heads=16, d=128, qk="i8", v="e4m3",
                     layers=[(0, 0.0), (256, 0.0)], bwd=True, seed=2),
    "longctx": dict(frags=4, seq=32768, heads=32, d=128, qk="e4m3", v="e4m3", layers=[(0, 0.0)], bwd=False, seed=4),
}
SM_COUNT = 148           # B200
EX2_PER_CLK_PER_SM = 16  # special-function results per clock and SM: one exponential per attended pair


def layer_flops(w, window):
    return 4.0 * w["d"] * pairs_window(w["seq"], window) * w["frags"] * w["heads"]


def workload_config(name, w, strong=False):
    cfg = {"workload": name, "fragments": w["frags"], "seq_len": w["seq"], "heads": w["heads"], "head_dim": w["d"],
           "qk_dtype": w["qk"], "v_dtype": w["v"],
           "layers": [{"window": "full" if win <= 0 else win, "alibi_slope": sl} for win, sl in w["layers"]],
           "backward": w["bwd"], "l2": "inputs larger than L2 (each layer has its own Q/K/V set)"}
    if strong:
        cfg["sharding"] = ("the batch's fragment x head units split contiguously over the ranks; every rank ends the step with the whole "
                           "bf16 output (gathered inside the timed region: by the attention kernel's own peer stores, or over NCCL)")
    else:
        cfg["sharding"] = "fragment x head, per-GPU work fixed"
    return cfg


# ----------------------------------------------------------------------------------------------------
# CPU arm: the reference's own CPU attention on a bounded sample
def cpu_sample_inputs(w, layer_idx, heads, seed):
    """One fragment of the workload's inputs for `heads` heads, generated with the GPU recipe (N(0,1)*0.5, abs-max 8-bit
    quantisation) through the oracle, dequantised to the f32 the reference's CPU code takes."""
    from oracle import oracle as O
    rng = np.random.default_rng(seed * 1000 + layer_idx)
    length, hd = w["seq"], heads * w["d"]
    res = []
    for _, dt in (("q", w["qk"]), ("k", w["qk"]), ("v", w["v"])):
        x = (rng.standard_normal((length, hd)) * 0.5).astype(np.float32)
        b, s = O.quant_rows("absmax", dt, 0.0, x, w["d"])
        deq = (O.dequant(b, dt).reshape(length, heads, w["d"]) * s.T[:, :, None]).reshape(length, hd)
        res.append(np.ascontiguousarray(deq, dtype=np.float32))
    return res


def row_sample_spans(seq, window, every):
    """Spans of one fragment in which only every `every`-th query row attends (rows without spans cost the reference's
    ComputeValLookup nothing, code/gpt/compute/gpt_cpu.cpp:411-431): a row subsample of the workload.  Returns
    (spans, span_ptr, attended pairs)."""
    spans, ptr, pairs = [], [0], 0
    for i in range(seq):
        lo = 0 if window <= 0 else max(0, i - window)
        if i % every == every - 1 and i - 1 >= lo:
            spans.append((lo, i - 1))
            pairs += i - lo
        ptr.append(len(spans))
    return np.array(spans, dtype=np.int32).reshape(-1, 2), np.array(ptr, dtype=np.int32), pairs


def make_cpu_sample(w):
    """About 10-20 s of host work: per distinct layer type one fragment, a few heads, every k-th query row."""
    budget_pairs = 6.0e7  # attended pairs per pass over the sample (all layer types together)
    kinds = []
    for idx, (window, slope) in enumerate(w["layers"]):
        if (window, slope) not in [(k[1], k[2]) for k in kinds]:
            kinds.append((idx, window, slope))
    sample = []
    for idx, window, slope in kinds:
        heads = min(w["heads"], 8)
        full = pairs_window(w["seq"], window) * heads
        every = max(1, int(np.ceil(full / (budget_pairs / len(kinds)))))
        spans, ptr, pairs = row_sample_spans(w["seq"], window, every)
        q, k, v = cpu_sample_inputs(w, idx, heads, w["seed"])
        sample.append(dict(window=window, slope=slope, heads=heads, every=every, spans=spans, ptr=ptr, pairs=pairs, q=q, k=k, v=v))
    return sample


def run_cpu_sample(w, sample, threads):
    """Runs the reference's CPU forward on the sample, one (layer type, head) job per host thread; returns
    (seconds, flops, kind)."""
    from concurrent.futures import ThreadPoolExecutor
    from oracle import oracle as O
    use_ref = "fast" if O.ref(fast=True) is not None else (O.ref() is not None)
    kind = "reference" if use_ref else "port"
    O.set_threads(1)
    jobs, flops = [], 0.0
    d = w["d"]
    for smp in sample:
        for h in range(smp["heads"]):
            cols = slice(h * d, (h + 1) * d)
            jobs.append((np.ascontiguousarray(smp["q"][:, cols]), np.ascontiguousarray(smp["k"][:, cols]),
                         np.ascontiguousarray(smp["v"][:, cols]), smp["spans"], smp["ptr"], smp["slope"]))
        flops += 4.0 * d * smp["pairs"] * smp["heads"]

    def one(job):
        q1, k1, v1, spans, ptr, slope = job
        O.att_fwd(q1, k1, v1, spans, ptr, 1, slope, use_ref=use_ref)

    t0 = time.perf_counter()
    with ThreadPoolExecutor(max_workers=threads) as ex:
        list(ex.map(one, jobs))
    return time.perf_counter() - t0, flops, kind


def sample_text(w, sample):
    return "; ".join("1 fragment x %d tokens x %d heads, window %s, slope %g, every %squery row" %
                     (w["seq"], s["heads"], "full" if s["window"] <= 0 else s["window"], s["slope"],
                      "" if s["every"] == 1 else "%d-th " % s["every"]) for s in sample)


def cpu_build_text(kind):
    if kind != "reference":
        return "oracle port (oracle/tsa_oracle.cpp)"
    return "the reference's own sources, -O3 -march=x86-64-v3 -mavxvnni (oracle/_ref/libtsa_ref_fast.so), one job per host thread"


def cpu_baseline_block(w, seconds_target=10.0):
    sample = make_cpu_sample(w)
    threads = os.cpu_count() or 1
    total, reps = 0.0, 0
    while reps < 2 or (total < seconds_target and reps < 50):
        sec, flops, kind = run_cpu_sample(w, sample, threads)
        total += sec
        reps += 1
    sec = total / reps
    return {"value": flops / sec / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": kind,
            "sample": sample_text(w, sample) + " (forward only), %d passes" % reps, "seconds": total, "build": cpu_build_text(kind)}


def reference_arm(args, name, w, rank):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    sample = make_cpu_sample(w)
    times = []
    for i in range(args.warmup + args.steps):
        sec, flops, kind = run_cpu_sample(w, sample, threads)
        if i >= args.warmup:
            times.append(sec)
    ms = 1000.0 * sum(times) / len(times)
    value = flops / (ms * 1e-3) / 1e12
    line = {
        "impl": "reference", "metric": "attention_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong" if name == "longctx" else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(name, w, strong=(name == "longctx")),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": kind, "sample": sample_text(w, sample),
                         "build": cpu_build_text(kind)},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------------------------------
# peaks measured on this GPU (cuBLASLt through torch), the way MEASURED_PEAKS.json measured bf16
def measure_fp8_peak(torch, dev):
    try:
        n = 8192
        a = torch.randn((n, n), device=dev).to(torch.float8_e4m3fn)
        b = torch.randn((n, n), device=dev).to(torch.float8_e4m3fn).t()
        one = torch.ones((), device=dev)
        for _ in range(3):
            torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        best = 1e9
        for _ in range(8):
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        return 2.0 * n ** 3 / (best * 1e-3) / 1e12
    except Exception:  # noqa: BLE001  (a peak probe must not break the benchmark)
        return None


def measure_int8_peak(torch, dev):
    try:
        n = 8192
        a = torch.randint(-127, 128, (n, n), device=dev, dtype=torch.int8)
        b = torch.randint(-127, 128, (n, n), device=dev, dtype=torch.int8).t()
        for _ in range(3):
            torch._int_mm(a, b)
        best = 1e9
        for _ in range(8):
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._int_mm(a, b)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        return 2.0 * n ** 3 / (best * 1e-3) / 1e12
    except Exception:  # noqa: BLE001
        return None


_PEAK_CACHE = {}


def tensor_roofline(torch, dev, w, kernel, achieved, ms, flops, clocks):
    """Roofline block of a tensor-bound attention kernel: the denominator is the measured dense GEMM rate of the operand
    type the kernel's MMAs run in (e4m3 or int8), the bf16 figure of MEASURED_PEAKS.json is kept beside it, and
    frac_mufu_bound compares with the ceiling one exponential per attended pair puts on the path at the sampled clock."""
    peaks = load_peaks()
    if "fp8" not in _PEAK_CACHE:
        _PEAK_CACHE["fp8"] = measure_fp8_peak(torch, dev)
        _PEAK_CACHE["int8"] = measure_int8_peak(torch, dev)
    fp8_peak, int8_peak = _PEAK_CACHE["fp8"], _PEAK_CACHE["int8"]
    if w["qk"] == "i8":
        peak, src = int8_peak, "int8 x int8 -> int32 GEMM 8192^3 through cuBLASLt, measured in this run (QK^T runs as kind::i8, PV as kind::f8f6f4)"
    else:
        peak, src = fp8_peak, "e4m3 GEMM 8192^3 through cuBLASLt, measured in this run"
    if not peak:
        peak, src = 2.0 * peaks["bf16_tflops"], "2 x MEASURED_PEAKS.json bf16 burst (the 8-bit GEMM probe failed)"
    mhz = (clocks or {}).get("sm_mhz") or 1965.0
    mufu = EX2_PER_CLK_PER_SM * SM_COUNT * mhz * 1e6 * 4.0 * w["d"] / 1e12
    return {
        "bound": "tensor", "kernel": kernel, "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
        "peak_source": src, "peak_fp8_measured": fp8_peak, "peak_int8_measured": int8_peak,
        "peak_bf16_measured": peaks["bf16_tflops"], "frac_bf16_measured": achieved / peaks["bf16_tflops"],
        "peak_fp8_nominal": 4500.0, "frac_fp8_nominal": achieved / 4500.0,
        "mufu_bound_tflops": mufu, "frac_mufu_bound": achieved / mufu,
        "mufu_bound_note": "one ex2 per attended pair at %d results/clk/SM x %d SMs x %.0f MHz, 4*D flops per pair" % (
            EX2_PER_CLK_PER_SM, SM_COUNT, mhz),
        "ms_per_launch": ms, "algorithmic_flops_per_launch": flops, "traffic": None,
    }


# ----------------------------------------------------------------------------------------------------
# default workload: one long-context batch, strong scaling over the ranks
def run_longctx(args, name, w, rank, world, local_rank, quick=False):
    import torch
    import torch.distributed as dist
    from tscale_b200 import ops, shard

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    frags, seq, heads, d = w["frags"], w["seq"], w["heads"], w["d"]
    hd = heads * d
    window, slope = w["layers"][0]
    rects = shard.rank_rects(frags, heads, world, rank)
    assert len(rects) == 1, "the bench shards %d units over %d ranks into one rectangle per rank" % (frags * heads, world)
    f0, f1, h0, h1 = rects[0]
    nf, nh = f1 - f0, h1 - h0
    rows = nf * seq
    # Head slices of the rank's rectangle.  With NCCL (or the copy kernel) four equal ones, so that the gather of a slice runs
    # under the next slice's kernel (slices shrinking towards the end, so that the last all-gather is small, were measured at
    # N = 2: the exposed gather time stayed at 0.5 ms, it is not the last slice's gather that shows).  One GPU, or the gather
    # fused into the kernel: one launch for the whole rectangle, since every launch ends in a tail of long work items.
    gather_mode = ("fused" if args.gather == "auto" else args.gather) if world > 1 else "none"
    k_slices = args.slices if args.slices > 0 else (1 if gather_mode in ("none", "fused") else 4)
    widths = [nh // k_slices] * k_slices if nh % k_slices == 0 else [nh]
    n_slices = len(widths)
    starts = [sum(widths[:i]) for i in range(n_slices)]
    cfg = ops.make_cfg(w["qk"], w["v"], d, d, out_dtype=torch.bfloat16)
    mask = ops.Mask.window([seq] * nf, window)
    mask.dev(dev)

    # the rank's fragments at full width: the same bytes whatever the number of ranks (seeded per fragment and tensor)
    gen = torch.Generator(device=dev)
    t = {}
    for idx, (nm, dt) in enumerate((("q", w["qk"]), ("k", w["qk"]), ("v", w["v"]))):
        t[nm] = torch.empty((rows, hd), dtype=torch.uint8, device=dev)
        t["s" + nm] = torch.empty((heads, rows), dtype=torch.float32, device=dev)
        for f in range(f0, f1):
            gen.manual_seed(w["seed"] * 100000 + f * 10 + idx)
            x = torch.randn((seq, hd), generator=gen, device=dev, dtype=torch.float32) * 0.5
            b, s = ops.quant_rows(x, "absmax", dt, d)
            t[nm][(f - f0) * seq:(f - f0 + 1) * seq] = b
            t["s" + nm][:, (f - f0) * seq:(f - f0 + 1) * seq] = s
            del x, b, s
    # Several ranks: the gathered output lives in symmetric memory (every rank's buffer mapped into every process), so that
    # the attention kernel can store its rows straight into the peers' copies (tsa_att_fwd_to: the all-gather fused into the
    # epilogue, plain peer stores over NVLink, no multicast).  --gather nccl, or a torch without symmetric memory, keeps the
    # per-slice NCCL all-gather.
    fused, scatter, symm_handle, peer_out, side = False, False, None, None, None
    if world > 1:
        # measured: fused is ahead at every N (four launches per step, two GPUs: 15.16 against 15.53 ms with NCCL; eight: 4.45
        # against 4.94 ms; as one launch per step 4.19 ms on eight)
        mode = gather_mode
        if mode in ("fused", "scatter"):
            try:
                assert len(set(widths)) == 1
                symm_handle = shard.FusedGather(n_slices, rows, widths[0] * d, torch.bfloat16, dev)
                gathered = [symm_handle.gathered(s) for s in range(n_slices)]
                peer_out = [symm_handle.peers(s) for s in range(n_slices)]
                fused = mode == "fused"
                scatter = mode == "scatter"
                side = torch.cuda.Stream(device=dev)
            except Exception as exc:  # noqa: BLE001 - any failure of the symmetric-memory set-up falls back to NCCL
                sys.stderr.write("symmetric memory unavailable (%s): gathering with NCCL\n" % (exc,))
            # every rank takes the same route: one rank without symmetric memory sends all of them to NCCL
            agreed = torch.tensor([1 if (fused or scatter) else 0], dtype=torch.int32, device=dev)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
            if int(agreed.item()) == 0:
                fused, scatter, symm_handle, peer_out = False, False, None, None
                if args.slices <= 0 and nh % 4 == 0:
                    widths = [nh // 4] * 4  # NCCL gathers overlap the following slices' kernels
                    n_slices = len(widths)
                    starts = [sum(widths[:i]) for i in range(n_slices)]
        if fused or scatter:
            # a rank's own block sits inside its gathered buffer: the kernel writes it there
            out_local = [gathered[s][rank] for s in range(n_slices)]
        else:
            gathered = [torch.empty((world, rows, wd * d), dtype=torch.bfloat16, device=dev) for wd in widths]
            out_local = [torch.empty((rows, wd * d), dtype=torch.bfloat16, device=dev) for wd in widths]
    else:
        gathered = None
        out_local = [torch.empty((rows, wd * d), dtype=torch.bfloat16, device=dev) for wd in widths]
    lse = torch.empty((heads, rows), dtype=torch.float32, device=dev)
    workspace = torch.empty(1 << 16, dtype=torch.uint8, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    launches = [0]

    def launch_slice(s, src=None, peers=False):
        src = t if src is None else src
        ha, hs = h0 + starts[s], widths[s]
        cols = slice(ha * d, (ha + hs) * d)
        ops.att_fwd(cfg, src["q"][:, cols], src["k"][:, cols], src["v"][:, cols], src["sk"][ha:ha + hs], mask, slope, hs,
                    qk_scale=src["sq"][ha:ha + hs], v_scale=src["sv"][ha:ha + hs], out=out_local[s], lse=lse[ha:ha + hs],
                    workspace=workspace, status=status, out_copies=peer_out[s] if peers else None)
        launches[0] += 2  # per-head V-scale maximum + attention kernel

    def step(gather=True, events=None):
        pending = []
        for s in range(n_slices):
            if events is not None:
                e0 = torch.cuda.Event(enable_timing=True)
                e0.record()
            launch_slice(s, peers=gather and fused)
            if events is not None:
                e1 = torch.cuda.Event(enable_timing=True)
                e1.record()
                events.append((e0, e1))
            if gather and scatter:
                # the library's copy kernel pushes this slice's block to the peers on a side stream, under the next slice's attention
                done = torch.cuda.Event()
                done.record()
                side.wait_event(done)
                symm_handle.scatter(s, stream=side)
            elif gather and world > 1 and not fused:
                # NCCL runs the gather on its own stream behind this slice's kernel: the next slice's kernel overlaps it
                pending.append(shard.gather_blocks(out_local[s], gathered[s], async_op=True))
        for h in pending:
            h.wait()
        if gather and (fused or scatter):
            if scatter:
                torch.cuda.current_stream().wait_stream(side)
            # every rank's blocks are in every buffer once all ranks are past this stream-ordered barrier
            symm_handle.barrier()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        barrier()
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record()
        barrier()
        tt = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item()) / n

    for _ in range(args.warmup):
        step()
    barrier()
    assert int(status.item()) == 0, "device status %#x during warm-up" % int(status.item())

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    launches[0] = 0
    kernel_events = []
    ms_step = timed(lambda: step(True, kernel_events), args.steps)
    timed_launches = launches[0]
    clocks = sampler.stop() if rank == 0 else None
    assert int(status.item()) == 0, "device status %#x in the timed region" % int(status.item())
    flops = layer_flops(w, window)
    value = flops / (ms_step * 1e-3) / 1e12
    # the rank's kernel time per step (sum over its slices), max over ranks
    k_ms = sum(a.elapsed_time(b) for a, b in kernel_events) / args.steps
    kt = torch.tensor([k_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(kt, op=dist.ReduceOp.MAX)
    k_ms = float(kt.item())

    gather = None
    if world > 1:
        n_probe = max(3, min(args.steps, 10))
        compute_ms = timed(lambda: step(False), n_probe)

        def only_gather():
            hs_ = [shard.gather_blocks(out_local[s], gathered[s], async_op=True) for s in range(n_slices)]
            for h in hs_:
                h.wait()
        gather_ms = timed(only_gather, n_probe)
        gather = {"gather_ms": gather_ms, "gather_exposed_ms": max(0.0, ms_step - compute_ms), "compute_only_ms": compute_ms,
                  "gather_bytes": (world - 1) * rows * nh * d * 2, "slices": n_slices, "slice_heads": widths,
                  "gather_note": "gather_ms: the step's NCCL all-gathers alone, back to back; gather_exposed_ms: step time minus the same "
                                 "step without any gather; gather_bytes: bytes this rank receives per step"}
        if fused or scatter:
            def nccl_step():
                pend = []
                for s in range(n_slices):
                    launch_slice(s)
                    pend.append(shard.gather_blocks(out_local[s], gathered[s], async_op=True))
                for h in pend:
                    h.wait()
            gather["mode"] = ("fused: tsa_att_fwd_to stores every output row into all ranks' buffers (symmetric memory, peer stores over "
                              "NVLink) from the attention epilogue; one stream-ordered cross-rank barrier per step") if fused else (
                              "scatter: the library's copy kernel (tsa_peer_scatter, peer stores over NVLink into symmetric memory) pushes each "
                              "slice's block to the other ranks on a side stream under the next slice's attention; one cross-rank barrier per step")
            if n_slices > 1:
                # the same slices with an NCCL all-gather behind each (with one slice nothing would overlap: run --gather nccl)
                gather["nccl_variant_ms_per_step"] = timed(nccl_step, n_probe)
        else:
            gather["mode"] = "per-slice NCCL all-gather behind each slice's kernel"

    # per-unit integer checksums of the whole batch's output as this rank holds it after the gather
    table = torch.zeros((frags, heads), dtype=torch.int64, device=dev)
    for r in range(world):
        (g0, g1, k0, k1), = shard.rank_rects(frags, heads, world, r)
        for s in range(n_slices):
            blk = gathered[s][r] if world > 1 else out_local[s]
            table[g0:g1, k0 + starts[s]:k0 + starts[s] + widths[s]] = shard.unit_checksums(blk, g1 - g0, seq, widths[s], d)
    weights = torch.arange(1, frags * heads + 1, dtype=torch.int64, device=dev).view(frags, heads)
    check = int(((table * weights).sum() % (1 << 61)).item())
    same = True
    if world > 1:
        lo = torch.tensor([check], dtype=torch.int64, device=dev)
        hi = lo.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        same = int(lo.item()) == int(hi.item())

    e2e = None
    if not args.no_e2e and not quick:
        e2e = longctx_e2e(torch, dist, shard, ops, args, cfg, mask, slope, t, out_local, starts, widths, h0, nh, d, world, dev, flops, status)

    if rank != 0:
        return None
    ref_gpu = None
    if world == 1 and not quick:
        ref_gpu = reference_gpu_kernel(torch, ops, w, t, mask, seq, d, cfg, workspace, status)
    achieved = (flops / world) / (k_ms * 1e-3) / 1e12
    roofline = tensor_roofline(torch, dev, w, "FwdSm100Kernel<128> (full causal, e4m3 QK^T and PV), this rank's %d (fragment, head) units" % (nf * nh),
                               achieved, k_ms, flops / world, clocks)
    roofline["timed"] = ("CUDA events around each slice's tsa_att_fwd call in the timed region (V-scale maximum kernel of a few "
                         "microseconds + the attention kernel), summed per step")
    # DRAM bytes per step (this rank's launches together, like ms_per_launch): the committed ncu capture of one launch over 8
    # (fragment, head) units of this workload (profiles/fwd_sm100_e4m3_d128_longctx_1frag.md: 188.7 MB read + 39.2 MB written,
    # against 171 MB of inputs and output), scaled by the units this rank processes; traffic grows in proportion to the units
    roofline["traffic"] = (188.742144e6 + 39.153152e6) * (nf * nh) / 8.0
    roofline["traffic_unit"] = "bytes per step"
    roofline["traffic_source"] = ("dram__bytes_read.sum + dram__bytes_write.sum of the committed ncu capture of one 8-unit launch, scaled to this "
                                  "rank's %d units; the kernel is not DRAM-bound (1.3 %% of the DRAM peak)" % (nf * nh))
    roofline["algorithmic_bytes"] = float(nf * nh) * seq * d * (3 + 2) + 3.0 * nf * nh * seq * 4
    line = {
        "metric": "attention_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "e4m3", "data": "synthetic", "config": workload_config(name, w, strong=True),
        "clocks": clocks, "e2e": e2e, "gpu_launches": timed_launches, "roofline": roofline,
        "gather_check": {"hash": check, "identical_on_all_ranks": same, "units": frags * heads,
                         "what": "sum over (fragment, head) units of (unit index + 1) x the integer sum of the unit's bf16 bit patterns, "
                                 "mod 2^61, over the gathered output; the same number at every N"},
    }
    if gather:
        line.update(gather)
    if ref_gpu:
        line["reference_gpu_kernel"] = ref_gpu
    return line


def reference_gpu_kernel(torch, ops, w, t, mask, seq, d, cfg, workspace, status, n_heads=8):
    """The reference's own GPU kernel Fp8Att (mma.sync e4m3, rebuilt for sm_100a behind oracle/ref_gpu_harness.cu) timed on
    this GPU on one fragment x n_heads heads of the workload, beside this library's kernel on the same slice.  The
    reference kernel takes a constant query scale and a transposed V; same shapes, spans and key scales."""
    from oracle import oracle as O
    if O.ref_gpu() is None or d != 128:
        return None
    dev = t["q"].device
    rows = seq
    cols = slice(0, n_heads * d)
    q = t["q"][:rows, cols].contiguous()
    k = t["k"][:rows, cols].contiguous()
    v = t["v"][:rows, cols].contiguous()
    sk = t["sk"][:n_heads, :rows].contiguous()
    sq = t["sq"][:n_heads, :rows].contiguous()
    sv = t["sv"][:n_heads, :rows].contiguous()
    v_tr = v.t().contiguous()
    m1 = ops.Mask.window([seq], w["layers"][0][0])
    groups, gptr, _, _ = m1.dev(dev)
    out_ref = torch.empty((rows, n_heads * d), dtype=torch.float16, device=dev)
    swl = torch.empty((n_heads, rows), dtype=torch.float32, device=dev)
    one = torch.ones(1, dtype=torch.float32, device=dev)
    try:
        O.ref_gpu_fp8_att(one, q, k, sk, v_tr, groups, gptr, 0.0, out_ref, swl, n_heads, rows, reps=1)   # warm-up
        ms_ref = O.ref_gpu_fp8_att(one, q, k, sk, v_tr, groups, gptr, 0.0, out_ref, swl, n_heads, rows, reps=3)
    except RuntimeError as e:
        return {"unavailable": str(e)}
    out = torch.empty((rows, n_heads * d), dtype=torch.bfloat16, device=dev)
    lse = torch.empty((n_heads, rows), dtype=torch.float32, device=dev)

    def ours():
        ops.att_fwd(cfg, q, k, v, sk, m1, 0.0, n_heads, qk_scale=sq, v_scale=sv, out=out, lse=lse, workspace=workspace, status=status)
    for _ in range(2):
        ours()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        ours()
    e1.record()
    torch.cuda.synchronize()
    ms_ours = e0.elapsed_time(e1) / 3
    fl = 4.0 * d * pairs_window(seq, w["layers"][0][0]) * n_heads
    return {"kernel": "Fp8Att of the reference (mma.sync e4m3, 4 warps per 64 query rows), rebuilt for sm_100a",
            "shape": "1 fragment x %d tokens x %d heads x %d, full causal" % (seq, n_heads, d),
            "ms": ms_ref, "tflops": fl / (ms_ref * 1e-3) / 1e12,
            "this_library_ms": ms_ours, "this_library_tflops": fl / (ms_ours * 1e-3) / 1e12,
            "speedup": ms_ref / ms_ours}


def longctx_e2e(torch, dist, shard, ops, args, cfg, mask, slope, t, out_local, starts, widths, h0, nh, d, world, dev, flops, status):
    """The same step through the library's host-buffer entry (tsa_att_fwd_host): the rank's vectors start in pinned host
    memory every step and its output block ends there; the library copies head slices in, computes and copies out
    concurrently.  With several ranks the result is also kept on the device and all-gathered.  Copies, kernels and the
    gather are inside the timed region."""
    cols = slice(h0 * d, (h0 + nh) * d)
    pin = lambda x: x.contiguous().cpu().pin_memory()
    hq, hk, hv = pin(t["q"][:, cols]), pin(t["k"][:, cols]), pin(t["v"][:, cols])
    hsq, hsk, hsv = pin(t["sq"][h0:h0 + nh]), pin(t["sk"][h0:h0 + nh]), pin(t["sv"][h0:h0 + nh])
    rows = hq.shape[0]
    host_out = torch.empty((rows, nh * d), dtype=torch.bfloat16).pin_memory()
    out_dev = torch.empty((rows, nh * d), dtype=torch.bfloat16, device=dev) if world > 1 else None
    gathered = torch.empty((world, rows, nh * d), dtype=torch.bfloat16, device=dev) if world > 1 else None
    slices = next(k for k in (16, 8, 4, 2, 1) if nh % k == 0 and (nh // k >= 2 or k == 1))
    h2d_bytes = sum(v.numel() * v.element_size() for v in (hq, hk, hv, hsq, hsk, hsv))
    d2h_bytes = host_out.numel() * host_out.element_size()
    box = [None]

    def step():
        box[0] = ops.att_fwd_host(cfg, hq, hk, hv, hsk, mask, slope, nh, host_out, qk_scale=hsq, v_scale=hsv, slices=slices,
                                  staging=box[0], status=status, device=dev, out_device=out_dev)
        if world > 1:
            shard.gather_blocks(out_dev, gathered)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    steps = max(2, min(args.steps, 4))
    step()
    barrier()
    # the host copy carries the bits of the device-resident run
    same = all(bool(torch.equal(host_out[:, starts[s] * d:(starts[s] + widths[s]) * d], out_local[s].cpu())) for s in range(len(out_local)))
    a = torch.cuda.Event(enable_timing=True)
    b = torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        step()
    b.record()
    barrier()
    assert int(status.item()) == 0, "device status %#x in the end-to-end run" % int(status.item())
    tt = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    ms = float(tt.item()) / steps
    return {"value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d_bytes,
            "d2h_bytes_per_step": d2h_bytes, "ms_per_step": ms, "steps": steps, "entry": "tsa_att_fwd_host", "slices": slices,
            "matches_device_run": same,
            "note": "bytes are this rank's: every rank copies its own shard in and its own output block out; head slices are "
                    "copied in, computed and copied out concurrently by the library"}


# ----------------------------------------------------------------------------------------------------
# layer-mix workloads (prefill125m, train15b): per-GPU work fixed
def run_layers(args, name, w, rank, world, local_rank, quick=False):
    import torch
    import torch.distributed as dist
    from tscale_b200 import ops

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    frag_lens = [w["seq"]] * w["frags"]
    length = sum(frag_lens)
    heads, d = w["heads"], w["d"]
    hd = heads * d
    masks = {}
    for window, _ in w["layers"]:
        if window not in masks:
            masks[window] = ops.Mask.window(frag_lens, window)
            masks[window].dev(dev)
    grad_dtype = torch.bfloat16
    cfg = ops.make_cfg(w["qk"], w["v"], d, d, out_dtype=torch.bfloat16, grad_dtype=grad_dtype)

    # inputs: one Q/K/V set per layer (each rank its own fragments: seed offset by rank)
    gen = torch.Generator(device=dev)
    layers = []
    for idx, (window, slope) in enumerate(w["layers"]):
        gen.manual_seed(w["seed"] * 1000 + idx + 100000 * rank)
        item = {"window": window, "slope": slope}
        for nm, dt in (("q", w["qk"]), ("k", w["qk"]), ("v", w["v"])):
            x = torch.randn((length, hd), generator=gen, device=dev, dtype=torch.float32) * 0.5
            item[nm], item["s" + nm] = ops.quant_rows(x, "absmax", dt, d)
            del x
        item["out"] = torch.empty((length, hd), dtype=torch.bfloat16, device=dev)
        item["lse"] = torch.empty((heads, length), dtype=torch.float32, device=dev)
        if w["bwd"]:
            item["d_out"] = (torch.randn((length, hd), generator=gen, device=dev, dtype=torch.float32) * 1e-2).to(grad_dtype)
        layers.append(item)
    workspace = torch.empty(1 << 20, dtype=torch.uint8, device=dev)
    bwd_ws = None
    if w["bwd"]:
        import ctypes
        from tscale_b200 import abi
        bwd_ws = torch.empty(max(1, abi.lib().tsa_att_bwd_workspace_bytes(ctypes.byref(cfg), heads, length)), dtype=torch.uint8, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)

    launches = [0]
    dom = max(range(len(layers)), key=lambda i: layer_flops(w, layers[i]["window"]))  # dominant layer
    layer_events = [[] for _ in layers]

    def run_layer(i, item, record):
        if record:
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record()
        ops.att_fwd(cfg, item["q"], item["k"], item["v"], item["sk"], masks[item["window"]], item["slope"], heads,
                    qk_scale=item["sq"], v_scale=item["sv"], out=item["out"], lse=item["lse"], workspace=workspace, status=status)
        launches[0] += 2  # per-head V-scale maximum + attention kernel
        if record:
            e1.record()
            layer_events[i].append((e0, e1))
        if w["bwd"]:
            ops.att_bwd(cfg, item["q"], item["k"], item["v"], item["sk"], item["d_out"], item["out"], item["lse"],
                        masks[item["window"]], item["slope"], heads, qk_scale=item["sq"], v_scale=item["sv"], workspace=bwd_ws,
                        status=status)
            launches[0] += 4  # dScale, bf16 widening of Q, K and V (one launch), dQ kernel, dK/dV kernel

    def step(record=False):
        for i, item in enumerate(layers):
            run_layer(i, item, record)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    assert int(status.item()) == 0, "device status %#x during warm-up" % int(status.item())

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    launches[0] = 0
    barrier()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        step(True)
    t1.record()
    barrier()
    ms_total = t0.elapsed_time(t1)
    clocks = sampler.stop() if rank == 0 else None
    assert int(status.item()) == 0, "device status %#x in the timed region" % int(status.item())
    tt = torch.tensor([ms_total], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    ms_step = float(tt.item()) / args.steps
    fl_step = sum(layer_flops(w, it["window"]) for it in layers) * (3.5 if w["bwd"] else 1.0)  # bwd = 10*D*pairs (5 GEMMs)
    value = fl_step * world / (ms_step * 1e-3) / 1e12

    dom_ms = float(np.mean([a.elapsed_time(b) for a, b in layer_events[dom]]))
    dom_flops = layer_flops(w, layers[dom]["window"])

    e2e = None
    if not args.no_e2e and not quick:
        e2e = layers_e2e(torch, ops, args, w, cfg, layers, masks, heads, workspace, bwd_ws, status, world, dist, fl_step)

    if rank != 0:
        return None
    achieved = dom_flops / (dom_ms * 1e-3) / 1e12
    roofline = tensor_roofline(torch, dev, w, "FwdSm100Kernel<%d> (full-causal layer, %s QK^T, e4m3 PV)" % (d, w["qk"]),
                               achieved, dom_ms, dom_flops, clocks)
    roofline["timed"] = "CUDA events around the layer's tsa_att_fwd call (V-scale maximum kernel of a few microseconds + the attention kernel)"
    per_layer = []
    for i, it in enumerate(layers):
        ms = float(np.mean([a.elapsed_time(b) for a, b in layer_events[i]]))
        per_layer.append({"window": "full" if it["window"] <= 0 else it["window"], "alibi_slope": it["slope"], "fwd_ms": ms,
                          "fwd_tflops": layer_flops(w, it["window"]) / (ms * 1e-3) / 1e12})
    line = {
        "metric": "attention_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "e4m3" if w["qk"] == "e4m3" else "i8+e4m3", "data": "synthetic", "config": workload_config(name, w),
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches[0], "roofline": roofline, "layers": per_layer,
    }
    if w["bwd"]:
        line["flop_counting"] = ("forward 4*D per attended pair + backward 10*D (5 GEMMs); the reference's own count credits the "
                                 "backward with 7 GEMMs (14*D)")
    return line


def layers_e2e(torch, ops, args, w, cfg, layers, masks, heads, workspace, bwd_ws, status, world, dist, fl_step):
    """Same step through the public call with HOST buffers: every step copies the layer inputs (and dOut for the
    training workload) from pinned host memory to the device, runs the layer, and copies the bf16 result (forward:
    out; training: dQ, dK, dV) back to pinned host memory."""
    dev = layers[0]["q"].device
    names = ("q", "k", "v", "sq", "sk", "sv") + (("d_out",) if w["bwd"] else ())
    host_in = [{n: it[n].cpu().pin_memory() for n in names} for it in layers]
    n_out = 3 if w["bwd"] else 1
    host_out = [[torch.empty(it["out"].shape, dtype=it["out"].dtype).pin_memory() for _ in range(n_out)] for it in layers]
    stage = [{n: torch.empty_like(layers[0][n]) for n in names} for _ in range(2)]
    out_stage = [torch.empty_like(layers[0]["out"]) for _ in range(2)]
    grad_stage = [None, None]
    lse = layers[0]["lse"]
    h2d = torch.cuda.Stream(device=dev)
    d2h = torch.cuda.Stream(device=dev)
    main_s = torch.cuda.current_stream()
    h2d_bytes = sum(sum(t.numel() * t.element_size() for t in hi.values()) for hi in host_in)
    d2h_bytes = sum(sum(t.numel() * t.element_size() for t in ho) for ho in host_out)

    def step():
        free_in = [None, None]
        free_out = [None, None]
        for i, it in enumerate(layers):
            sl = i % 2
            with torch.cuda.stream(h2d):
                if free_in[sl] is not None:
                    h2d.wait_event(free_in[sl])
                for n in names:
                    stage[sl][n].copy_(host_in[i][n], non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(h2d)
            main_s.wait_event(ready)
            if free_out[sl] is not None:
                main_s.wait_event(free_out[sl])
            s = stage[sl]
            ops.att_fwd(cfg, s["q"], s["k"], s["v"], s["sk"], masks[it["window"]], it["slope"], heads, qk_scale=s["sq"],
                        v_scale=s["sv"], out=out_stage[sl], lse=lse, workspace=workspace, status=status)
            results = [out_stage[sl]]
            if w["bwd"]:
                grad_stage[sl] = ops.att_bwd(cfg, s["q"], s["k"], s["v"], s["sk"], s["d_out"], out_stage[sl], lse, masks[it["window"]],
                                             it["slope"], heads, qk_scale=s["sq"], v_scale=s["sv"], workspace=bwd_ws, status=status)
                results = list(grad_stage[sl])
            done = torch.cuda.Event()
            done.record(main_s)
            free_in[sl] = done
            with torch.cuda.stream(d2h):
                d2h.wait_event(done)
                for dst, src in zip(host_out[i], results):
                    dst.copy_(src, non_blocking=True)
                    src.record_stream(d2h)
                fo = torch.cuda.Event()
                fo.record(d2h)
            free_out[sl] = fo
        main_s.wait_stream(d2h)
        main_s.wait_stream(h2d)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    steps = max(2, min(args.steps, 5))
    step()
    barrier()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        step()
    t1.record()
    barrier()
    tt = torch.tensor([t0.elapsed_time(t1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    ms = float(tt.item()) / steps
    return {"value": fl_step * world / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d_bytes,
            "d2h_bytes_per_step": d2h_bytes, "ms_per_step": ms, "steps": steps}


# ----------------------------------------------------------------------------------------------------
def short(line):
    """What an `also` entry keeps of a workload's line."""
    keys = ("metric", "value", "unit", "ms_per_step", "steps", "warmup", "dtype", "scaling", "config", "roofline", "layers",
            "gpu_launches", "flop_counting")
    return {k: line[k] for k in keys if k in line}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="longctx", choices=sorted(WORKLOADS) + ["decode", "infer", "neighbours"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-also", action="store_true", help="skip the short runs of the other workloads")
    ap.add_argument("--gather", default="auto", choices=["auto", "fused", "scatter", "nccl"],
                    help="several GPUs: how every rank gets the whole output: 'fused' = the attention kernel stores its rows into every rank's "
                         "buffer itself, 'scatter' = the library's copy kernel pushes each slice's block to the peers under the next slice's "
                         "attention, 'nccl' = per-slice NCCL all-gathers; 'auto' = fused")
    ap.add_argument("--slices", type=int, default=0,
                    help="head slices (launches) per step of the default workload; 0 = one, or four when the gather is not fused")
    ap.add_argument("--frags", type=int, default=0, help="override the number of fragments (profiling on a small case)")
    ap.add_argument("--heads", type=int, default=0, help="override the number of heads (profiling on a small case)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.workload == "decode":
        from benchlib import decode
        return decode.run(args, rank, world, local_rank)
    if args.workload == "infer":
        from benchlib import infer
        return infer.run(args, rank, world, local_rank)
    if args.workload == "neighbours":
        from benchlib import neighbours
        return neighbours.run(args, rank, world, local_rank)

    name = args.workload
    w = dict(WORKLOADS[name])
    if args.frags > 0:
        w["frags"] = args.frags
    if args.heads > 0:
        w["heads"] = args.heads
    if args.impl == "reference":
        return reference_arm(args, name, w, rank)

    runner = run_longctx if name == "longctx" else run_layers
    line = runner(args, name, w, rank, world, local_rank)
    if rank == 0:
        line["cpu_baseline"] = cpu_baseline_block(w) if (world == 1 and not args.no_cpu_baseline) else None
        if world == 1 and name == "longctx" and not args.no_also:
            # the other workloads of the path, short runs, so that one record carries their numbers too
            import copy
            import torch
            quick = copy.copy(args)
            quick.steps, quick.warmup = 5, 3
            also = []
            for other in ("prefill125m", "train15b"):
                torch.cuda.empty_cache()
                also.append(short(run_layers(quick, other, dict(WORKLOADS[other]), 0, 1, local_rank, quick=True)))
            from benchlib import decode
            torch.cuda.empty_cache()
            quick.steps = 20
            also.append(short(decode.run(quick, 0, 1, local_rank, emit=False, quick=True)))
            line["also"] = also
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
