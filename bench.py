#!/usr/bin/env python
"""Benchmark of the quantized attention path on B200.

    python bench.py --gpus N --steps K --warmup W [--workload prefill125m|train15b|decode|longctx|infer|neighbours] [--impl reference]

Default workload `prefill125m` is the 125M-style prefill forward: 16 fragments x 4096 tokens, 12 heads x 64,
e4m3 Q/K/V with per-row f32 scales, bf16 output; one step = 3 window-64 layers (ALiBi slope 0.5) + 1 full
causal layer.  Inputs are seeded synthetic N(0,1)*0.5, quantised on the GPU by the library's abs-max
quantiser.  The metric is algorithmic attention TFLOP/s: 4 * D * (attended pairs) per (fragment, head),
masked-out work inside partially filled tiles not counted.

One process per GPU.  With N > 1 every rank runs the same per-GPU workload on its own fragments (the path
shards by fragment x head with no exchange step), so scaling is weak and `value` is the sum over ranks
divided by the slowest rank's time; `--gather` adds the NCCL all-gather of the bf16 outputs.

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

from tscale_b200.benchutil import ClockSampler, load_peaks  # noqa: E402


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


def layer_flops(w, window):
    return 4.0 * w["d"] * pairs_window(w["seq"], window) * w["frags"] * w["heads"]


# ----------------------------------------------------------------------------------------------------
# CPU arm
def cpu_sample_inputs(w, layer_idx, n_frags, seed):
    """A bounded sample of the workload for the CPU arm: the first n_frags fragments of one layer, generated
    with the same recipe as the GPU inputs (N(0,1)*0.5, abs-max 8-bit quantisation) through the oracle."""
    from oracle import oracle as O
    rng = np.random.default_rng(seed * 1000 + layer_idx)
    length = n_frags * w["seq"]
    hd = w["heads"] * w["d"]
    res = []
    for name, dt in (("q", w["qk"]), ("k", w["qk"]), ("v", w["v"])):
        x = (rng.standard_normal((length, hd)) * 0.5).astype(np.float32)
        b, s = O.quant_rows("absmax", dt, 0.0, x, w["d"])
        deq = (O.dequant(b, dt).reshape(length, w["heads"], w["d"]) * s.T[:, :, None]).reshape(length, hd)
        res.append(np.ascontiguousarray(deq, dtype=np.float32))
    return res


def run_cpu_sample(w, sample, threads):
    """Runs the reference's CPU forward on the sample; returns (seconds, flops, kind)."""
    from concurrent.futures import ThreadPoolExecutor
    from oracle import oracle as O
    use_ref = O.ref() is not None
    kind = "reference" if use_ref else "port"
    O.set_threads(1)
    jobs = []
    flops = 0.0
    for (window, slope, n_frags, q, k, v) in sample:
        spans, ptr = O.window_spans([w["seq"]], window)
        for f in range(n_frags):
            rows = slice(f * w["seq"], (f + 1) * w["seq"])
            for h in range(w["heads"]):
                cols = slice(h * w["d"], (h + 1) * w["d"])
                jobs.append((np.ascontiguousarray(q[rows, cols]), np.ascontiguousarray(k[rows, cols]),
                             np.ascontiguousarray(v[rows, cols]), spans, ptr, slope))
        flops += 4.0 * w["d"] * pairs_window(w["seq"], window) * n_frags * w["heads"]

    def one(job):
        q1, k1, v1, spans, ptr, slope = job
        O.att_fwd(q1, k1, v1, spans, ptr, 1, slope, use_ref=use_ref)

    t0 = time.perf_counter()
    with ThreadPoolExecutor(max_workers=threads) as ex:
        list(ex.map(one, jobs))
    return time.perf_counter() - t0, flops, kind


def make_cpu_sample(w):
    # about 10-20 s of host work: one fragment of a window layer and one of the widest layer, all heads
    sample = []
    done = set()
    for idx, (window, slope) in enumerate(w["layers"]):
        if (window, slope) in done:
            continue
        done.add((window, slope))
        q, k, v = cpu_sample_inputs(w, idx, 1, w["seed"])
        sample.append((window, slope, 1, q, k, v))
    return sample


def sample_text(w, sample):
    return "; ".join("%d fragment(s) x %d tokens x %d heads, window %s, slope %g" %
                     (n, w["seq"], w["heads"], "full" if win <= 0 else win, sl) for (win, sl, n, _, _, _) in sample)


# ----------------------------------------------------------------------------------------------------
def reference_arm(args, w, rank):
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
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, w),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": kind, "sample": sample_text(w, sample)},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def workload_config(args, w):
    return {"workload": args.workload, "fragments": w["frags"], "seq_len": w["seq"], "heads": w["heads"], "head_dim": w["d"],
            "qk_dtype": w["qk"], "v_dtype": w["v"], "layers": [{"window": "full" if win <= 0 else win, "alibi_slope": sl} for win, sl in w["layers"]],
            "backward": w["bwd"], "l2": "inputs larger than L2 (each layer has its own Q/K/V set)", "sharding": "fragment x head, per-GPU work fixed"}


# ----------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="prefill125m", choices=sorted(WORKLOADS) + ["decode", "infer", "neighbours"])
    ap.add_argument("--gather", action="store_true", help="all-gather the bf16 outputs over NCCL inside the timed region")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--frags", type=int, default=0, help="override the number of fragments (profiling on a small case)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.workload == "decode":
        from tscale_b200 import bench_decode
        return bench_decode.run(args, rank, world, local_rank)
    if args.workload == "infer":
        from tscale_b200 import bench_infer
        return bench_infer.run(args, rank, world, local_rank)
    if args.workload == "neighbours":
        from tscale_b200 import bench_neighbours
        return bench_neighbours.run(args, rank, world, local_rank)

    w = dict(WORKLOADS[args.workload])
    if args.frags > 0:
        w["frags"] = args.frags
    if args.impl == "reference":
        return reference_arm(args, w, rank)

    import torch
    import torch.distributed as dist
    from tscale_b200 import ops

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
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
        for name, dt in (("q", w["qk"]), ("k", w["qk"]), ("v", w["v"])):
            x = torch.randn((length, hd), generator=gen, device=dev, dtype=torch.float32) * 0.5
            item[name], item["s" + name] = ops.quant_rows(x, "absmax", dt, d)
            del x
        item["out"] = torch.empty((length, hd), dtype=torch.bfloat16, device=dev)
        item["lse"] = torch.empty((heads, length), dtype=torch.float32, device=dev)
        if w["bwd"]:
            item["d_out"] = (torch.randn((length, hd), generator=gen, device=dev, dtype=torch.float32) * 1e-2).to(grad_dtype)
        layers.append(item)
    workspace = torch.empty(1 << 20, dtype=torch.uint8, device=dev)
    bwd_ws = None
    if w["bwd"]:
        from tscale_b200 import abi
        import ctypes
        bwd_ws = torch.empty(max(1, abi.lib().tsa_att_bwd_workspace_bytes(ctypes.byref(cfg), heads, length)), dtype=torch.uint8, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    gathered = None
    pending = []
    if args.gather and world > 1:
        gathered = [torch.empty((world, length, hd), dtype=torch.bfloat16, device=dev) for _ in layers]

    launches = [0]
    dom = max(range(len(layers)), key=lambda i: layer_flops(w, layers[i]["window"]))  # dominant layer
    dom_events = []

    def run_layer(item, record=None):
        if record is not None:
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record()
        ops.att_fwd(cfg, item["q"], item["k"], item["v"], item["sk"], masks[item["window"]], item["slope"], heads,
                    qk_scale=item["sq"], v_scale=item["sv"], out=item["out"], lse=item["lse"], workspace=workspace, status=status)
        launches[0] += 2  # per-head V-scale maximum + attention kernel
        if record is not None:
            e1.record()
            record.append((e0, e1))
        if w["bwd"]:
            ops.att_bwd(cfg, item["q"], item["k"], item["v"], item["sk"], item["d_out"], item["out"], item["lse"],
                        masks[item["window"]], item["slope"], heads, qk_scale=item["sq"], v_scale=item["sv"], workspace=bwd_ws,
                        status=status)
            launches[0] += 6  # dScale, bf16 widening of Q / K / V, dQ kernel, dK/dV kernel
        if gathered is not None:
            # NCCL runs the gather on its own stream: the next layer's kernels overlap with it
            pending.append(dist.all_gather_into_tensor(gathered[len(pending) % len(gathered)].view(-1), item["out"].view(-1), async_op=True))

    def step(record=None):
        for i, item in enumerate(layers):
            run_layer(item, record if i == dom else None)
        while pending:
            pending.pop().wait()

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
        step(dom_events)
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

    dom_ms = float(np.mean([a.elapsed_time(b) for a, b in dom_events]))
    dom_flops = layer_flops(w, layers[dom]["window"])

    # ---- end to end: host buffers in, host buffers out, copies inside the timed region
    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(torch, ops, args, w, cfg, layers, masks, heads, workspace, bwd_ws, status, world, dist, fl_step)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = load_peaks()
    fp8_peak = measure_fp8_peak(torch, dev)
    int8_peak = measure_int8_peak(torch, dev)
    achieved = dom_flops / (dom_ms * 1e-3) / 1e12
    roofline = {
        "bound": "tensor", "kernel": "FwdSm100Kernel (full-causal layer, %s QK^T, e4m3 PV)" % w["qk"],
        "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"],
        "peak_source": "MEASURED_PEAKS.json bf16 burst (%s)" % peaks["_source"],
        "peak_fp8_measured": fp8_peak, "frac_fp8_measured": (achieved / fp8_peak) if fp8_peak else None,
        "peak_fp8_nominal": 4500.0, "frac_fp8_nominal": achieved / 4500.0,
        "peak_int8_measured": int8_peak, "frac_int8_measured": (achieved / int8_peak) if int8_peak else None,
        "ms_per_launch": dom_ms, "algorithmic_flops_per_launch": dom_flops, "traffic": None,
        "timed": "CUDA events around the layer's tsa_att_fwd call (V-scale maximum kernel of a few microseconds + the attention kernel)",
    }
    if args.workload == "prefill125m":
        # ncu capture of this kernel on 2 fragments (profiles/fwd_sm100_e4m3_d64_fullcausal_2frag.md): 20.2 MB read, 0 written
        # to DRAM while the kernel runs; traffic grows with the fragment count
        roofline["traffic"] = 20.2e6 / 2 * w["frags"]
        roofline["traffic_source"] = "dram bytes of a 2-fragment ncu capture scaled by fragments; algorithmic input bytes %.1f MB" % (
            3 * w["frags"] * w["seq"] * heads * d / 1e6)
    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        sample = make_cpu_sample(w)
        threads = os.cpu_count() or 1
        # repeated until about 10 s of host work have been timed (at least 3 passes over the sample)
        total, reps = 0.0, 0
        while reps < 3 or (total < 10.0 and reps < 50):
            sec, flops, kind = run_cpu_sample(w, sample, threads)
            total += sec
            reps += 1
        sec = total / reps
        cpu_baseline = {"value": flops / sec / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": kind,
                        "sample": sample_text(w, sample) + " (forward only), %d passes" % reps, "seconds": total}
    line = {
        "metric": "attention_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "e4m3" if w["qk"] == "e4m3" else "i8+e4m3", "data": "synthetic", "config": workload_config(args, w),
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches[0], "roofline": roofline, "cpu_baseline": cpu_baseline,
    }
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def measure_fp8_peak(torch, dev):
    """Dense e4m3 GEMM rate of this GPU (cuBLASLt through torch._scaled_mm), the way the bf16 peak was measured."""
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
    """Dense int8 x int8 -> int32 GEMM rate of this GPU (cuBLASLt through torch._int_mm), in TOP/s; None if the library
    has no such kernel here."""
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
    except Exception:  # noqa: BLE001  (a peak probe must not break the benchmark)
        return None


def run_e2e(torch, ops, args, w, cfg, layers, masks, heads, workspace, bwd_ws, status, world, dist, fl_step):
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


if __name__ == "__main__":
    main()
