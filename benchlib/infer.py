"""Inference workload of bench.py (`--workload infer`): one token for each of 64 sequences through a 12-layer int8 model
with per-layer KV caches (tsa_infer_step), contexts uniform in [1024, 8192].

Model shape: dim 768, 12 heads x 64, relu 1536, vocabulary 50304; layers repeat three window-64 layers (ALiBi slope
0.5) and one wide layer like the reference's model family; random int8 weights and caches.  The metric is tokens
per second for the batch; the roofline object gives the bytes every step has to stream (the keys and values the
layers attend plus every weight once) over the step time.
"""
import json
import os
import time

import numpy as np

from .util import ClockSampler, load_peaks

N_SEQ, DIM, HEADS, D, RELU_MULT, VOCAB, LAYERS = 64, 768, 12, 64, 1, 50304, 12
CTX_LO, CTX_HI = 1024, 8192
SEED = 5


def layer_plan():
    return [(64, 0.5) if (i % 4) != 3 else (1 << 20, 0.0) for i in range(LAYERS)]


def make_model(layers):
    """Seeded random int8 model (dict of numpy arrays in the layout tsa_infer_model takes)."""
    rng = np.random.default_rng(SEED)
    hs, relu_dim = HEADS * D, HEADS * 128 * RELU_MULT

    def mat(rows, cols):
        return rng.integers(-60, 61, (rows, cols), dtype=np.int8)

    out = []
    for width, slope in layers:
        out.append(dict(qk=mat(hs, DIM), qv=mat(hs, DIM), k=mat(hs, DIM), v=mat(hs, DIM), combiner=mat(DIM, hs * 4), expand=mat(relu_dim, DIM),
                        contract=mat(DIM, relu_dim), qv_scale=1 / 32.0, combiner_scale=1 / 32.0, contract_scale=1 / 32.0, width=width, slope=slope))
    return dict(dim=DIM, head_dim=D, heads=HEADS, relu_mult=RELU_MULT, vocab=VOCAB, label_count=VOCAB + 33, layers=out,
                label_embed=mat(VOCAB + 33, DIM), label_embed_scale=1 / 32.0, final_layer=mat(VOCAB, DIM), final_layer_scale=1 / 32.0,
                bias=np.zeros(VOCAB, dtype=np.float32))


def fill_rope(width, max_len):
    """Rope table in the layout of FillRopeBuf (code/gpt/att/rope.cpp:4-24): per 64-element block 32 cosines, 32 sines."""
    k = np.arange(width // 2)
    freq = np.exp(-np.log(np.float32(500000.0)) * (k * 2.0 / width)).astype(np.float32)
    t = np.arange(max_len, dtype=np.float32)[:, None]
    table = np.zeros((max_len, width), dtype=np.float32)
    for base in range(0, width, 64):
        angle = t * freq[None, base // 2:base // 2 + 32]
        table[:, base:base + 32] = np.cos(angle)
        table[:, base + 32:base + 64] = np.sin(angle)
    return table


def weight_bytes():
    hs, relu_dim = HEADS * D, HEADS * 128 * RELU_MULT
    per_layer = 4 * hs * DIM + DIM * hs * 4 + 2 * relu_dim * DIM
    return LAYERS * per_layer + VOCAB * DIM


def kv_bytes(ctx_lens, layers):
    """Bytes of keys, values and their f32 scales the layers attend in one step (lengths after the append)."""
    total = 0
    for width, _ in layers:
        for n in ctx_lens:
            keys = min(n - 1, width)
            total += keys * HEADS * (2 * D + 8)
    return float(total)


def config():
    return {"workload": "infer", "sequences": N_SEQ, "context": "uniform[%d,%d]" % (CTX_LO, CTX_HI), "dim": DIM, "heads": HEADS, "head_dim": D,
            "relu_dim": HEADS * 128 * RELU_MULT, "vocab": VOCAB, "layers": "12: (3 x window 64 slope 0.5, 1 x wide) x 3", "weights": "i8",
            "kv_dtype": "i8", "scale_dtype": "f32", "l2": "the wide layers' caches (about 0.9 GB per step) and the weights (124 MB) exceed L2",
            "launch": "one CUDA graph per step", "sharding": "sequences, per-GPU work fixed"}


def cpu_sample(threads, n_seq_sample, ctx_len, steps):
    """The reference's own ComputePrediction (oracle/_ref, else the oracle port): n_seq_sample sequences in parallel
    threads, a short prefill of ctx_len tokens each (not timed), then `steps` timed tokens."""
    from concurrent.futures import ThreadPoolExecutor
    from oracle import oracle as O
    use_ref = O.ref() is not None
    model = make_model(layer_plan())
    ctxs = [O.InferOracle(model, ctx_len + steps + 1, use_ref=use_ref, exp_mode="poly") for _ in range(n_seq_sample)]

    def run(c, n):
        for t in range(n):
            c.step([1 + (t * 7919) % VOCAB])

    with ThreadPoolExecutor(max_workers=threads) as ex:
        list(ex.map(lambda c: run(c, ctx_len), ctxs))
        t0 = time.perf_counter()
        list(ex.map(lambda c: run(c, steps), ctxs))
        sec = time.perf_counter() - t0
    return n_seq_sample * steps / sec, "reference" if use_ref else "port", \
        "%d sequences in parallel, %d timed tokens each after a %d-token context (the GPU workload's contexts average 4608)" % (
            n_seq_sample, steps, ctx_len), sec


def run(args, rank, world, local_rank):
    if args.impl == "reference":
        if rank != 0:
            return
        threads = os.cpu_count() or 1
        vals = []
        for i in range(args.warmup + args.steps):
            v = cpu_sample(threads, threads, 256, 4)
            if i >= args.warmup:
                vals.append(v)
        tps = float(np.mean([v[0] for v in vals]))
        print(json.dumps({
            "impl": "reference", "metric": "infer_tokens_per_s", "value": tps, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1000.0 * float(np.mean([v[3] for v in vals])), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "i8", "data": "synthetic", "config": config(),
            "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": vals[0][1], "sample": vals[0][2]},
            "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}))
        return

    import torch
    import torch.distributed as dist
    from tscale_b200 import infer

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    steps, warmup = args.steps, max(args.warmup, 3)
    layers = layer_plan()
    rng = np.random.default_rng(SEED + 1000 * rank)
    ctx0 = [int(x) for x in rng.integers(CTX_LO, CTX_HI + 1, N_SEQ)]
    e_steps = min(steps, 50)
    cap = CTX_HI + 2 * steps + warmup + e_steps + 16
    model = infer.InferModel(make_model(layers), fill_rope(D, cap), dev)
    ctx = infer.InferContext(model, N_SEQ, cap)
    gen = torch.Generator(device=dev)
    gen.manual_seed(SEED + 1000 * rank)
    for l in range(LAYERS):
        ctx.k[l].copy_(torch.randint(-127, 128, ctx.k[l].shape, generator=gen, device=dev, dtype=torch.int8))
        ctx.v[l].copy_(torch.randint(-127, 128, ctx.v[l].shape, generator=gen, device=dev, dtype=torch.int8))
        ctx.k_scale[l].copy_(torch.rand(ctx.k_scale[l].shape, generator=gen, device=dev) * 2e-4 + 1e-4)
        ctx.v_scale[l].fill_(1 / 24.0)
    ctx.set_lengths(ctx0)
    labels = torch.randint(0, VOCAB, (N_SEQ, 1), generator=gen, device=dev, dtype=torch.int32)
    pred = torch.empty((N_SEQ, VOCAB), dtype=torch.float32, device=dev)
    launches_per_step = 2 + LAYERS * 7 + 4   # embedding, first normalise; per layer 4 matrix products, rope, 2 attention kernels; count, final layer, 2 softmax kernels

    # one eager step (also sets the kernels' attributes), then the step as a CUDA graph
    ctx.compute_prediction(labels, prediction=pred)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            ctx.compute_prediction(labels, prediction=pred, max_ctx_bound=cap - 1)
    torch.cuda.synchronize()
    lens = [n + 1 for n in ctx0]   # the captured step has not run yet

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        graph.replay()
        lens = [n + 1 for n in lens]
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    nbytes = 0.0
    barrier()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        graph.replay()
        lens = [n + 1 for n in lens]
        nbytes += kv_bytes(lens, layers) + weight_bytes()
    t1.record()
    barrier()
    ms_total = t0.elapsed_time(t1)
    clocks = sampler.stop() if rank == 0 else None
    assert int(ctx.status.item()) == 0
    assert abs(float(pred.sum().item()) - N_SEQ) < 1e-2
    tt = torch.tensor([ms_total], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    ms_step = float(tt.item()) / steps
    value = N_SEQ * world / (ms_step * 1e-3)

    # end to end: labels from pinned host memory, the distributions back to the host, every step
    host_labels = labels.cpu().pin_memory()
    host_pred = torch.empty(pred.shape, dtype=pred.dtype).pin_memory()

    def e2e_step():
        labels.copy_(host_labels, non_blocking=True)
        graph.replay()
        host_pred.copy_(pred, non_blocking=True)

    e2e_step()
    barrier()
    t0.record()
    for _ in range(e_steps):
        e2e_step()
    t1.record()
    barrier()
    tt = torch.tensor([t0.elapsed_time(t1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    e_ms = float(tt.item()) / e_steps
    e2e = {"value": N_SEQ * world / (e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": host_labels.numel() * 4,
           "d2h_bytes_per_step": host_pred.numel() * 4, "ms_per_step": e_ms, "steps": e_steps}
    assert int(ctx.status.item()) == 0

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peaks = load_peaks()
    step_bytes = nbytes / steps
    achieved = step_bytes / (ms_step * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": "whole step: DecodePartialKernel<64> on the wide layers + int8 matrix products", "achieved": achieved,
                "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                "peak_source": "MEASURED_PEAKS.json copy bandwidth (%s)" % peaks["_source"], "ms_per_launch": ms_step,
                "algorithmic_bytes_per_launch": step_bytes, "kv_bytes_per_step": step_bytes - weight_bytes(), "weight_bytes_per_step": weight_bytes(),
                "traffic": None}
    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        tps, kind, sample, sec = cpu_sample(threads, threads, 256, 4)
        cpu_baseline = {"value": tps, "unit": "tokens/s", "cores": threads, "kind": kind, "sample": sample, "seconds": sec}
    print(json.dumps({
        "metric": "infer_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "i8", "data": "synthetic",
        "config": config(), "clocks": clocks, "e2e": e2e, "gpu_launches": launches_per_step * steps, "roofline": roofline,
        "cpu_baseline": cpu_baseline}))
    if world > 1:
        dist.destroy_process_group()
