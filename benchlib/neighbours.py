"""`bench.py --workload neighbours`: the kernels on either side of the attention path, timed alone with CUDA events on
the shapes of the prefill (65536 rows, 12 heads x 64) and training (32768 rows, 16 heads x 128) workloads:

  producer  tsa_norm_rope_quant / tsa_rope_norm_bwd      HBM-bound, algorithmic bytes = source + rope + bytes out + scales
  fused     tsa_matmul_norm_rope_quant                   int8 projection (tensor) with the producer as its epilogue
  consumer  tsa_kv_product / tsa_kv_product_bwd          HBM-bound
  fused consumer  tsa_att_fwd_kv against tsa_att_fwd followed by tsa_kv_product (same buffers, same results)

One JSON line: `value` is the producer's forward bandwidth on the first shape, `kernels` lists every measurement.
Inputs are larger than L2 except the fused kernel's int8 operands; each kernel runs 3 warm-up and 20 timed launches.
"""
import json

import numpy as np

from .util import ClockSampler, load_peaks

SHAPES = ((65536, 768, 12, 64), (32768, 2048, 16, 128))


def run(args, rank, world, local_rank):
    if args.impl == "reference" or rank != 0:
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "the neighbours workload times GPU kernels only; the CPU arm covers prefill125m, decode and infer"}))
        return
    import torch
    from tscale_b200 import ops

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    peaks = load_peaks()
    sampler = ClockSampler(local_rank)
    sampler.start()
    out = []
    launches = [0]

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(20):
            fn()
        e1.record()
        torch.cuda.synchronize()
        launches[0] += 20
        return e0.elapsed_time(e1) / 20

    def note(kernel, shape, ms, nbytes=None, ops_count=None):
        rec = {"kernel": kernel, "rows": shape[0], "dim": shape[1], "heads": shape[2], "head_dim": shape[3], "ms": ms}
        if nbytes is not None:
            rec["gbs"] = nbytes / ms / 1e6
            rec["frac_of_measured_hbm"] = rec["gbs"] / peaks["hbm_gbs"]
        if ops_count is not None:
            rec["tops"] = ops_count / ms / 1e9
        out.append(rec)

    for shape in SHAPES:
        rows, dim, heads, d = shape
        n = rows * heads * d
        gen = torch.Generator(device=dev)
        gen.manual_seed(7)
        rope16 = torch.randn((rows, d), generator=gen, device=dev).half()
        rope32 = rope16.float()
        for sdt, name in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
            x = (torch.randn((rows, heads * d), generator=gen, device=dev) * 2).to(sdt)
            g = torch.randn_like(x)
            es = x.element_size()
            note("tsa_norm_rope_quant %s -> e4m3" % name, shape, timed(lambda: ops.norm_rope_quant(x, rope16, "e4m3", heads, d, 0.25)),
                 nbytes=n * es + n + rows * d * 2 + rows * heads * 4)
            note("tsa_rope_norm_bwd %s" % name, shape, timed(lambda: ops.rope_norm_bwd(x, g, rope16, heads, d)), nbytes=3 * n * es + rows * d * 2)
            del x, g
        xi = torch.randint(-127, 128, (rows, dim), generator=gen, device=dev, dtype=torch.int8)
        wi = torch.randint(-127, 128, (heads * d, dim), generator=gen, device=dev, dtype=torch.int8)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        note("tsa_matmul_norm_rope_quant i8 x i8 -> e4m3", shape,
             timed(lambda: ops.matmul_norm_rope_quant(xi, wi, rope32, "e4m3", heads, d, vec_scale=0.25, src_scale=1 / 4096.0, status=status)),
             nbytes=rows * dim + heads * d * dim + n + rows * d * 4 + rows * heads * 4, ops_count=2.0 * rows * dim * heads * d)
        assert int(status.item()) == 0
        k = torch.randn((rows, heads * d), generator=gen, device=dev).bfloat16()
        v = torch.randn((rows, heads * d), generator=gen, device=dev).bfloat16()
        gk = torch.randn((rows, heads * d * 4), generator=gen, device=dev).bfloat16()
        note("tsa_kv_product bf16", shape, timed(lambda: ops.kv_product(k, v, heads, d)), nbytes=2 * (2 + 4) * n)
        note("tsa_kv_product_bwd bf16", shape, timed(lambda: ops.kv_product_bwd(k, v, gk, heads, d)), nbytes=2 * (2 + 4 + 2) * n + rows * heads * 4)
        del k, v, gk
    # the consumer fused into the attention kernel against the two launches it replaces
    for name, frags, seq, heads, d, window in (("window 64", 16, 4096, 12, 64, 64), ("full causal", 16, 4096, 12, 64, 0),
                                                ("full causal", 1, 32768, 16, 128, 0)):
        rows = frags * seq
        gen = torch.Generator(device=dev)
        gen.manual_seed(3)
        t = {}
        for nm in ("q", "k", "v"):
            x = torch.randn((rows, heads * d), generator=gen, device=dev) * 0.5
            t[nm], t["s" + nm] = ops.quant_rows(x, "absmax", "e4m3", d)
            del x
        mask = ops.Mask.window([seq] * frags, window)
        cfg = ops.make_cfg("e4m3", "e4m3", d, d, out_dtype=torch.bfloat16)
        att_out = torch.empty((rows, heads * d), dtype=torch.bfloat16, device=dev)
        lse = torch.empty((heads, rows), dtype=torch.float32, device=dev)
        ws = torch.empty(1 << 16, dtype=torch.uint8, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        ck = torch.randn((rows, heads * d), generator=gen, device=dev).bfloat16()
        kv_a = torch.empty((rows, 4 * heads * d), dtype=torch.bfloat16, device=dev)
        kv_b = torch.empty_like(kv_a)

        def att(**kw):
            return ops.att_fwd(cfg, t["q"], t["k"], t["v"], t["sk"], mask, 0.0, heads, qk_scale=t["sq"], v_scale=t["sv"], out=att_out, lse=lse,
                               workspace=ws, status=status, **kw)

        def two_launches():
            att()
            ops.kv_product(ck, att_out, heads, d, kv_mult=0.5, out=kv_a)

        shape = (rows, heads * d, heads, d)
        ms_att = timed(att)
        ms_two = timed(two_launches)
        ms_fused = timed(lambda: att(combiner_k=ck, kv_mult=0.5, kv=kv_b))
        assert int(status.item()) == 0 and torch.equal(kv_a, kv_b)
        out.append({"kernel": "tsa_att_fwd_kv e4m3 %s, %d x %d" % (name, frags, seq), "rows": rows, "dim": heads * d, "heads": heads, "head_dim": d,
                    "ms": ms_fused, "ms_attention_alone": ms_att, "ms_attention_then_kv_product": ms_two, "same_bits": True})
        del t, att_out, kv_a, kv_b, ck
    clocks = sampler.stop()
    first = out[0]
    print(json.dumps({
        "metric": "producer_hbm_gbs", "value": first["gbs"], "unit": "GB/s", "n_gpus": 1, "steps": 20, "warmup": 3, "ms_per_step": first["ms"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "neighbours", "shapes": [list(s) for s in SHAPES], "l2": "inputs larger than L2"}, "clocks": clocks,
        "gpu_launches": launches[0], "roofline": {"bound": "hbm", "achieved": first["gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                                  "frac": first["gbs"] / peaks["hbm_gbs"], "traffic": None,
                                                  "peak_source": "MEASURED_PEAKS.json copy bandwidth (%s)" % peaks["_source"]},
        "kernels": out}))
