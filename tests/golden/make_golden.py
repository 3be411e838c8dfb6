"""Generates tests/golden/*.npz from the reference's own CPU code (oracle/_ref/libtsa_ref.so, built by
oracle/Makefile from a reference checkout).  The reference ships no golden vectors for its attention
path, so these known-answer files are produced by running its code on small seeded inputs; they pin
the restated oracle on machines where the reference checkout is absent.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
from oracle import oracle as O  # noqa: E402
from tests.util import INFER_CASES  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def spans_from_rows(rows):
    spans, ptr = [], [0]
    for r in rows:
        spans.extend(r)
        ptr.append(len(spans))
    return np.array(spans, dtype=np.int32).reshape(-1, 2), np.array(ptr, dtype=np.int32)


def att_case(name, seed, frag_lens, heads, dq, dv, window, slope, custom_rows=None):
    rng = np.random.default_rng(seed)
    ln = sum(frag_lens)
    q = rng.standard_normal((ln, heads * dq)).astype(np.float32)
    k = rng.standard_normal((ln, heads * dq)).astype(np.float32)
    v = rng.standard_normal((ln, heads * dv)).astype(np.float32)
    d_out = (rng.standard_normal((ln, heads * dv)) * 1e-2).astype(np.float32)
    if custom_rows is None:
        spans, ptr = O.window_spans(frag_lens, window)
    else:
        spans, ptr = spans_from_rows(custom_rows)
    fwd = O.att_fwd(q, k, v, spans, ptr, heads, slope, use_ref=True)
    bwd = O.att_bwd(q, k, v, d_out, spans, ptr, heads, slope, use_ref=True, fwd=fwd,
                    rev=O.transpose_attention(spans, ptr, use_ref=True))
    rev = O.transpose_attention(spans, ptr, use_ref=True)
    grp = O.group_attention(spans, ptr, use_ref=True)
    rgrp = O.group_attention(rev[0], rev[1], use_ref=True)
    np.savez_compressed(
        os.path.join(HERE, name + ".npz"), heads=heads, slope=np.float32(slope), q=q, k=k, v=v, d_out=d_out,
        spans=spans, span_ptr=ptr, out=fwd["out"], sum_weight=fwd["sum_weight"], max_dp=fwd["max_dp"],
        dq=bwd["dq"], dk=bwd["dk"], dv=bwd["dv"], dscale=bwd["dscale"],
        rev_spans=rev[0], rev_span_ptr=rev[1], groups=grp[0], group_ptr=grp[1],
        rev_groups=rgrp[0], rev_group_ptr=rgrp[1])
    print(name, "len", ln, "spans", len(spans), "groups", len(grp[0]))


def decode_case(name, seed, ctx, heads, d, width, slope):
    rng = np.random.default_rng(seed)
    kc = rng.integers(-127, 128, (ctx, heads * d)).astype(np.int8)
    vc = rng.integers(-127, 128, (ctx, heads * d)).astype(np.int8)
    ks = (rng.random((ctx, heads)) * 2e-4 + 1e-4).astype(np.float32)
    q8 = rng.integers(-127, 128, (heads * d,)).astype(np.int8)
    out = O.decode_step(kc, ks, vc, None, q8, None, heads, width, slope, use_ref=True)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), heads=heads, width=width, slope=np.float32(slope),
                        k_cache=kc, v_cache=vc, k_scale=ks, q8=q8, out=out,
                        vec_scale=np.float32(O.ref().ref_vec_scale()))
    print(name, "ctx", ctx)


def producer_case(name, seed, rows, heads, d):
    """NormalizeState + ApplyRope of the reference (gpt_cpu.cpp:297-324, 625-630; att/rope.cpp) on seeded projections."""
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal((rows, heads * d)) * 2.0).astype(np.float32)
    x[3] = 0
    table = O.fill_rope(d, rows, use_ref=True)
    norm = O.normalize_state_ref(x, heads)
    fwd = O.apply_rope(table, norm, 1.0, use_ref=True)
    back = O.apply_rope(table, fwd, -1.0, use_ref=True)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), heads=heads, d=d, src=x, rope=table, roped=fwd, unroped=back)
    print(name, rows, heads, d)


def consumer_case(name, seed, rows, heads, d):
    """KVProduct / KVProductBackprop of the reference (gpt_cpu.cpp:191-262)."""
    rng = np.random.default_rng(seed)
    k = rng.standard_normal((rows, heads * d)).astype(np.float32)
    v = rng.standard_normal((rows, heads * d)).astype(np.float32)
    g = rng.standard_normal((rows, heads * d * 4)).astype(np.float32)
    kv = O.kv_product(k, v, heads, use_ref=True)
    dk, dv, ds = O.kv_product_bwd(k, v, g, heads, use_ref=True)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), heads=heads, d=d, k=k, val=v, dkv=g, kv=kv, dk=dk, dval=dv, dscale=ds)
    print(name, rows, heads, d)


def infer_case(name, steps, n_seq):
    """Predictions of the reference's own ComputePrediction (cpu_infer.cpp:530-560) for n_seq label streams."""
    model = O.make_infer_model(**INFER_CASES[name])
    rng = np.random.default_rng(INFER_CASES[name]["seed"] + 1000)
    labels = rng.integers(0, model["label_count"], (n_seq, steps, 1)).astype(np.int32)
    pred = np.zeros((n_seq, steps, model["vocab"]), dtype=np.float32)
    for s in range(n_seq):
        ref = O.InferOracle(model, steps, use_ref=True)
        for t in range(steps):
            pred[s, t] = ref.step(labels[s, t])
    np.savez_compressed(os.path.join(HERE, name + ".npz"), labels=labels, prediction=pred)
    print(name, steps, n_seq)


def main():
    assert O.ref() is not None, "build oracle/_ref first (make -C oracle ref)"
    # window-64 layers of the reference use ALiBi slope 0.5, wide layers slope 0 (model_dim.cpp:83-90)
    att_case("att_w64_slope05", 0, [160, 96], 2, 64, 64, 64, 0.5)
    att_case("att_full_slope0", 1, [130, 62], 2, 128, 128, 0, 0.0)
    att_case("att_w1_d32", 2, [40], 3, 32, 64, 1, 0.0)
    # hand-made mask: empty rows, multi-span rows, a key visited from non-adjacent rows, self-attention row
    rows = [[], [(0, 0)], [(0, 1)], [], [(0, 0), (2, 3)], [(1, 1), (3, 4)], [(6, 6)], [(0, 2), (4, 4), (6, 6)],
            [(5, 7)], [], [(9, 9)], [(0, 10)]]
    att_case("att_handmade", 3, [12], 2, 16, 16, None, 0.25, custom_rows=rows)
    decode_case("decode_w64", 10, 200, 2, 128, 64, 0.5)
    decode_case("decode_wide", 11, 333, 3, 64, 1024, 0.0)
    decode_case("decode_w0", 12, 17, 2, 128, 0, 0.0)
    decode_case("decode_first", 13, 1, 2, 64, 64, 0.5)
    producer_case("producer_d64", 20, 150, 3, 64)
    producer_case("producer_d128", 21, 90, 2, 128)
    consumer_case("consumer_d64", 30, 40, 3, 64)
    infer_case("infer_d64", 24, 3)
    infer_case("infer_d128", 12, 2)
    # 8-bit code points: ConvertE4toFloat for all bytes, Float2I8 on a grid
    e4 = np.array([O.ref().ref_e4m3_to_float(i) for i in range(256)], dtype=np.float32)
    grid = np.concatenate([np.linspace(-130, 130, 2081), np.array([0.5, 1.5, 2.5, -0.5, -1.5, -2.5])]).astype(np.float32)
    i8 = np.array([O.ref().ref_float2i8(float(x)) for x in grid], dtype=np.int32)
    np.savez_compressed(os.path.join(HERE, "codes.npz"), e4m3=e4, i8_grid=grid, i8=i8)


if __name__ == "__main__":
    main()
