"""Shared helpers of the parity tests: seeded inputs, quantisation through the oracle, error metrics."""
import numpy as np

from oracle import oracle as O

# tolerances of the path (softmax outputs / fp8 paths against the fp32-accumulated oracle)
OUT_MAX_ABS = 2e-2
OUT_MEAN_ABS = 2e-3
GRAD_REL_L2 = 1e-2

# arguments of oracle.make_infer_model for the inference fixtures tests/golden/infer_*.npz (the models are rebuilt
# from their seeds; the fixtures hold the label streams and the reference's predictions)
INFER_CASES = {
    "infer_d64": dict(seed=40, dim=256, head_dim=64, heads=2, relu_mult=1, vocab=300, label_count=40,
                      widths_slopes=[(8, 0.5), (0, 0.0), (64, 0.0)]),
    "infer_d128": dict(seed=41, dim=384, head_dim=128, heads=3, relu_mult=2, vocab=150, label_count=20, widths_slopes=[(16, 0.0), (4, 0.5)]),
}


def make_qkv(seed, length, heads, dq, dv, scale=1.0):
    rng = np.random.default_rng(seed)
    q = (rng.standard_normal((length, heads * dq)) * scale).astype(np.float32)
    k = (rng.standard_normal((length, heads * dq)) * scale).astype(np.float32)
    v = (rng.standard_normal((length, heads * dv)) * scale).astype(np.float32)
    return q, k, v


def quantize(x, dtype, tile):
    """abs-max per (row, head) quantisation through the oracle; returns bytes, scale [H][len], dequantised."""
    b, s = O.quant_rows("absmax", dtype, 0.0, x, tile)
    ln, xs = x.shape
    deq = (O.dequant(b, dtype).reshape(ln, xs // tile, tile) * s.T[:, :, None]).reshape(ln, xs)
    return b, s, deq.astype(np.float32)


def err_stats(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    d = np.abs(a - b)
    return float(d.max()) if d.size else 0.0, float(d.mean()) if d.size else 0.0


def rel_l2(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    den = np.sqrt((b * b).sum())
    return float(np.sqrt(((a - b) ** 2).sum()) / max(den, 1e-30))


def to_np(t):
    import torch
    if t.dtype == torch.bfloat16:
        t = t.float()
    return t.detach().cpu().numpy()


def describe(got, want):
    """Short diagnosis of a mismatch: error stats, median ratio, worst rows."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    d = np.abs(got - want)
    big = np.abs(want) > 0.05
    ratio = np.median(got[big] / want[big]) if big.any() else float("nan")
    rows = np.argsort(d.max(axis=1))[-4:][::-1]
    return "max %.3g mean %.3g median ratio %.4g worst rows %s (err %s) nan %d" % (
        d.max(), d.mean(), ratio, rows.tolist(), np.round(d.max(axis=1)[rows], 4).tolist(), int(np.isnan(got).sum()))
