"""Full-size runs of the four GPU workloads (the sizes bench.py uses), checked through properties that do not need
the CPU oracle to finish the whole problem:
  * causal prefix: the first rows of a fragment depend only on its first keys, so the oracle runs on a prefix /
    a few heads of ONE fragment of the big batch and must agree with those rows of the GPU result;
  * fragment permutation: rolling the order of the concatenated fragments rolls the result, bit for bit;
  * exact scaling: doubling the V scales (forward) or dOut (backward) doubles every result bit for bit.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import util

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _quant_batch(seed, length, heads, d, qk_dtype):
    from tscale_b200 import ops
    gen = torch.Generator(device=DEV)
    gen.manual_seed(seed)
    res = {}
    for name, dt in (("q", qk_dtype), ("k", qk_dtype), ("v", "e4m3")):
        x = torch.randn((length, heads * d), generator=gen, device=DEV) * 0.5
        res[name], res["s" + name] = ops.quant_rows(x, "absmax", dt, d)
        del x
    return res


def _deq(bytes_t, scale_t, dtype, rows, h0, nh, d):
    """Dequantised [len(rows)][nh*d] float32 of heads h0..h0+nh of the given row range (numpy, for the oracle)."""
    b = bytes_t[rows, h0 * d:(h0 + nh) * d].cpu().numpy()
    s = scale_t[h0:h0 + nh, rows].cpu().numpy()
    x = O.dequant(np.ascontiguousarray(b), dtype).reshape(b.shape[0], nh, d) * s.T[:, :, None]
    return np.ascontiguousarray(x.reshape(b.shape[0], nh * d).astype(np.float32))


def _oracle_prefix(g, qk_dtype, frag, seq, n, h0, nh, d, window, slope):
    rows = slice(frag * seq, frag * seq + n)
    qd = _deq(g["q"], g["sq"], qk_dtype, rows, h0, nh, d)
    kd = _deq(g["k"], g["sk"], qk_dtype, rows, h0, nh, d)
    vd = _deq(g["v"], g["sv"], "e4m3", rows, h0, nh, d)
    spans, ptr = O.window_spans([n], window)
    return O.att_fwd(qd, kd, vd, spans, ptr, nh, slope), (qd, kd, vd, spans, ptr)


def _fwd(cfg, g, mask, slope, heads, sv=None):
    from tscale_b200 import ops
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out, lse = ops.att_fwd(cfg, g["q"], g["k"], g["v"], g["sk"], mask, slope, heads, qk_scale=g["sq"],
                           v_scale=g["sv"] if sv is None else sv, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return out, lse


def _rolled(g, shift_rows):
    r = {}
    for n in ("q", "k", "v"):
        r[n] = torch.roll(g[n], shift_rows, 0)
        r["s" + n] = torch.roll(g["s" + n], shift_rows, 1)
    return r


@pytest.mark.parametrize("window,slope", [(64, 0.5), (0, 0.0)])
def test_prefill_125m_full_size(window, slope):
    from tscale_b200 import ops
    frags, seq, heads, d = 16, 4096, 12, 64
    g = _quant_batch(1, frags * seq, heads, d, "e4m3")
    cfg = ops.make_cfg("e4m3", "e4m3", d, d, out_dtype=torch.bfloat16)
    mask = ops.Mask.window([seq] * frags, window)
    out, lse = _fwd(cfg, g, mask, slope, heads)
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    # oracle on the first 1024 rows of fragment 11, all heads
    n, frag = 1024, 11
    ref, _ = _oracle_prefix(g, "e4m3", frag, seq, n, 0, heads, d, window, slope)
    got = util.to_np(out[frag * seq:frag * seq + n])
    mx, mean = util.err_stats(got, ref["out"])
    assert mx < util.OUT_MAX_ABS and mean < util.OUT_MEAN_ABS, util.describe(got, ref["out"])
    assert np.abs(util.to_np(lse[:, frag * seq:frag * seq + n]) - ref["lse"]).max() < 2e-2
    # fragments are independent: rolling their order by 5 rolls the result bit for bit
    out_r, lse_r = _fwd(cfg, _rolled(g, 5 * seq), mask, slope, heads)
    assert torch.equal(out_r, torch.roll(out, 5 * seq, 0)) and torch.equal(lse_r, torch.roll(lse, 5 * seq, 1))
    # doubling the value scales doubles the result exactly
    out_2, _ = _fwd(cfg, g, mask, slope, heads, sv=g["sv"] * 2)
    assert torch.equal(out_2.float(), out.float() * 2)


def test_longctx_full_size():
    from tscale_b200 import ops
    frags, seq, heads, d = 4, 32768, 32, 128
    g = _quant_batch(4, frags * seq, heads, d, "e4m3")
    cfg = ops.make_cfg("e4m3", "e4m3", d, d, out_dtype=torch.bfloat16)
    mask = ops.Mask.window([seq] * frags, 0)
    out, lse = _fwd(cfg, g, mask, 0.0, heads)
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    # oracle on the first 2048 rows of fragment 2, heads 29-31
    n, frag, h0, nh = 2048, 2, 29, 3
    ref, _ = _oracle_prefix(g, "e4m3", frag, seq, n, h0, nh, d, 0, 0.0)
    got = util.to_np(out[frag * seq:frag * seq + n, h0 * d:(h0 + nh) * d])
    mx, mean = util.err_stats(got, ref["out"])
    assert mx < util.OUT_MAX_ABS and mean < util.OUT_MEAN_ABS, util.describe(got, ref["out"])
    # the last rows of a fragment attend 32767 keys: their weights must still sum to one (lse finite and ordered)
    out_r, _ = _fwd(cfg, _rolled(g, seq), mask, 0.0, heads)
    assert torch.equal(out_r, torch.roll(out, seq, 0))


@pytest.mark.parametrize("window", [256, 0])
def test_train_15b_full_size(window):
    from tscale_b200 import ops
    frags, seq, heads, d = 8, 4096, 16, 128
    g = _quant_batch(2, frags * seq, heads, d, "i8")
    cfg = ops.make_cfg("i8", "e4m3", d, d, out_dtype=torch.bfloat16, grad_dtype=torch.bfloat16)
    mask = ops.Mask.window([seq] * frags, window)
    out, lse = _fwd(cfg, g, mask, 0.0, heads)
    gen = torch.Generator(device=DEV)
    gen.manual_seed(22)
    d_out = (torch.randn(out.shape, generator=gen, device=DEV) * 1e-2).to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)

    def bwd(gg, o, l, do):
        res = ops.att_bwd(cfg, gg["q"], gg["k"], gg["v"], gg["sk"], do, o, l, mask, 0.0, heads, qk_scale=gg["sq"],
                          v_scale=gg["sv"], status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        return res

    dq, dk, dv = bwd(g, out, lse, d_out)
    for t in (dq, dk, dv):
        assert torch.isfinite(t.float()).all()
    # doubling dOut doubles every gradient exactly (powers of two commute with every rounding on the path)
    dq2, dk2, dv2 = bwd(g, out, lse, d_out * 2)
    for a, b in ((dq, dq2), (dk, dk2), (dv, dv2)):
        assert torch.equal(b.float(), a.float() * 2)
    # fragments are independent
    gr = _rolled(g, 3 * seq)
    dqr, dkr, dvr = bwd(gr, torch.roll(out, 3 * seq, 0), torch.roll(lse, 3 * seq, 1), torch.roll(d_out, 3 * seq, 0))
    for a, b in ((dq, dqr), (dk, dkr), (dv, dvr)):
        assert torch.equal(b, torch.roll(a, 3 * seq, 0))
    if window > 0:
        # oracle on a whole fragment, 2 heads (window layers are cheap on the host); dK / dV of a fragment need all its rows
        frag, h0, nh = 5, 7, 2
        ref, (qd, kd, vd, spans, ptr) = _oracle_prefix(g, "i8", frag, seq, seq, h0, nh, d, window, 0.0)
        rows = slice(frag * seq, (frag + 1) * seq)
        cols = slice(h0 * d, (h0 + nh) * d)
        do_np = np.ascontiguousarray(d_out[rows, cols].float().cpu().numpy())
        gref = O.att_bwd(qd, kd, vd, do_np, spans, ptr, nh, 0.0, fwd=ref)
        for name, got in (("dq", dq), ("dk", dk), ("dv", dv)):
            r = util.rel_l2(util.to_np(got[rows, cols]), gref[name])
            assert r < 1.5 * util.GRAD_REL_L2, (name, r)  # + bf16 rounding of out, dOut and the gradients
    else:
        # full causal: dQ of the first n rows of a fragment depends only on the fragment's first n keys, so the oracle on that
        # prefix checks it (dK / dV of those rows also collect from later queries and are left to the invariances above)
        frag, h0, nh, n = 6, 3, 2, 1024
        ref, (qd, kd, vd, spans, ptr) = _oracle_prefix(g, "i8", frag, seq, n, h0, nh, d, 0, 0.0)
        rows = slice(frag * seq, frag * seq + n)
        cols = slice(h0 * d, (h0 + nh) * d)
        do_np = np.ascontiguousarray(d_out[rows, cols].float().cpu().numpy())
        gref = O.att_bwd(qd, kd, vd, do_np, spans, ptr, nh, 0.0, fwd=ref)
        r = util.rel_l2(util.to_np(dq[rows, cols]), gref["dq"])
        assert r < 1.5 * util.GRAD_REL_L2, ("dq prefix", r)


def test_decode_full_size():
    """64 sequences, contexts uniform in [1024, 8192], 16 heads x 128, fp16 scales: every sequence against the oracle."""
    from tscale_b200 import ops
    n_seq, heads, d = 64, 16, 128
    rng = np.random.default_rng(3)
    ctx = [int(x) for x in rng.integers(1024, 8193, n_seq)]
    cache = ops.KVCache(n_seq, 8200, heads, d, DEV, scale_dtype=torch.float16, out_dtype=torch.float32)
    gen = torch.Generator(device=DEV)
    gen.manual_seed(3)
    cache.k.copy_(torch.randint(-127, 128, cache.k.shape, generator=gen, device=DEV, dtype=torch.int8))
    cache.v.copy_(torch.randint(-127, 128, cache.v.shape, generator=gen, device=DEV, dtype=torch.int8))
    cache.k_scale.copy_((torch.rand(cache.k_scale.shape, generator=gen, device=DEV) * 2e-4 + 1e-4).half())
    cache.v_scale.copy_((torch.rand(cache.v_scale.shape, generator=gen, device=DEV) * 0.02 + 0.01).half())
    cache.ctx_lens.copy_(torch.tensor(ctx, dtype=torch.int32))
    cache.max_ctx = max(ctx)
    q = torch.randint(-127, 128, (n_seq, heads * d), generator=gen, device=DEV, dtype=torch.int8)
    qs = torch.full((n_seq, heads), 1 / 24.0, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = cache.decode(q, qs, 1 << 30, 0.0, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    got = out.cpu().numpy()
    k = cache.k.cpu().numpy()
    v = cache.v.cpu().numpy()
    ks = cache.k_scale.float().cpu().numpy()
    vs = cache.v_scale.float().cpu().numpy()
    qn = q.cpu().numpy()
    qsn = qs.cpu().numpy()
    worst = 0.0
    for s in range(n_seq):
        n = ctx[s]
        ref = O.decode_step(np.ascontiguousarray(k[s, :n]), np.ascontiguousarray(ks[s, :n]), np.ascontiguousarray(v[s, :n]),
                            np.ascontiguousarray(vs[s, :n]), qn[s], qsn[s], heads, 1 << 30, 0.0, exp_mode="exact")
        vmax = 127 * float(vs[s, :n].max())
        worst = max(worst, float(np.abs(got[s] - ref).max()) / vmax)
    assert worst < 2e-4, worst
