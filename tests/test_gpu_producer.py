"""GPU parity of tsa_norm_rope_quant (per-head RMS normalise, rope, quantise) against the CPU oracle, and the chain
producer -> attention forward against the oracle chain."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import util

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _codes_close(got, want, dst):
    """Bytes equal except where the value sat on a rounding boundary: there the neighbouring code is accepted."""
    got = got.astype(np.int8)
    want = want.astype(np.int8)
    diff = got != want
    frac = diff.mean()
    if dst == "i8":
        step = np.abs(got.astype(np.int32) - want.astype(np.int32))
    else:
        step = np.abs(O.dequant(got, "e4m3") - O.dequant(want, "e4m3")) / np.maximum(np.abs(O.dequant(want, "e4m3")), 2.0 ** -6)
        step = np.where(diff, np.ceil(step * 8 - 1e-6), 0)  # in units of the e4m3 spacing (1/8 relative)
    return frac, float(step.max()) if step.size else 0.0


@pytest.mark.parametrize("d,heads", [(64, 12), (128, 5)])
@pytest.mark.parametrize("dst", ["i8", "e4m3"])
@pytest.mark.parametrize("src_dtype,rope_dtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.float16), (torch.float16, None)])
@pytest.mark.parametrize("direction", [1.0, -1.0])
def test_norm_rope_quant(d, heads, dst, src_dtype, rope_dtype, direction):
    from tscale_b200 import ops
    rng = np.random.default_rng(31)
    rows = 777
    src_t = torch.from_numpy(rng.standard_normal((rows, heads * d)).astype(np.float32) * 3.0).to(src_dtype)
    src_t[5] = 0  # an all-zero row: scale 0, zeros out
    rope_np = O.fill_rope(d, rows)
    rope_t = None if rope_dtype is None else torch.from_numpy(rope_np).to(rope_dtype)
    vec_scale = 1 / 24.0 if dst == "i8" else 1 / 4.0
    want_b, want_s, _ = O.norm_rope_quant(dst, vec_scale, src_t.float().numpy(), None if rope_t is None else rope_t.float().numpy(), d, direction)
    got_b, got_s = ops.norm_rope_quant(src_t.to(DEV), None if rope_t is None else rope_t.to(DEV), dst, heads, d, vec_scale, direction)
    torch.cuda.synchronize()
    got_s = got_s.cpu().numpy()
    assert np.allclose(got_s, want_s, rtol=2e-6, atol=0), float(np.abs(got_s - want_s).max())
    assert got_s[:, 5].max() == 0
    frac, step = _codes_close(got_b.cpu().numpy().view(np.int8), want_b, dst)
    assert frac < 2e-3 and step <= 1, (frac, step)


def test_producer_feeds_attention():
    """fp32 projections -> tsa_norm_rope_quant -> tsa_att_fwd against the oracle chain on the same inputs."""
    from tscale_b200 import ops
    rng = np.random.default_rng(32)
    frag_lens, heads, d, window, slope = [300, 212], 4, 64, 64, 0.5
    rows = sum(frag_lens)
    rope_np = O.fill_rope(d, rows)
    proj = {n: (rng.standard_normal((rows, heads * d)) * 2.0).astype(np.float32) for n in ("q", "k", "v")}
    vec = 1 / 4.0
    dev_in, deq = {}, {}
    for n in ("q", "k", "v"):
        rope = rope_np if n != "v" else None
        b, s, _ = O.norm_rope_quant("e4m3", vec, proj[n], rope, d)
        deq[n] = (O.dequant(b, "e4m3").reshape(rows, heads, d) * s.T[:, :, None]).reshape(rows, heads * d).astype(np.float32)
        dev_in[n] = ops.norm_rope_quant(torch.from_numpy(proj[n]).to(DEV), None if rope is None else torch.from_numpy(rope).to(DEV),
                                        "e4m3", heads, d, vec)
    spans, ptr = O.window_spans(frag_lens, window)
    ref = O.att_fwd(deq["q"], deq["k"], deq["v"], spans, ptr, heads, slope)
    cfg = ops.make_cfg("e4m3", "e4m3", d, d, out_dtype=torch.float32)
    mask = ops.Mask.window(frag_lens, window)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out, lse = ops.att_fwd(cfg, dev_in["q"][0], dev_in["k"][0], dev_in["v"][0], dev_in["k"][1], mask, slope, heads,
                           qk_scale=dev_in["q"][1], v_scale=dev_in["v"][1], status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    vmax = float(np.abs(deq["v"]).max())
    mx, mean = util.err_stats(util.to_np(out), ref["out"])
    # a handful of bytes may sit one code off a rounding boundary: tolerance relative to the value range as elsewhere
    assert mx < max(util.OUT_MAX_ABS, 0.06 * vmax) and mean < max(util.OUT_MEAN_ABS, 0.01 * vmax), util.describe(util.to_np(out), ref["out"])


@pytest.mark.parametrize("d,heads", [(64, 12), (128, 5), (256, 2)])
@pytest.mark.parametrize("src_dtype,grad_dtype,rope_dtype", [(torch.float32, torch.float32, torch.float32),
                                                             (torch.bfloat16, torch.bfloat16, torch.float16),
                                                             (torch.float32, torch.bfloat16, None)])
def test_rope_norm_bwd(d, heads, src_dtype, grad_dtype, rope_dtype):
    from tscale_b200 import ops
    rng = np.random.default_rng(33)
    rows = 555
    src_t = torch.from_numpy((rng.standard_normal((rows, heads * d)) * 2.0).astype(np.float32)).to(src_dtype)
    src_t[9] = 0
    grad_t = torch.from_numpy(rng.standard_normal((rows, heads * d)).astype(np.float32)).to(grad_dtype)
    rope_t = None if rope_dtype is None else torch.from_numpy(O.fill_rope(d, rows)).to(rope_dtype)
    want = O.rope_norm_bwd(src_t.float().numpy(), grad_t.float().numpy(), None if rope_t is None else rope_t.float().numpy(), d)
    got = ops.rope_norm_bwd(src_t.to(DEV), grad_t.to(DEV), None if rope_t is None else rope_t.to(DEV), heads, d)
    torch.cuda.synchronize()
    got = util.to_np(got)
    assert np.abs(got[9]).max() == 0
    tol = 1e-5 if grad_dtype == torch.float32 else 1e-2  # bf16 results carry their own rounding
    assert util.rel_l2(got, want) < tol, util.rel_l2(got, want)


def test_norm_rope_quant_pads_with_zeros():
    """Rows in [len, rows) of the destination are written with zeros and scale 0, like the reference's padding rows."""
    from tscale_b200 import ops
    rng = np.random.default_rng(34)
    heads, d, rows, length = 3, 64, 128, 100
    src = torch.from_numpy(rng.standard_normal((rows, heads * d)).astype(np.float32)).to(DEV)
    rope = torch.from_numpy(O.fill_rope(d, rows)).to(DEV)
    b, s = ops.norm_rope_quant(src, rope, "i8", heads, d, 1 / 24.0, length=length)
    torch.cuda.synchronize()
    assert int(b[length:].abs().max().item()) == 0 and float(s[:, length:].abs().max().item()) == 0
    want_b, want_s, _ = O.norm_rope_quant("i8", 1 / 24.0, src[:length].cpu().numpy(), rope[:length].cpu().numpy(), d)
    frac, step = _codes_close(b[:length].cpu().numpy().view(np.int8), want_b, "i8")
    assert frac < 2e-3 and step <= 1


@pytest.mark.parametrize("dst", ["i8", "e4m3"])
@pytest.mark.parametrize("rows,length,dim,heads,d,with_rope", [
    (300, 300, 256, 3, 64, True), (257, 200, 768, 12, 64, True), (130, 130, 384, 2, 128, True), (512, 512, 512, 5, 128, False),
])
def test_matmul_norm_rope_quant_bit_exact(dst, rows, length, dim, heads, d, with_rope):
    """The projection fused with the producer: int32 products are exact and the epilogue follows the oracle's rounding
    order (sequential sum of squares, separate roundings), so bytes and scales equal the oracle's
    norm_rope_quant of the same projection bit for bit; padding rows are zero."""
    from tscale_b200 import ops
    rng = np.random.default_rng(rows + dim + heads)
    x = rng.integers(-127, 128, (rows, dim)).astype(np.int8)
    x[7] = 0                                                 # a row of zeros: scale 0, bytes 0
    w = rng.integers(-127, 128, (heads * d, dim)).astype(np.int8)
    src_scale = np.float32(1.0 / 4096)
    y = (x[:length].astype(np.int32) @ w.T.astype(np.int32)).astype(np.float32) * src_scale
    table = O.fill_rope(d, rows) if with_rope else None
    want_b, want_s, _ = O.norm_rope_quant(dst, 1 / 24.0, y, None if table is None else table[:length], d)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    got_b, got_s = ops.matmul_norm_rope_quant(torch.from_numpy(x).to(DEV), torch.from_numpy(w).to(DEV),
                                              None if table is None else torch.from_numpy(table).to(DEV), dst, heads, d,
                                              vec_scale=1 / 24.0, src_scale=float(src_scale), length=length, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    got_b = got_b.cpu().numpy().view(np.int8)
    got_s = got_s.cpu().numpy()
    assert np.array_equal(got_s[:, :length], want_s)
    assert np.array_equal(got_b[:length], want_b)
    assert np.abs(got_b[length:]).max(initial=0) == 0 and np.abs(got_s[:, length:]).max(initial=0) == 0
    assert got_s[:, 7].max() == 0


@pytest.mark.parametrize("rows,dim,heads,d", [(300, 256, 3, 64), (200, 512, 2, 128)])
def test_matmul_norm_rope_quant_e4m3_operands(rows, dim, heads, d):
    """e4m3 x e4m3 projection: the tensor cores add the products in f32 in their own order, so the projection matches
    the float64 product to f32 rounding and the output codes differ from the oracle's at rounding boundaries only."""
    from tscale_b200 import ops
    rng = np.random.default_rng(rows + dim)
    xf = (rng.standard_normal((rows, dim)) * 0.7).astype(np.float32)
    wf = (rng.standard_normal((heads * d, dim)) * 0.7).astype(np.float32)
    x8 = np.array([O.lib().oracle_f32_to_e4m3(float(v)) for v in xf.ravel()], dtype=np.uint8).reshape(xf.shape)
    w8 = np.array([O.lib().oracle_f32_to_e4m3(float(v)) for v in wf.ravel()], dtype=np.uint8).reshape(wf.shape)
    y = (O.e4m3_to_f32(x8).astype(np.float64) @ O.e4m3_to_f32(w8).astype(np.float64).T).astype(np.float32)
    table = O.fill_rope(d, rows)
    want_b, want_s, _ = O.norm_rope_quant("i8", 1 / 24.0, y, table, d)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    got_b, got_s = ops.matmul_norm_rope_quant(torch.from_numpy(x8).to(DEV), torch.from_numpy(w8).to(DEV), torch.from_numpy(table).to(DEV), "i8",
                                              heads, d, vec_scale=1 / 24.0, status=status, src="e4m3")
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert np.allclose(got_s.cpu().numpy(), want_s, rtol=2e-6, atol=0)
    frac, step = _codes_close(got_b.cpu().numpy().view(np.int8), want_b, "i8")
    assert frac < 2e-3 and step <= 1, (frac, step)


def test_block_chain_projection_attention_consumer():
    """The whole block front to back: int8 state x int8 matrices -> fused projection + producer (bit-exact, so the
    attention sees the oracle's own bytes and scale planes, in the layout it takes them) -> tsa_att_fwd -> tsa_kv_product,
    against the oracle chain."""
    from tscale_b200 import ops
    rng = np.random.default_rng(52)
    frag_lens, heads, d, dim, window, slope = [260, 124], 4, 64, 256, 64, 0.5
    rows = sum(frag_lens)
    x = rng.integers(-127, 128, (rows, dim)).astype(np.int8)
    rope_np = O.fill_rope(d, rows)
    vec, src_scale = 1 / 4.0, np.float32(1 / 2048.0)
    xd = torch.from_numpy(x).to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    dev_in, deq = {}, {}
    for n in ("q", "k", "v"):
        w = rng.integers(-127, 128, (heads * d, dim)).astype(np.int8)
        rope = rope_np if n != "v" else None
        y = (x.astype(np.int32) @ w.T.astype(np.int32)).astype(np.float32) * src_scale
        b, s, _ = O.norm_rope_quant("e4m3", vec, y, rope, d)
        deq[n] = (O.dequant(b, "e4m3").reshape(rows, heads, d) * s.T[:, :, None]).reshape(rows, heads * d).astype(np.float32)
        dev_in[n] = ops.matmul_norm_rope_quant(xd, torch.from_numpy(w).to(DEV), None if rope is None else torch.from_numpy(rope).to(DEV), "e4m3",
                                               heads, d, vec_scale=vec, src_scale=float(src_scale), status=status)
        assert np.array_equal(dev_in[n][0].cpu().numpy().view(np.int8), b) and np.array_equal(dev_in[n][1].cpu().numpy(), s), n
    spans, ptr = O.window_spans(frag_lens, window)
    ref = O.att_fwd(deq["q"], deq["k"], deq["v"], spans, ptr, heads, slope)
    cfg = ops.make_cfg("e4m3", "e4m3", d, d, out_dtype=torch.float32)
    mask = ops.Mask.window(frag_lens, window)
    out, _ = ops.att_fwd(cfg, dev_in["q"][0], dev_in["k"][0], dev_in["v"][0], dev_in["k"][1], mask, slope, heads,
                         qk_scale=dev_in["q"][1], v_scale=dev_in["v"][1], status=status)
    comb_key = rng.standard_normal((rows, heads * d)).astype(np.float32)
    kv = ops.kv_product(torch.from_numpy(comb_key).to(DEV), out, heads, d)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    # the values here are the projections themselves (tens in magnitude): the tolerances scale with their range
    vmax = float(np.abs(deq["v"]).max())
    mx, mean = util.err_stats(util.to_np(out), ref["out"])
    assert mx < util.OUT_MAX_ABS * vmax and mean < util.OUT_MEAN_ABS * vmax, util.describe(util.to_np(out), ref["out"])
    want_kv = O.kv_product(comb_key, ref["out"], heads)
    scale = float(np.abs(comb_key).max())
    assert np.abs(util.to_np(kv) - want_kv).max() < util.OUT_MAX_ABS * vmax * scale
    # the consumer itself is exact on the attention output it was given
    assert np.array_equal(util.to_np(kv), O.kv_product(comb_key, util.to_np(out), heads))


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,dim,heads,d,with_rope", [(200, 256, 3, 64, False), (150, 384, 2, 128, True)])
def test_matmul_norm_rope_16bit_output(dt, rows, dim, heads, d, with_rope):
    """16-bit output of the fused projection (the reference's K16): the oracle's normalised, rotated fp32 values rounded to
    the output type, bit for bit."""
    from tscale_b200 import ops
    rng = np.random.default_rng(rows + heads)
    x = rng.integers(-127, 128, (rows, dim)).astype(np.int8)
    w = rng.integers(-127, 128, (heads * d, dim)).astype(np.int8)
    src_scale = np.float32(1.0 / 1024)
    y = (x.astype(np.int32) @ w.T.astype(np.int32)).astype(np.float32) * src_scale
    table = O.fill_rope(d, rows) if with_rope else None
    _, want_s, roped = O.norm_rope_quant("i8", 0.5, y, table, d)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    got, got_s = ops.matmul_norm_rope_quant(torch.from_numpy(x).to(DEV), torch.from_numpy(w).to(DEV),
                                            None if table is None else torch.from_numpy(table).to(DEV), dt, heads, d,
                                            vec_scale=0.5, src_scale=float(src_scale), status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(got.cpu(), torch.from_numpy(roped).to(dt))
    assert np.array_equal(got_s.cpu().numpy(), want_s)
