"""GPU parity of the attention forward / backward against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import util

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda:0")


def _setup(seed, frag_lens, heads, d, qk_dtype, v_dtype, scale=1.0, spans=None):
    from tscale_b200 import ops
    length = sum(frag_lens)
    q, k, v = util.make_qkv(seed, length, heads, d, d, scale)
    q8, sq, qd = util.quantize(q, qk_dtype, d)
    k8, sk, kd = util.quantize(k, qk_dtype, d)
    v8, sv, vd = util.quantize(v, v_dtype, d)
    dev = _dev()
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    g = dict(q8=t(q8.view(np.uint8)), k8=t(k8.view(np.uint8)), v8=t(v8.view(np.uint8)), sq=t(sq), sk=t(sk), sv=t(sv))
    return g, (qd, kd, vd)


def _run_fwd(seed, frag_lens, window, slope, heads, d, qk_dtype, v_dtype, out_dtype=torch.float32, scale=1.0,
             force_generic=False, custom=None):
    from tscale_b200 import ops
    g, (qd, kd, vd) = _setup(seed, frag_lens, heads, d, qk_dtype, v_dtype, scale)
    if custom is None:
        spans, ptr = O.window_spans(frag_lens, window)
        mask = ops.Mask.window(frag_lens, window)
    else:
        spans, ptr = custom
        mask = ops.Mask.from_spans(spans, ptr)
    ref = O.att_fwd(qd, kd, vd, spans, ptr, heads, slope)
    cfg = ops.make_cfg(qk_dtype, v_dtype, d, d, out_dtype=out_dtype, force_generic=force_generic)
    status = torch.zeros(1, dtype=torch.int32, device=_dev())
    out, lse = ops.att_fwd(cfg, g["q8"], g["k8"], g["v8"], g["sk"], mask, slope, heads, qk_scale=g["sq"], v_scale=g["sv"],
                           status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "device status %#x" % int(status.item())
    return util.to_np(out), util.to_np(lse), ref, (g, mask, cfg, spans, ptr, (qd, kd, vd))


@pytest.mark.parametrize("window,slope", [(64, 0.5), (64, 0.0), (0, 0.0)])
def test_fwd_generic_int8_config1_shape(window, slope):
    # configs[0] at reduced length: int8 Q/K/V with per-row absmax scales, D=64, fp32 output
    out, lse, ref, _ = _run_fwd(0, [320, 192], window, slope, 4, 64, "i8", "i8", force_generic=True)
    mx, mean = util.err_stats(out, ref["out"])
    assert mx < 1e-4 and mean < 1e-5, (mx, mean)
    assert util.err_stats(lse, ref["lse"])[0] < 1e-4


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("window,slope", [(64, 0.5), (0, 0.0), (256, 0.0)])
@pytest.mark.parametrize("qk_dtype,v_dtype", [("e4m3", "e4m3"), ("i8", "e4m3"), ("i8", "i8")])
def test_fwd_tcgen05(d, window, slope, qk_dtype, v_dtype):
    out_dtype = torch.float32 if v_dtype == "i8" else torch.bfloat16
    out, lse, ref, _ = _run_fwd(1, [384, 256, 128], window, slope, 3, d, qk_dtype, v_dtype, out_dtype=out_dtype, scale=0.5)
    mx, mean = util.err_stats(out, ref["out"])
    if v_dtype == "i8":
        # int8 values reach the tensor cores exactly and the weights carry their e4m3 residual on every tile (two e4m3
        # terms = a relative weight error of 2^-8, which a row with a single key shows in full: 0.4 % of |v| ~ 0.3)
        assert mx < 2e-3 and mean < 1e-4, util.describe(out, ref["out"])
    else:
        assert mx < util.OUT_MAX_ABS and mean < util.OUT_MEAN_ABS, util.describe(out, ref["out"])
    assert util.err_stats(lse, ref["lse"])[0] < 2e-3, util.describe(lse, ref["lse"])


@pytest.mark.parametrize("slope", [0.0, 0.5])
def test_fwd_config0_full_size_default_dispatch(slope, golden_dir):
    """The CPU-runnable configuration at its stated size (seed 0: batch 2 x 1024 tokens, 8 heads x 64, window 64, int8
    Q/K/V with per-row abs-max scales, fp32 output) through the default dispatch, i.e. the tensor-core kernel, against the
    oracle on the same quantised inputs."""
    out, lse, ref, _ = _run_fwd(0, [1024, 1024], 64, slope, 8, 64, "i8", "i8", out_dtype=torch.float32, scale=1.0)
    assert out.shape == (2048, 8 * 64)
    mx, mean = util.err_stats(out, ref["out"])
    # two e4m3 terms per weight = a relative weight error of 2^-8; a row with one or two keys shows it in full, so the
    # bound scales with the value range (N(0,1) values here: |v| up to about 4)
    vmax = float(np.abs(ref["out"]).max())
    assert mx < 5e-3 * vmax and mean < 2e-4 * vmax, (vmax, util.describe(out, ref["out"]))
    assert mx < util.OUT_MAX_ABS and mean < util.OUT_MEAN_ABS
    assert util.err_stats(lse, ref["lse"])[0] < 2e-3
    # and against the generic kernel (exact fp32 weights) on the same inputs
    out_g, lse_g, _, _ = _run_fwd(0, [1024, 1024], 64, slope, 8, 64, "i8", "i8", out_dtype=torch.float32, scale=1.0, force_generic=True)
    assert util.err_stats(out_g, ref["out"])[0] < 1e-4
    assert util.err_stats(out, out_g)[0] < 5e-3 * vmax


@pytest.mark.parametrize("heads,slices,qk_dtype,d", [(6, 4, "i8", 128), (5, 2, "e4m3", 64), (3, 3, "i8", 64), (4, 1, "e4m3", 128)])
def test_fwd_host_buffers_match_device_call(heads, slices, qk_dtype, d):
    """tsa_att_fwd_host (pinned host vectors, head slices copied in, computed and copied out concurrently) gives the bits of
    tsa_att_fwd on the same vectors in device memory, ragged last slice included, and the oracle's values; the optional
    device copy of the result holds the same bits; rows and columns around the host output stay untouched."""
    from tscale_b200 import ops
    frag_lens, window, slope = [384, 256, 128], 256, 0.25
    out_d, lse_d, ref, (g, mask, cfg, _, _, _) = _run_fwd(3, frag_lens, window, slope, heads, d, qk_dtype, "e4m3", out_dtype=torch.bfloat16, scale=0.5)
    rows = sum(frag_lens)
    pin = lambda x: x.cpu().pin_memory()
    h = {n: pin(g[n]) for n in ("q8", "k8", "v8", "sq", "sk", "sv")}
    # host output inside a guard band: one row before and after, 8 columns to the right
    guard = torch.full((rows + 2, heads * d + 8), -7.0, dtype=torch.bfloat16).pin_memory()
    out_h = guard[1:rows + 1, :heads * d]
    lse_h = torch.zeros((heads, rows), dtype=torch.float32).pin_memory()
    out_dev = torch.zeros((rows, heads * d), dtype=torch.bfloat16, device=_dev())
    status = torch.zeros(1, dtype=torch.int32, device=_dev())
    staging = None
    for _ in range(2):  # the second call reuses the staging area and the library's streams
        staging = ops.att_fwd_host(cfg, h["q8"], h["k8"], h["v8"], h["sk"], mask, slope, heads, out_h, lse=lse_h, qk_scale=h["sq"],
                                   v_scale=h["sv"], slices=slices, staging=staging, status=status, out_device=out_dev)
        torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert np.array_equal(util.to_np(out_h.contiguous()), out_d)
    assert np.array_equal(util.to_np(out_dev), out_d)
    assert np.array_equal(lse_h.numpy(), lse_d)
    assert util.err_stats(out_d, ref["out"])[0] < util.OUT_MAX_ABS
    assert bool((guard[0] == -7.0).all()) and bool((guard[rows + 1] == -7.0).all()) and bool((guard[:, heads * d:] == -7.0).all())
    # too small a staging area is refused with a message, nothing is queued
    with pytest.raises(Exception):
        ops.att_fwd_host(cfg, h["q8"], h["k8"], h["v8"], h["sk"], mask, slope, heads, out_h, qk_scale=h["sq"], v_scale=h["sv"],
                         slices=slices, staging=staging[:1024], status=status)


@pytest.mark.parametrize("d,out_dtype,ragged", [(128, torch.bfloat16, False), (64, torch.float32, False), (64, torch.bfloat16, True)])
def test_fwd_extra_destinations_receive_the_same_rows(d, out_dtype, ragged):
    """tsa_att_fwd_to (the forward with its all-gather fused in) stores every output row to each destination it is given: here
    three more buffers of the same GPU stand in for the peers' (the multi-GPU bench passes peer pointers).  Bits equal to
    tsa_att_fwd, rows and columns around each destination untouched, also when a destination is only 16-byte aligned."""
    from tscale_b200 import ops
    frag_lens, heads, window, slope = [384, 200], 3, 128, 0.25
    out_ref, lse_ref, _, (g, mask, cfg, _, _, _) = _run_fwd(6, frag_lens, window, slope, heads, d, "e4m3", "e4m3", out_dtype=out_dtype, scale=0.5)
    rows, width = sum(frag_lens), heads * d
    pad = 8 if ragged else 16  # bf16: 8 columns = 16 bytes: rows of the copies are then 16- but not 32-byte aligned
    guards = [torch.full((rows + 2, width + pad), -3.0, dtype=out_dtype, device=_dev()) for _ in range(4)]
    views = [x[1:rows + 1, :width] for x in guards]
    status = torch.zeros(1, dtype=torch.int32, device=_dev())
    out, lse = ops.att_fwd(cfg, g["q8"], g["k8"], g["v8"], g["sk"], mask, slope, heads, qk_scale=g["sq"], v_scale=g["sv"], status=status,
                           out=views[0], out_copies=[views[1], views[2], (views[3].data_ptr(), views[3].stride(0) * views[3].element_size())])
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for x, v in zip(guards, views):
        assert np.array_equal(util.to_np(v.contiguous()), out_ref)
        assert bool((x[0] == -3.0).all()) and bool((x[rows + 1] == -3.0).all()) and bool((x[:, width:] == -3.0).all())
    assert np.array_equal(util.to_np(lse), lse_ref)
    # a single further destination is stored by the softmax threads themselves (three went through the forwarding warp)
    one = torch.full((rows, width), -3.0, dtype=out_dtype, device=_dev())
    ops.att_fwd(cfg, g["q8"], g["k8"], g["v8"], g["sk"], mask, slope, heads, qk_scale=g["sq"], v_scale=g["sv"], status=status,
                out=views[0], out_copies=[one])
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert np.array_equal(util.to_np(one), out_ref) and np.array_equal(util.to_np(views[0].contiguous()), out_ref)
    # the SIMT path has one destination only
    cfg.flags |= 1
    with pytest.raises(Exception):
        ops.att_fwd(cfg, g["q8"], g["k8"], g["v8"], g["sk"], mask, slope, heads, qk_scale=g["sq"], v_scale=g["sv"], status=status,
                    out=views[0], out_copies=[views[1]])


@pytest.mark.parametrize("d,window,slope", [(128, 128, 0.25), (64, 64, 0.0), (64, 0, 0.0)])
def test_fwd_fused_consumer_equals_attention_then_kv_product(d, window, slope):
    """tsa_att_fwd_kv (the forward with the consumer of its output fused in: KVProduct, code/gpt/compute/gpt_combiner.cuh:12-39)
    gives the output of tsa_att_fwd and the combiner input of tsa_kv_product on that output, bit for bit; the combiner input
    also equals the oracle's KVProduct of the same bf16 rows up to the bf16 rounding of the result; rows and columns around
    kv stay untouched (ragged last fragment)."""
    from tscale_b200 import ops
    frag_lens, heads, kv_mult = [384, 200], 3, 0.375
    out_ref, lse_ref, _, (g, mask, cfg, _, _, _) = _run_fwd(7, frag_lens, window, slope, heads, d, "e4m3", "e4m3", out_dtype=torch.bfloat16, scale=0.5)
    rows, width = sum(frag_lens), heads * d
    gen = torch.Generator(device="cpu").manual_seed(11)
    ck = torch.randn((rows, width), generator=gen).to(torch.bfloat16).to(_dev())
    guard = torch.full((rows + 2, 4 * width + 16), -3.0, dtype=torch.bfloat16, device=_dev())
    kv_view = guard[1:rows + 1, :4 * width]
    status = torch.zeros(1, dtype=torch.int32, device=_dev())
    out, lse, kv = ops.att_fwd(cfg, g["q8"], g["k8"], g["v8"], g["sk"], mask, slope, heads, qk_scale=g["sq"], v_scale=g["sv"], status=status,
                               combiner_k=ck, kv_mult=kv_mult, kv=kv_view)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert np.array_equal(util.to_np(out), out_ref) and np.array_equal(util.to_np(lse), lse_ref)
    alone = ops.kv_product(ck, out, heads, d, kv_mult=kv_mult)
    torch.cuda.synchronize()
    assert torch.equal(kv.contiguous(), alone)
    assert bool((guard[0] == -3.0).all()) and bool((guard[rows + 1] == -3.0).all()) and bool((guard[:, 4 * width:] == -3.0).all())
    want = O.kv_product(ck.float().cpu().numpy(), out.float().cpu().numpy(), heads) * kv_mult
    got = kv.float().cpu().numpy()
    assert np.max(np.abs(got - want)) <= 2.0 ** -8 * np.max(np.abs(want)) + 1e-30
    # what the fused form does not cover is refused, not computed some other way
    cfg32 = ops.make_cfg("e4m3", "e4m3", d, d, out_dtype=torch.float32)
    with pytest.raises(Exception):
        ops.att_fwd(cfg32, g["q8"], g["k8"], g["v8"], g["sk"], mask, slope, heads, qk_scale=g["sq"], v_scale=g["sv"], status=status, combiner_k=ck)


def test_fwd_head_groups_equal_single_head_calls():
    """The forward hands its work items out in groups of heads sized by the key / value bytes of one head; with 98304 key rows
    of 6 heads x 128 the groups are 5 + 1 heads (an incomplete last group).  Per-head work is independent, so the call over
    all heads must equal six single-head calls on the head's columns bit for bit (inputs generated and quantised on the
    device; the window-64 mask over 24 fragments of 4096 rows keeps it short)."""
    from tscale_b200 import ops
    heads, d, frag, nfrag, window = 6, 128, 4096, 24, 64
    rows = frag * nfrag
    gen = torch.Generator(device=_dev())
    gen.manual_seed(21)
    t = {}
    for nm in ("q", "k", "v"):
        x = torch.randn((rows, heads * d), generator=gen, device=_dev()) * 0.5
        t[nm], t["s" + nm] = ops.quant_rows(x, "absmax", "e4m3", d)
        del x
    mask = ops.Mask.window([frag] * nfrag, window)
    cfg = ops.make_cfg("e4m3", "e4m3", d, d, out_dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=_dev())
    out, lse = ops.att_fwd(cfg, t["q"], t["k"], t["v"], t["sk"], mask, 0.25, heads, qk_scale=t["sq"], v_scale=t["sv"], status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for h in range(heads):
        cols = slice(h * d, (h + 1) * d)
        o1, l1 = ops.att_fwd(cfg, t["q"][:, cols], t["k"][:, cols], t["v"][:, cols], t["sk"][h:h + 1], mask, 0.25, 1,
                             qk_scale=t["sq"][h:h + 1], v_scale=t["sv"][h:h + 1], status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert torch.equal(o1, out[:, cols]) and torch.equal(l1[0], lse[h]), "head %d" % h


def test_peer_scatter_copies_block_to_every_destination():
    """tsa_peer_scatter (one rank's part of the all-gather over peer memory, the library's own copy kernel): the rows of the
    source land in every destination, nothing else is touched; local buffers stand in for the peers'."""
    import ctypes
    from tscale_b200 import abi, ops
    rows, cols = 777, 384  # bf16: 768-byte rows
    src = torch.randn((rows, cols), device=_dev()).to(torch.bfloat16)
    guards = [torch.full((rows + 2, cols + 16), -5.0, dtype=torch.bfloat16, device=_dev()) for _ in range(3)]
    views = [g[1:rows + 1, :cols] for g in guards]
    dsts = (ops.Ptr2D * 3)(*[ops.p2d(v) for v in views])
    abi.check(abi.lib().tsa_peer_scatter(ops.p2d(src), dsts, 3, rows, cols * 2, 0, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    for g, v in zip(guards, views):
        assert torch.equal(v, src)
        assert bool((g[0] == -5.0).all()) and bool((g[rows + 1] == -5.0).all()) and bool((g[:, cols:] == -5.0).all())
    with pytest.raises(Exception):  # rows that are not 32-byte aligned are refused
        abi.check(abi.lib().tsa_peer_scatter(ops.p2d(src[:, 8:]), dsts, 3, rows, (cols - 8) * 2, 0, None))


@pytest.mark.parametrize("d", [64, 128])
def test_fwd_tcgen05_constant_scales(d):
    # the reference's call shape: constant query and value scales (QK_VEC_SCALE / V_VEC_SCALE), per-row key scale
    from tscale_b200 import ops
    frag_lens, heads, window, slope = [256, 128], 2, 0, 0.0
    length = sum(frag_lens)
    rng = np.random.default_rng(7)
    k = (rng.standard_normal((length, heads * d)) * 0.5).astype(np.float32)
    k8, sk, kd = util.quantize(k, "e4m3", d)
    # q and v are stored directly as e4m3 codes with a constant scale of 1/24
    qf = rng.standard_normal((length, heads * d)).astype(np.float32) * 8
    vf = rng.standard_normal((length, heads * d)).astype(np.float32) * 8
    enc = np.vectorize(lambda x: O.lib().oracle_f32_to_e4m3(float(x)))
    q8 = enc(qf).astype(np.uint8)
    v8 = enc(vf).astype(np.uint8)
    qd = O.e4m3_to_f32(q8) / 24.0
    vd = O.e4m3_to_f32(v8) / 24.0
    spans, ptr = O.window_spans(frag_lens, window)
    ref = O.att_fwd(qd, kd, vd, spans, ptr, heads, slope)
    cfg = ops.make_cfg("e4m3", "e4m3", d, d, out_dtype=torch.float32, qk_vec_scale=1 / 24.0, v_vec_scale=1 / 24.0)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(_dev())
    status = torch.zeros(1, dtype=torch.int32, device=_dev())
    out, lse = ops.att_fwd(cfg, t(q8), t(k8.view(np.uint8)), t(v8), t(sk), ops.Mask.window(frag_lens, window), slope, heads,
                           status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    out = util.to_np(out)
    mx, mean = util.err_stats(out, ref["out"])
    assert mx < util.OUT_MAX_ABS and mean < util.OUT_MEAN_ABS, util.describe(out, ref["out"])


def test_fwd_tcgen05_large_logits_rescale():
    # logits of several units so that the running floor(max) moves and the accumulator is rescaled
    out, lse, ref, _ = _run_fwd(2, [512], 0, 0.0, 2, 64, "e4m3", "e4m3", out_dtype=torch.float32, scale=2.5)
    assert ref["max_dp"].max() > 4
    # peaked softmax: a few e4m3-rounded weights (3 mantissa bits, like the reference's fp8 kernel) carry each row,
    # so the error is a few percent of the value range (|v| up to ~10 here) instead of being averaged out
    mx, mean = util.err_stats(out, ref["out"])
    vmax = float(np.abs(ref["out"]).max())
    assert mx < 0.06 * vmax and mean < 0.01 * vmax, util.describe(out, ref["out"])
    assert util.err_stats(lse, ref["lse"])[0] < 5e-3
    # the same data through the generic kernel (exact fp32 weights) pins the rescale logic itself
    out_g, lse_g, _, _ = _run_fwd(2, [512], 0, 0.0, 2, 64, "e4m3", "e4m3", out_dtype=torch.float32, scale=2.5, force_generic=True)
    assert util.err_stats(out_g, ref["out"])[0] < 1e-3
    assert util.err_stats(lse, lse_g)[0] < 5e-3


def test_fwd_tcgen05_ragged_and_multispan():
    # ragged length (not a multiple of 64), rows with no span, rows with two spans (two rounds)
    length = 300
    rows = []
    for i in range(length):
        if i % 7 == 0:
            rows.append([])
        elif i > 140 and i % 5 == 0:
            rows.append([(3, 40), (i - 20, i - 1)])
        else:
            rows.append([(max(0, i - 90), i - 1)] if i > 0 else [])
    spans, ptr = [], [0]
    for r in rows:
        spans.extend(r)
        ptr.append(len(spans))
    custom = (np.array(spans, dtype=np.int32).reshape(-1, 2), np.array(ptr, dtype=np.int32))
    for force in (True, False):
        out, lse, ref, _ = _run_fwd(3, [length], None, 0.25, 2, 64, "e4m3", "e4m3", out_dtype=torch.float32, scale=0.5,
                                    force_generic=force, custom=custom)
        mx, mean = util.err_stats(out, ref["out"])
        assert mx < util.OUT_MAX_ABS and mean < util.OUT_MEAN_ABS, (force, util.describe(out, ref["out"]))
        empty = [i for i, r in enumerate(rows) if not r]
        assert np.all(out[empty] == 0)


def test_fwd_matches_golden_fixture(golden_dir):
    # the reference's own output on a committed fixture, inputs int8-quantised here
    import os
    from tscale_b200 import ops
    z = np.load(os.path.join(golden_dir, "att_w64_slope05.npz"))
    heads, d = int(z["heads"]), z["q"].shape[1] // int(z["heads"])
    mask = ops.Mask.from_spans(z["spans"], z["span_ptr"])
    q8, sq, qd = util.quantize(z["q"], "i8", d)
    k8, sk, kd = util.quantize(z["k"], "i8", d)
    v8, sv, vd = util.quantize(z["v"], "i8", d)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(_dev())
    # int8 quantisation error of the inputs dominates: compare to the fp32 fixture loosely and to the
    # oracle on the same quantised inputs tightly
    ref_q = O.att_fwd(qd, kd, vd, z["spans"], z["span_ptr"], heads, float(z["slope"]))
    vmax = float(np.abs(ref_q["out"]).max())
    dev_in = [t(q8.view(np.uint8)), t(k8.view(np.uint8)), t(v8.view(np.uint8)), t(sk), t(sq), t(sv)]
    for force_generic, tol in ((False, 5e-3 * vmax), (True, 1e-4)):
        # default dispatch: tensor cores, two e4m3 terms per weight; generic kernels: exact fp32 weights
        cfg = ops.make_cfg("i8", "i8", d, d, out_dtype=torch.float32, force_generic=force_generic)
        out, lse = ops.att_fwd(cfg, dev_in[0], dev_in[1], dev_in[2], dev_in[3], mask, float(z["slope"]), heads,
                               qk_scale=dev_in[4], v_scale=dev_in[5])
        torch.cuda.synchronize()
        assert util.err_stats(util.to_np(out), ref_q["out"])[0] < tol, (force_generic, util.describe(util.to_np(out), ref_q["out"]))
        assert util.err_stats(util.to_np(out), z["out"])[1] < 2e-2


@pytest.mark.parametrize("window,slope,d", [(64, 0.5, 64), (0, 0.0, 128), (256, 0.0, 128)])
def test_bwd_against_oracle(window, slope, d):
    from tscale_b200 import ops
    frag_lens, heads = [256, 192], 2
    out, lse, ref, (g, mask, cfg, spans, ptr, (qd, kd, vd)) = _run_fwd(
        4, frag_lens, window, slope, heads, d, "i8", "e4m3", out_dtype=torch.float32, scale=0.5)
    rng = np.random.default_rng(5)
    d_out = (rng.standard_normal(out.shape) * 1e-2).astype(np.float32)
    gref = O.att_bwd(qd, kd, vd, d_out, spans, ptr, heads, slope, fwd=ref)
    cfg.grad_dtype = 4  # f32
    out_t = torch.from_numpy(ref["out"]).to(_dev())
    lse_t = torch.from_numpy(ref["lse"]).to(_dev())
    status = torch.zeros(1, dtype=torch.int32, device=_dev())
    dq, dk, dv = ops.att_bwd(cfg, g["q8"], g["k8"], g["v8"], g["sk"], torch.from_numpy(d_out).to(_dev()), out_t, lse_t,
                             mask, slope, heads, qk_scale=g["sq"], v_scale=g["sv"], status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for name, got in (("dq", dq), ("dk", dk), ("dv", dv)):
        r = util.rel_l2(util.to_np(got), gref[name])
        assert r < util.GRAD_REL_L2, (name, r)
    # the SIMT kernels (every head size, the path odd shapes take) against the same oracle
    cfg.flags |= 1
    dq, dk, dv = ops.att_bwd(cfg, g["q8"], g["k8"], g["v8"], g["sk"], torch.from_numpy(d_out).to(_dev()), out_t, lse_t,
                             mask, slope, heads, qk_scale=g["sq"], v_scale=g["sv"], status=status)
    torch.cuda.synchronize()
    for name, got in (("dq", dq), ("dk", dk), ("dv", dv)):
        r = util.rel_l2(util.to_np(got), gref[name])
        assert r < util.GRAD_REL_L2, ("generic " + name, r)


@pytest.mark.parametrize("d", [64, 128])
def test_bwd_bits_are_stable_from_run_to_run(d):
    """Both 64-column halves of a tile add into the same output accumulators and each half has its own MMA-issuing warp:
    the warps take turns, so the f32 sums see their terms in one order and repeated runs agree bit for bit."""
    from tscale_b200 import ops
    frag_lens, heads, slope = [1024, 640, 384], 4, 0.0
    out, lse, ref, (g, mask, cfg, _, _, _) = _run_fwd(9, frag_lens, 0, slope, heads, d, "i8", "e4m3", out_dtype=torch.float32, scale=0.5)
    cfg.grad_dtype = 4  # f32: no output rounding that could hide a difference
    gen = torch.Generator(device=_dev())
    gen.manual_seed(3)
    d_out = torch.randn(out.shape, generator=gen, device=_dev()) * 1e-2
    out_t, lse_t = torch.from_numpy(out).to(_dev()), torch.from_numpy(lse).to(_dev())
    status = torch.zeros(1, dtype=torch.int32, device=_dev())
    first = None
    for _ in range(6):
        res = ops.att_bwd(cfg, g["q8"], g["k8"], g["v8"], g["sk"], d_out, out_t, lse_t, mask, slope, heads, qk_scale=g["sq"],
                          v_scale=g["sv"], status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        if first is None:
            first = res
        else:
            for a, b in zip(first, res):
                assert torch.equal(a, b)


@pytest.mark.parametrize("d", [64, 128])
def test_bwd_ragged_and_multispan(d):
    """Backward on a ragged length with empty rows and rows of two spans: the tensor-core path (transposed spans from
    the library's own transpose) and the SIMT path against the oracle."""
    from tscale_b200 import ops
    length = 300
    rows = []
    for i in range(length):
        if i % 7 == 0:
            rows.append([])
        elif i > 140 and i % 5 == 0:
            rows.append([(3, 40), (i - 20, i - 1)])
        else:
            rows.append([(max(0, i - 90), i - 1)] if i > 0 else [])
    spans, ptr = [], [0]
    for r in rows:
        spans.extend(r)
        ptr.append(len(spans))
    custom = (np.array(spans, dtype=np.int32).reshape(-1, 2), np.array(ptr, dtype=np.int32))
    heads, slope = 2, 0.25
    out, lse, ref, (g, mask, cfg, spans_np, ptr_np, (qd, kd, vd)) = _run_fwd(
        7, [length], None, slope, heads, d, "i8", "e4m3", out_dtype=torch.float32, scale=0.5, custom=custom)
    rng = np.random.default_rng(8)
    d_out = (rng.standard_normal(out.shape) * 1e-2).astype(np.float32)
    gref = O.att_bwd(qd, kd, vd, d_out, spans_np, ptr_np, heads, slope, fwd=ref)
    cfg.grad_dtype = 4  # f32
    out_t = torch.from_numpy(ref["out"]).to(_dev())
    lse_t = torch.from_numpy(ref["lse"]).to(_dev())
    status = torch.zeros(1, dtype=torch.int32, device=_dev())
    for flags in (0, 1):
        cfg.flags = flags
        dq, dk, dv = ops.att_bwd(cfg, g["q8"], g["k8"], g["v8"], g["sk"], torch.from_numpy(d_out).to(_dev()), out_t, lse_t,
                                 mask, slope, heads, qk_scale=g["sq"], v_scale=g["sv"], status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        for name, got in (("dq", dq), ("dk", dk), ("dv", dv)):
            r = util.rel_l2(util.to_np(got), gref[name])
            assert r < util.GRAD_REL_L2, (flags, name, r)
        empty = [i for i, r in enumerate(rows) if not r]
        assert float(dq[empty].abs().max().item()) == 0


@pytest.mark.parametrize("d", [64, 128])
def test_int8_scores_bit_exact(d):
    from tscale_b200 import ops
    rng = np.random.default_rng(6)
    heads, lq, lk = 3, 200, 333
    q8 = rng.integers(-128, 128, (lq, heads * d)).astype(np.int8)
    k8 = rng.integers(-128, 128, (lk, heads * d)).astype(np.int8)
    ref = O.qk_int32(q8, k8, heads)
    status = torch.zeros(1, dtype=torch.int32, device=_dev())
    got = ops.qk_scores_i32(torch.from_numpy(q8).to(_dev()), torch.from_numpy(k8).to(_dev()), heads, d, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert np.array_equal(got.cpu().numpy(), ref)


@pytest.mark.parametrize("d", [64, 128])
def test_fwd_int8_accumulators_bit_exact_inside_forward(d):
    """The s32 tile the forward itself read from tensor memory (a key tile late enough that the K/V ring has wrapped
    and every barrier has changed phase), against the integer oracle."""
    import ctypes
    from tscale_b200 import abi, ops
    heads, seq = 2, 1024
    g, (qd, kd, vd) = _setup(11, [seq], heads, d, "i8", "e4m3", 0.5)
    mask = ops.Mask.window([seq], 0)
    cfg = ops.make_cfg("i8", "e4m3", d, d, out_dtype=torch.float32)
    head, q_tile, k_tile = 1, 7, 5
    dump = torch.full((128, 128), -7, dtype=torch.int32, device=_dev())
    status = torch.zeros(1, dtype=torch.int32, device=_dev())
    abi.check(abi.lib().tsa_att_fwd_set_score_dump(ctypes.c_void_p(dump.data_ptr()), head, q_tile, k_tile))
    try:
        ops.att_fwd(cfg, g["q8"], g["k8"], g["v8"], g["sk"], mask, 0.0, heads, qk_scale=g["sq"], v_scale=g["sv"], status=status)
        torch.cuda.synchronize()
    finally:
        abi.check(abi.lib().tsa_att_fwd_set_score_dump(None, 0, 0, 0))
    assert int(status.item()) == 0
    q8 = g["q8"].cpu().numpy().view(np.int8)[q_tile * 128:(q_tile + 1) * 128]
    k8 = g["k8"].cpu().numpy().view(np.int8)[k_tile * 128:(k_tile + 1) * 128]
    ref = O.qk_int32(np.ascontiguousarray(q8), np.ascontiguousarray(k8), heads)[head]
    assert np.array_equal(dump.cpu().numpy(), ref)
