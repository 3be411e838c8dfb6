"""GPU parity of the per-row quantisers, dScale and the KV-cache decode step, through the C ABI."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import util

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("dst", ["i8", "e4m3"])
@pytest.mark.parametrize("tile", [64, 128])
def test_quant_absmax_bit_exact(dst, tile):
    from tscale_b200 import ops
    rng = np.random.default_rng(0)
    x = (rng.standard_normal((300, 4 * tile)) * rng.uniform(0.01, 30, (300, 1))).astype(np.float32)
    x[5] = 0            # all-zero row: scale 0, zeros
    x[6, :tile] = 0     # one all-zero tile
    b_ref, s_ref = O.quant_rows("absmax", dst, 0.0, x, tile)
    b, s = ops.quant_rows(torch.from_numpy(x).to(DEV), "absmax", dst, tile)
    assert np.array_equal(s.cpu().numpy(), s_ref)
    assert np.array_equal(b.cpu().numpy().view(np.int8), b_ref)


@pytest.mark.parametrize("dst", ["i8", "e4m3"])
@pytest.mark.parametrize("src_dtype", [torch.float32, torch.bfloat16])
def test_quant_rms(dst, src_dtype):
    from tscale_b200 import ops
    rng = np.random.default_rng(1)
    x = torch.from_numpy(rng.standard_normal((257, 512)).astype(np.float32)).to(src_dtype)
    xf = x.float().numpy()
    b_ref, s_ref = O.quant_rows("rms", dst, 1 / 24.0, xf, 128)
    b, s = ops.quant_rows(x.to(DEV), "rms", dst, 128, vec_scale=1 / 24.0)
    s = s.cpu().numpy()
    # the sum of squares is reduced in a different order than the sequential CPU loop: scales agree to
    # a few ulp, bytes agree except where x/scale sits on a rounding boundary (then they differ by one code)
    assert np.allclose(s, s_ref, rtol=1e-6, atol=0)
    got = O.dequant(b.cpu().numpy(), dst)
    want = O.dequant(b_ref, dst)
    mism = got != want
    assert mism.mean() < 1e-3
    step = np.maximum(np.abs(want), 1.0) * (0.126 if dst == "e4m3" else 0.0) + 1.0
    assert np.all(np.abs(got - want)[mism] <= step[mism])


def test_quant_padding_rows_zeroed():
    from tscale_b200 import ops
    x = torch.randn(256, 128, device=DEV)
    b, s = ops.quant_rows(x, "absmax", "i8", 128, length=200)
    assert int(b[200:].abs().sum().item()) == 0 and float(s[:, 200:].abs().sum().item()) == 0


def test_dscale():
    from tscale_b200 import ops
    rng = np.random.default_rng(2)
    out = rng.standard_normal((333, 6 * 64)).astype(np.float32)
    d_out = rng.standard_normal((333, 6 * 64)).astype(np.float32)
    ref = O.dscale(out, d_out, 6)
    got = ops.calc_dscale(torch.from_numpy(out).to(DEV), torch.from_numpy(d_out).to(DEV), 6, 64).cpu().numpy()
    assert np.allclose(got, ref, rtol=1e-5, atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("heads,d", [(6, 64), (3, 128), (5, 32)])
def test_dscale_16bit_vector_path(dt, heads, d):
    """16-bit out / dOut take the 16-byte-load kernel; the oracle sees the same rounded values."""
    from tscale_b200 import ops
    rng = np.random.default_rng(12)
    out_t = torch.from_numpy(rng.standard_normal((333, heads * d)).astype(np.float32)).to(dt)
    d_out_t = torch.from_numpy(rng.standard_normal((333, heads * d)).astype(np.float32)).to(dt)
    ref = O.dscale(out_t.float().numpy(), d_out_t.float().numpy(), heads)
    got = ops.calc_dscale(out_t.to(DEV), d_out_t.to(DEV), heads, d).cpu().numpy()
    assert np.allclose(got, ref, rtol=1e-4, atol=1e-4)


def _decode_case(seed, ctx_lens, heads, d, window, slope, steps=2, scale_dtype=torch.float16):
    from tscale_b200 import ops
    rng = np.random.default_rng(seed)
    n_seq = len(ctx_lens)
    cap = max(ctx_lens) + steps
    cache = ops.KVCache(n_seq, cap, heads, d, DEV, scale_dtype=scale_dtype, out_dtype=torch.float32)
    row = heads * d
    k_host = rng.integers(-127, 128, (n_seq, cap, row)).astype(np.int8)
    v_host = rng.integers(-127, 128, (n_seq, cap, row)).astype(np.int8)
    ks_host = (rng.random((n_seq, cap, heads)) * 2e-4 + 1e-4).astype(np.float16).astype(np.float32)
    vs_host = (rng.random((n_seq, cap, heads)) * 0.02 + 0.01).astype(np.float16).astype(np.float32)
    # pre-fill the caches with the existing context
    for s, n in enumerate(ctx_lens):
        cache.k[s, :n] = torch.from_numpy(k_host[s, :n]).to(DEV)
        cache.v[s, :n] = torch.from_numpy(v_host[s, :n]).to(DEV)
        cache.k_scale[s, :n] = torch.from_numpy(ks_host[s, :n]).to(DEV).to(scale_dtype)
        cache.v_scale[s, :n] = torch.from_numpy(vs_host[s, :n]).to(DEV).to(scale_dtype)
    cache.ctx_lens.copy_(torch.tensor(ctx_lens, dtype=torch.int32))
    cache.max_ctx = max(ctx_lens)
    lens = list(ctx_lens)
    for step in range(steps):
        q8 = rng.integers(-127, 128, (n_seq, row)).astype(np.int8)
        qs = (rng.random((n_seq, heads)) * 0.05 + 0.02).astype(np.float32)
        pos = np.array(lens)
        k_new = k_host[np.arange(n_seq), pos]
        v_new = v_host[np.arange(n_seq), pos]
        ks_new = ks_host[np.arange(n_seq), pos]
        vs_new = vs_host[np.arange(n_seq), pos]
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
        cache.append(t(k_new), t(ks_new).to(scale_dtype), t(v_new), t(vs_new).to(scale_dtype))
        lens = [n + 1 for n in lens]
        out = cache.decode(t(q8), t(qs), window, slope).cpu().numpy()
        assert cache.ctx_lens.cpu().tolist() == lens
        for s in range(n_seq):
            n = lens[s]
            ref = O.decode_step(k_host[s, :n], ks_host[s, :n], v_host[s, :n], vs_host[s, :n], q8[s], qs[s], heads, window,
                                slope, exp_mode="exact")
            scale = max(1.0, float(np.abs(ref).max()))
            assert np.abs(out[s] - ref).max() < 2e-4 * scale, (step, s, np.abs(out[s] - ref).max(), scale)


@pytest.mark.parametrize("d,heads", [(128, 16), (64, 12), (128, 3), (64, 4), (128, 8)])
def test_decode_wide(d, heads):
    _decode_case(3, [700, 1, 255, 256, 257, 1024], heads, d, 100000, 0.0)


def test_decode_window_alibi_and_self():
    _decode_case(4, [300, 70, 5], 4, 128, 64, 0.5)
    _decode_case(5, [300, 70, 5], 4, 64, 0, 0.0)      # width 0: the new token itself
    _decode_case(6, [40, 0], 2, 128, 64, 0.5)         # an empty sequence gets its first token


def test_decode_matches_reference_fixture(golden_dir):
    from tscale_b200 import ops
    z = np.load(os.path.join(golden_dir, "decode_w64.npz"))
    heads, width, slope = int(z["heads"]), int(z["width"]), float(z["slope"])
    kc, vc, ks, q8 = z["k_cache"], z["v_cache"], z["k_scale"], z["q8"]
    ctx, row = kc.shape
    d = row // heads
    vec_scale = float(z["vec_scale"])
    cache = ops.KVCache(1, ctx, heads, d, DEV, scale_dtype=torch.float32, out_dtype=torch.float32, qk_vec_scale=vec_scale)
    cache.k[0] = torch.from_numpy(kc).to(DEV)
    cache.v[0] = torch.from_numpy(vc).to(DEV)
    cache.k_scale[0] = torch.from_numpy(ks).to(DEV)
    cache.v_scale[0] = vec_scale
    cache.ctx_lens.fill_(ctx)
    cache.max_ctx = ctx
    out = cache.decode(torch.from_numpy(q8[None]).to(DEV), None, width, slope).cpu().numpy()[0]
    # the reference's polynomial 2^x is accurate to ~1e-4 relative; exact exp2 on the GPU
    assert np.abs(out - z["out"]).max() < 1e-3 * max(1.0, np.abs(z["out"]).max())


@pytest.mark.parametrize("frag_lens", [[4096] * 4, [1, 1, 1, 300, 1, 64, 63, 65, 129], [70], [5000, 3, 2049]])
@pytest.mark.parametrize("window", [0, 1, 64, 256])
def test_device_span_generation_equals_host(frag_lens, window):
    """tsa_group_window_spans_device writes the records the host helper computes, bit for bit, for the mask and its transpose."""
    from tscale_b200 import ops
    host = ops.Mask.window(frag_lens, window)
    length = sum(frag_lens)
    starts = torch.tensor(np.concatenate([[0], np.cumsum(frag_lens)]), dtype=torch.int32, device=DEV)
    dev = ops.Mask.window_on_device(starts, length, window, DEV)
    torch.cuda.synchronize()
    g, gp, rg, rgp = (x.cpu().numpy() for x in dev.dev(DEV))
    for got_g, got_p, want_g, want_p in ((g, gp, host.groups, host.group_ptr), (rg, rgp, host.rev_groups, host.rev_group_ptr)):
        assert np.array_equal(got_p, want_p)
        n = int(want_p[-1])
        assert np.array_equal(got_g[:n], want_g[:n])
