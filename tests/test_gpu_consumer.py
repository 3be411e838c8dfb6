"""GPU parity of the combiner input (tsa_kv_product) and its back-propagation against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import util

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


@pytest.mark.parametrize("d,heads", [(64, 12), (128, 5), (256, 1)])
def test_kv_product_f32_bit_exact(d, heads):
    from tscale_b200 import ops
    rng = np.random.default_rng(51)
    rows = 333
    k = rng.standard_normal((rows, heads * d)).astype(np.float32)
    val = rng.standard_normal((rows, heads * d)).astype(np.float32)
    want = O.kv_product(k, val, heads)
    got = ops.kv_product(torch.from_numpy(k).to(DEV), torch.from_numpy(val).to(DEV), heads, d).cpu().numpy()
    assert np.array_equal(got, want)
    dkv = rng.standard_normal((rows, heads * d * 4)).astype(np.float32)
    wk, wv, ws = O.kv_product_bwd(k, val, dkv, heads)
    gk, gv, gs = ops.kv_product_bwd(torch.from_numpy(k).to(DEV), torch.from_numpy(val).to(DEV), torch.from_numpy(dkv).to(DEV), heads, d)
    torch.cuda.synchronize()
    assert np.array_equal(gk.cpu().numpy(), wk) and np.array_equal(gv.cpu().numpy(), wv)
    assert np.allclose(gs.cpu().numpy(), ws, rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_kv_product_16bit(dt):
    from tscale_b200 import ops
    rng = np.random.default_rng(52)
    rows, heads, d = 257, 6, 128
    k = torch.from_numpy(rng.standard_normal((rows, heads * d)).astype(np.float32)).to(dt)
    val = torch.from_numpy(rng.standard_normal((rows, heads * d)).astype(np.float32)).to(dt)
    dkv = torch.from_numpy(rng.standard_normal((rows, heads * d * 4)).astype(np.float32)).to(dt)
    kf, vf, gf = k.float().numpy(), val.float().numpy(), dkv.float().numpy()
    got = ops.kv_product(k.to(DEV), val.to(DEV), heads, d, kv_mult=0.5)
    assert util.rel_l2(util.to_np(got), O.kv_product(kf, vf, heads) * 0.5) < 5e-3
    got32 = ops.kv_product(k.to(DEV), val.to(DEV), heads, d, out_dtype=torch.float32)
    assert np.array_equal(got32.cpu().numpy(), O.kv_product(kf, vf, heads))
    gk, gv, gs = ops.kv_product_bwd(k.to(DEV), val.to(DEV), dkv.to(DEV), heads, d)
    wk, wv, ws = O.kv_product_bwd(kf, vf, gf, heads)
    assert util.rel_l2(util.to_np(gk), wk) < 5e-3 and util.rel_l2(util.to_np(gv), wv) < 5e-3
    assert util.rel_l2(gs.cpu().numpy(), ws) < 1e-5


def test_dscale_of_the_consumer_feeds_the_attention_backward():
    """dScale from tsa_kv_product_bwd equals tsa_calc_dscale(valLookup, dValLookup): the attention backward can take it
    from the consumer's back-propagation instead of a separate pass."""
    from tscale_b200 import ops
    rng = np.random.default_rng(53)
    rows, heads, d = 300, 4, 64
    k = torch.from_numpy(rng.standard_normal((rows, heads * d)).astype(np.float32)).to(DEV)
    val = torch.from_numpy(rng.standard_normal((rows, heads * d)).astype(np.float32)).to(DEV)
    dkv = torch.from_numpy(rng.standard_normal((rows, heads * d * 4)).astype(np.float32)).to(DEV)
    _, dv, ds = ops.kv_product_bwd(k, val, dkv, heads, d)
    ds2 = ops.calc_dscale(val, dv, heads, d)
    torch.cuda.synchronize()
    assert torch.allclose(ds, ds2, rtol=1e-5, atol=1e-4)
