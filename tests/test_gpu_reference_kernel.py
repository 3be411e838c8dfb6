"""The reference's own GPU attention kernel (Fp8Att, mma.sync, rebuilt for sm_100a behind oracle/ref_gpu_harness.cu)
against the CPU oracle and against this library's forward, on the same inputs.  Skipped where the harness library was
not built (it needs the reference checkout at build time)."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import util

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


@pytest.mark.parametrize("heads,length,window", [(1, 256, 0), (3, 1024, 0), (2, 512, 64)])
def test_reference_fp8att_matches_oracle_and_this_library(heads, length, window):
    if O.ref_gpu() is None:
        pytest.skip("oracle/_ref/libtsa_ref_gpu.so not built")
    from tscale_b200 import ops
    d = 128
    rng = np.random.default_rng(50 + heads)
    # the reference kernel's call shape: constant query and value scales (1/32), per-row key scale
    k = (rng.standard_normal((length, heads * d)) * 0.5).astype(np.float32)
    k8, sk, kd = util.quantize(k, "e4m3", d)
    enc = np.vectorize(lambda x: O.lib().oracle_f32_to_e4m3(float(x)))
    q8 = enc(rng.standard_normal((length, heads * d)).astype(np.float32) * 8).astype(np.uint8)
    v8 = enc(rng.standard_normal((length, heads * d)).astype(np.float32) * 8).astype(np.uint8)
    qd = O.e4m3_to_f32(q8) / 32.0
    vd = O.e4m3_to_f32(v8)           # stored-V units: the kernel returns sum w * v8 / sum w
    spans, ptr = O.window_spans([length], window)
    ref = O.att_fwd(qd, kd, vd, spans, ptr, heads, 0.0)

    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    q_t, k_t, v_t, sk_t = t(q8), t(k8.view(np.uint8)), t(v8), t(sk)
    mask = ops.Mask.window([length], window)
    groups, gptr, _, _ = mask.dev(DEV)
    out_ref = torch.zeros((length, heads * d), dtype=torch.float16, device=DEV)
    swl_ref = torch.zeros((heads, length), dtype=torch.float32, device=DEV)
    one = torch.ones(1, dtype=torch.float32, device=DEV)
    v_tr = v_t.t().contiguous()
    ms = O.ref_gpu_fp8_att(one, q_t, k_t, sk_t, v_tr, groups, gptr, 0.0, out_ref, swl_ref, heads, length, reps=1)
    torch.cuda.synchronize()
    assert ms > 0
    got_ref = out_ref.float().cpu().numpy()
    # the reference kernel keeps its scores in half precision and its weights in e4m3: a few percent of |v8| ~ 8
    vmax = float(np.abs(ref["out"]).max())
    assert np.abs(got_ref - ref["out"]).max() < 0.03 * vmax
    assert np.abs(got_ref - ref["out"]).mean() < 0.003 * vmax
    # its log-sum adds the e4m3-rounded weights (gpt_att_fp8.cuh:189-190): up to log2(1 + 2^-4) off where one key carries a row
    assert np.abs(swl_ref.cpu().numpy() - ref["lse"]).max() < 0.09

    cfg = ops.make_cfg("e4m3", "e4m3", d, d, out_dtype=torch.float16, qk_vec_scale=1 / 32.0, v_vec_scale=1.0)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out, lse = ops.att_fwd(cfg, q_t, k_t, v_t, sk_t, mask, 0.0, heads, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    got = out.float().cpu().numpy()
    assert np.abs(got - ref["out"]).max() < 0.03 * vmax and np.abs(got - ref["out"]).mean() < 0.003 * vmax
    assert np.abs(got - got_ref).mean() < 0.004 * vmax
