"""Decode through the entry point that takes no workspace (tsa_att_decode_static).

Some callers of this library fix their device memory at start-up and cannot allocate per call; for them the
decode keeps its chunk partials in an array built into the library.  This file checks, through the C ABI, that
the entry point gives the same result as tsa_att_decode with a caller workspace, on two calls in a row (the
built-in array is shared by all calls and still holds the first call's partials when the second one runs), and
that it refuses a problem larger than the array.  It is collected last so that a run stopping at the first
failure has already covered every other test; it also passes when run alone in a fresh process.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _filled_cache(seed, ctx_lens, heads, d):
    from tscale_b200 import ops
    rng = np.random.default_rng(seed)
    n_seq, cap = len(ctx_lens), max(ctx_lens)
    cache = ops.KVCache(n_seq, cap, heads, d, DEV, scale_dtype=torch.float16, out_dtype=torch.float32)
    cache.k.copy_(torch.from_numpy(rng.integers(-127, 128, tuple(cache.k.shape)).astype(np.int8)))
    cache.v.copy_(torch.from_numpy(rng.integers(-127, 128, tuple(cache.v.shape)).astype(np.int8)))
    cache.k_scale.copy_(torch.from_numpy((rng.random(tuple(cache.k_scale.shape)) * 2e-4 + 1e-4).astype(np.float16)))
    cache.v_scale.copy_(torch.from_numpy((rng.random(tuple(cache.v_scale.shape)) * 0.02 + 0.01).astype(np.float16)))
    cache.ctx_lens.copy_(torch.tensor(ctx_lens, dtype=torch.int32))
    cache.max_ctx = cap
    q = torch.from_numpy(rng.integers(-127, 128, (n_seq, heads * d)).astype(np.int8)).to(DEV)
    qs = torch.from_numpy((rng.random((n_seq, heads)) * 0.05 + 0.02).astype(np.float32)).to(DEV)
    return cache, q, qs


def test_static_scratch_decode_matches_workspace_decode_twice():
    # first call: long contexts fill many chunk slots; second call: a different, smaller problem reuses the
    # same array while the first call's partials are still in it
    for seed, ctx_lens, heads, d, window, slope in ((0, [1500, 700, 257, 3], 8, 128, 100000, 0.0),
                                                    (1, [300, 40], 12, 64, 64, 0.5)):
        cache, q, qs = _filled_cache(seed, ctx_lens, heads, d)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        want = cache.decode(q, qs, window, slope, status=status)
        got = cache.decode_static(q, qs, window, slope, status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0                           # no device-side complaint from either entry point
        scale = max(1.0, float(want.abs().max()))
        assert float((got - want).abs().max()) <= 2e-4 * scale   # tolerance of the decode parity tests
        assert torch.equal(got, want)                            # same kernels, same order: in fact identical
        # and against the CPU oracle directly, sequence by sequence (the cache already holds the token that attends)
        from oracle import oracle as O
        for s_i, n in enumerate(ctx_lens):
            ref = O.decode_step(cache.k[s_i, :n].cpu().numpy(), cache.k_scale[s_i, :n].float().cpu().numpy(),
                                cache.v[s_i, :n].cpu().numpy(), cache.v_scale[s_i, :n].float().cpu().numpy(),
                                q[s_i].cpu().numpy(), qs[s_i].cpu().numpy(), heads, window, slope)
            assert np.abs(got[s_i].cpu().numpy() - ref).max() <= 2e-4 * max(1.0, np.abs(ref).max())


def test_static_scratch_decode_rejects_oversized_problem():
    from tscale_b200 import abi, ops
    lib = abi.lib()
    cap = lib.tsa_att_decode_static_capacity_bytes()
    assert cap == 32 << 20
    cache, q, qs = _filled_cache(2, [16], 4, 128)
    cfg = cache.cfg
    n_seq, max_ctx, heads = 4096, 8192, 16   # far beyond the built-in array; rejected before any launch
    assert lib.tsa_att_decode_workspace_bytes(ctypes.byref(cfg), n_seq, heads, max_ctx) > cap
    big_q = abi.Ptr2D(q.data_ptr(), heads * 128, heads * 128, n_seq)
    big_out = abi.Ptr2D(q.data_ptr(), heads * 128 * 4, heads * 128, n_seq)
    rc = lib.tsa_att_decode_static(ctypes.byref(cfg), cache.seqs.data_ptr(), cache.ctx_lens.data_ptr(), n_seq, max_ctx,
                                   big_q, abi.Ptr2D(None, 0, 0, 0), 64, 0.0, big_out, heads, None, None)
    assert rc == abi.TSA_UNSUPPORTED
    assert b"built-in scratch" in lib.tsa_last_error()
