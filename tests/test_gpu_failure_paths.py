"""Failure paths and stray writes, without faulting or hanging the GPU.

* A bounded device wait that nobody satisfies gives up, reports through the status word and leaves the context usable
  (tsa_selftest_bounded_wait; the forward itself with one key-tile copy withheld).  The reference aborts the process on
  any CUDA error instead (code/lib/cuda/cuda_graph.cuh:147-150).
* Guard bands: outputs sit inside larger buffers filled with a byte pattern (rows before and after, columns to the
  right); nothing outside the output proper may change.  Input rows past the logical length hold poison and must not
  leak into any result.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import util

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
PATTERN = 0xA5


def test_bounded_wait_runs_out_and_reports():
    from tscale_b200 import abi
    lib = abi.lib()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    abi.check(lib.tsa_selftest_bounded_wait(200000, ctypes.c_void_p(status.data_ptr()), None))
    torch.cuda.synchronize()
    word = int(status.item())
    assert word == 0x10
    assert lib.tsa_status_from_word(word) == abi.TSA_TIMEOUT
    assert lib.tsa_status_from_word(0) == abi.TSA_OK
    # the context is still usable
    assert float(torch.ones(4, device=DEV).sum().item()) == 4.0


def test_forward_with_a_withheld_copy_times_out_cleanly_and_recovers():
    from tscale_b200 import abi, ops
    lib = abi.lib()
    heads, d, seq = 2, 64, 1024
    q, k, v = util.make_qkv(21, seq, heads, d, d, 0.5)
    q8, sq, qd = util.quantize(q, "e4m3", d)
    k8, sk, kd = util.quantize(k, "e4m3", d)
    v8, sv, vd = util.quantize(v, "e4m3", d)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    g = dict(q=t(q8.view(np.uint8)), k=t(k8.view(np.uint8)), v=t(v8.view(np.uint8)), sq=t(sq), sk=t(sk), sv=t(sv))
    mask = ops.Mask.window([seq], 0)
    cfg = ops.make_cfg("e4m3", "e4m3", d, d, out_dtype=torch.float32)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)

    def fwd():
        return ops.att_fwd(cfg, g["q"], g["k"], g["v"], g["sk"], mask, 0.0, heads, qk_scale=g["sq"], v_scale=g["sv"], status=status)

    # every CTA's second key tile never arrives; waits give up after about a millisecond
    abi.check(lib.tsa_selftest_fwd_withhold_copy(2000000, 1))
    try:
        fwd()
        torch.cuda.synchronize()
    finally:
        abi.check(lib.tsa_selftest_fwd_withhold_copy(0, -1))
    word = int(status.item())
    assert word & 0x30, hex(word)
    assert lib.tsa_status_from_word(word) == abi.TSA_TIMEOUT
    # the same call without the fault: correct results from the same context
    status.zero_()
    out, lse = fwd()
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    spans, ptr = O.window_spans([seq], 0)
    ref = O.att_fwd(qd, kd, vd, spans, ptr, heads, 0.0)
    mx, mean = util.err_stats(util.to_np(out), ref["out"])
    assert mx < util.OUT_MAX_ABS and mean < util.OUT_MEAN_ABS


def _banded(rows, cols, dtype, pad_rows=3, pad_cols=16):
    """A [rows][cols] view inside a larger buffer filled with the guard pattern; returns (view, whole buffer)."""
    whole = torch.empty((rows + 2 * pad_rows, cols + pad_cols), dtype=dtype, device=DEV)
    whole.view(torch.uint8).fill_(PATTERN)
    return whole[pad_rows:pad_rows + rows, :cols], whole


def _band_untouched(whole, rows, cols, pad_rows=3):
    raw = whole.view(torch.uint8)
    esz = whole.element_size()
    ok = bool((raw[:pad_rows] == PATTERN).all()) and bool((raw[pad_rows + rows:] == PATTERN).all())
    return ok and bool((raw[pad_rows:pad_rows + rows, cols * esz:] == PATTERN).all())


@pytest.mark.parametrize("qk_dtype,v_dtype,d,window,force_generic", [
    ("e4m3", "e4m3", 64, 64, False), ("e4m3", "e4m3", 128, 0, False), ("i8", "e4m3", 128, 256, False),
    ("i8", "i8", 64, 64, False), ("i8", "i8", 64, 64, True)])
def test_forward_writes_nothing_outside_its_outputs(qk_dtype, v_dtype, d, window, force_generic):
    from tscale_b200 import ops
    heads, frag_lens = 3, [300, 212]     # 512 rows of buffers, 512 logical rows; a ragged 300 + 212 split
    length, rows_alloc = sum(frag_lens), 640
    q, k, v = util.make_qkv(31, length, heads, d, d, 0.5)
    q8, sq, qd = util.quantize(q, qk_dtype, d)
    k8, sk, kd = util.quantize(k, qk_dtype, d)
    v8, sv, vd = util.quantize(v, v_dtype, d)

    def padded(b8):  # rows past the logical length hold poison bytes (0x7f: the largest int8 / an e4m3 NaN code)
        buf = torch.full((rows_alloc, heads * d), 0x7f, dtype=torch.uint8, device=DEV)
        buf[:length] = torch.from_numpy(np.ascontiguousarray(b8).view(np.uint8)).to(DEV)
        return buf[:length]

    def padded_scale(s):
        buf = torch.full((heads, rows_alloc), float("nan"), dtype=torch.float32, device=DEV)
        buf[:, :length] = torch.from_numpy(s).to(DEV)
        return buf[:, :length]

    out_dtype = torch.float32
    out, out_whole = _banded(length, heads * d, out_dtype)
    lse, lse_whole = _banded(heads, length, torch.float32, pad_rows=2, pad_cols=32)
    cfg = ops.make_cfg(qk_dtype, v_dtype, d, d, out_dtype=out_dtype, force_generic=force_generic)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.att_fwd(cfg, padded(q8), padded(k8), padded(v8), padded_scale(sk), ops.Mask.window(frag_lens, window), 0.25, heads,
                qk_scale=padded_scale(sq), v_scale=padded_scale(sv), out=out, lse=lse, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert _band_untouched(out_whole, length, heads * d)
    assert _band_untouched(lse_whole, heads, length, pad_rows=2)
    spans, ptr = O.window_spans(frag_lens, window)
    ref = O.att_fwd(qd, kd, vd, spans, ptr, heads, 0.25)
    got = util.to_np(out)
    assert np.isfinite(got).all()
    mx, mean = util.err_stats(got, ref["out"])
    assert mx < util.OUT_MAX_ABS and mean < util.OUT_MEAN_ABS, util.describe(got, ref["out"])


def test_backward_writes_nothing_outside_its_outputs():
    from tscale_b200 import abi, ops
    heads, d, frag_lens, window, slope = 2, 128, [256, 192], 0, 0.0
    length = sum(frag_lens)
    q, k, v = util.make_qkv(33, length, heads, d, d, 0.5)
    q8, sq, qd = util.quantize(q, "i8", d)
    k8, sk, kd = util.quantize(k, "i8", d)
    v8, sv, vd = util.quantize(v, "e4m3", d)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    spans, ptr = O.window_spans(frag_lens, window)
    ref = O.att_fwd(qd, kd, vd, spans, ptr, heads, slope)
    rng = np.random.default_rng(34)
    d_out = (rng.standard_normal(ref["out"].shape) * 1e-2).astype(np.float32)
    gref = O.att_bwd(qd, kd, vd, d_out, spans, ptr, heads, slope, fwd=ref)
    mask = ops.Mask.window(frag_lens, window)
    cfg = ops.make_cfg("i8", "e4m3", d, d, out_dtype=torch.float32, grad_dtype=torch.float32)
    bands = [_banded(length, heads * d, torch.float32) for _ in range(3)]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ws = torch.empty(max(1, abi.lib().tsa_att_bwd_workspace_bytes(ctypes.byref(cfg), heads, length)), dtype=torch.uint8, device=DEV)
    groups, gptr, rgroups, rgptr = mask.dev(DEV)
    p = ops.p2d
    # the device tensors stay referenced until the call has been synchronised
    dv_ = dict(q=t(q8.view(np.uint8)), k=t(k8.view(np.uint8)), sq=t(sq), sk=t(sk), v=t(v8.view(np.uint8)), sv=t(sv),
               d_out=t(d_out), out=t(ref["out"]), lse=t(ref["lse"]))
    abi.check(abi.lib().tsa_att_bwd(ctypes.byref(cfg), None, p(dv_["q"]), p(dv_["k"]), p(dv_["sq"]), p(dv_["sk"]),
                                    p(dv_["v"]), p(dv_["sv"]), p(dv_["d_out"]), p(dv_["out"]), p(None), p(dv_["lse"]),
                                    ctypes.c_void_p(groups.data_ptr()), ctypes.c_void_p(gptr.data_ptr()),
                                    ctypes.c_void_p(rgroups.data_ptr()), ctypes.c_void_p(rgptr.data_ptr()), slope, 1.0,
                                    p(bands[0][0]), p(bands[1][0]), p(bands[2][0]), heads, mask.len_att_tiles,
                                    ctypes.c_void_p(ws.data_ptr()), ws.numel(), ctypes.c_void_p(status.data_ptr()), None))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for (view, whole), name in zip(bands, ("dq", "dk", "dv")):
        assert _band_untouched(whole, length, heads * d), name
        assert util.rel_l2(util.to_np(view), gref[name]) < util.GRAD_REL_L2, name
