"""Torch-tensor front-end of the C ABI: builds tsa_ptr2d views of CUDA tensors and calls the library.

Names follow the reference's attention operators (code/gpt/compute/gpt_cuda.cu:445-564, 618-894):
qk = queries, qv = keys, v = values, per-head scale planes [H][len], grouped spans for the mask.
Everything runs on the GPU through libtsa_b200.so; torch only owns the memory and the stream.
"""
import ctypes

import numpy as np
import torch

from . import abi
from .abi import Ptr2D, check

_DT = {"i8": abi.TSA_I8, "e4m3": abi.TSA_E4M3, torch.float16: abi.TSA_F16, torch.bfloat16: abi.TSA_BF16,
       torch.float32: abi.TSA_F32}


def p2d(t, xsize=None, ysize=None):
    """tsa_ptr2d view of a 2-D tensor whose last dimension is contiguous (None -> absent argument)."""
    if t is None:
        return Ptr2D(None, 0, 0, 0)
    assert t.dim() == 2 and t.stride(1) == 1, "expected a row-major 2-D tensor"
    return Ptr2D(t.data_ptr(), t.stride(0) * t.element_size(), xsize or t.shape[1], ysize or t.shape[0])


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _np_ip(a):
    return a.ctypes.data_as(abi.c_int_p)


class Mask:
    """Attention mask in the grouped form the kernels take (TAttentionSpanGroup<64> records), for the
    mask itself and for its transpose.  Built on the host by the library's span helpers."""

    def __init__(self, length, groups, group_ptr, rev_groups, rev_group_ptr):
        self.len = length
        self.len_att_tiles = (length + abi.ATT_GROUP - 1) // abi.ATT_GROUP
        self.groups, self.group_ptr = groups, group_ptr          # numpy int32 [n][130], [tiles+1]
        self.rev_groups, self.rev_group_ptr = rev_groups, rev_group_ptr
        self._dev = {}

    @staticmethod
    def _run_grouper(fn, cap):
        while True:
            groups = np.zeros((max(cap, 1), 130), dtype=np.int32)
            n = fn(cap, groups)
            if n >= 0:
                return groups[:n].copy()
            cap = -n

    @classmethod
    def window(cls, frag_lens, window):
        """Causal window mask of concatenated fragments; window <= 0 means full causal."""
        L = abi.lib()
        fl = np.ascontiguousarray(frag_lens, dtype=np.int32)
        length = int(fl.sum())
        tiles = (length + abi.ATT_GROUP - 1) // abi.ATT_GROUP
        res = []
        for transposed in (0, 1):
            gptr = np.zeros(tiles + 1, dtype=np.int32)
            groups = cls._run_grouper(
                lambda cap, g: L.tsa_group_window_spans(len(fl), _np_ip(fl), int(window or 0), transposed, cap,
                                                        g.ctypes.data, _np_ip(gptr)), tiles + 1)
            res += [groups, gptr]
        return cls(length, *res)

    @classmethod
    def window_on_device(cls, frag_starts, length, window, device):
        """The same mask built by tsa_group_window_spans_device: frag_starts is an int32 CUDA tensor of fragment offsets
        (first 0, last = length); nothing is computed or copied on the host."""
        L = abi.lib()
        tiles = (length + abi.ATT_GROUP - 1) // abi.ATT_GROUP
        bufs = []
        for transposed in (0, 1):
            groups = torch.empty((max(tiles, 1), 130), dtype=torch.int32, device=device)
            gptr = torch.empty(tiles + 1, dtype=torch.int32, device=device)
            check(L.tsa_group_window_spans_device(_ptr(frag_starts), frag_starts.numel() - 1, length, int(window or 0), transposed,
                                                  max(tiles, 1), _ptr(groups), _ptr(gptr), _stream()))
            bufs += [groups, gptr]
        m = cls(length, None, None, None, None)
        m._dev[str(device)] = tuple(bufs)
        return m

    @classmethod
    def from_spans(cls, spans, span_ptr):
        """General mask from per-row inclusive spans in CSR form."""
        L = abi.lib()
        spans = np.ascontiguousarray(spans, dtype=np.int32).reshape(-1, 2)
        span_ptr = np.ascontiguousarray(span_ptr, dtype=np.int32)
        length = len(span_ptr) - 1
        tiles = (length + abi.ATT_GROUP - 1) // abi.ATT_GROUP
        cap = max(16, 2 * len(spans) + length)
        while True:
            rev = np.zeros((cap, 2), dtype=np.int32)
            rev_ptr = np.zeros(length + 1, dtype=np.int32)
            n = L.tsa_transpose_attention(length, _np_ip(spans), _np_ip(span_ptr), cap, _np_ip(rev), _np_ip(rev_ptr))
            if n >= 0:
                rev = rev[:n].copy()
                break
            cap = -n
        res = []
        for sp, pt in ((spans, span_ptr), (rev, rev_ptr)):
            gptr = np.zeros(tiles + 1, dtype=np.int32)
            groups = cls._run_grouper(
                lambda cap, g: L.tsa_group_attention(length, _np_ip(sp), _np_ip(pt), cap, g.ctypes.data, _np_ip(gptr)),
                tiles + 1)
            res += [groups, gptr]
        m = cls(length, *res)
        m.rev_spans, m.rev_span_ptr = rev, rev_ptr
        return m

    @classmethod
    def from_spans_device(cls, spans_dev, span_ptr_dev, max_rev_spans=None, max_groups=None):
        """General mask built entirely on the GPU from per-row inclusive spans that are already in device memory (int32
        CSR: spans [n][2], span_ptr [len + 1]; every row's spans sorted by start and disjoint): transpose, then group the
        mask and its transpose.  The capacities default to bounds that always suffice for causal masks; the device
        counters are read back once at the end to size the result views (the kernels themselves never wait for the host)."""
        L = abi.lib()
        dev = spans_dev.device
        length = span_ptr_dev.numel() - 1
        n_in = spans_dev.shape[0]
        tiles = (length + abi.ATT_GROUP - 1) // abi.ATT_GROUP
        cap_rev = max_rev_spans if max_rev_spans is not None else max(16, 2 * n_in + length)
        i32 = dict(dtype=torch.int32, device=dev)
        rev = torch.zeros((cap_rev, 2), **i32)
        rev_ptr = torch.zeros(length + 1, **i32)
        counts = torch.zeros((3, 2), **i32)
        ws = torch.empty(max(64, L.tsa_transpose_attention_device_workspace_bytes(length, n_in)), dtype=torch.uint8, device=dev)
        check(L.tsa_transpose_attention_device(length, _ptr(spans_dev), _ptr(span_ptr_dev), n_in, cap_rev, _ptr(rev), _ptr(rev_ptr),
                                               _ptr(counts[0]), _ptr(ws), ws.numel(), _stream()))
        gws = torch.empty(max(64, L.tsa_group_attention_device_workspace_bytes(length)), dtype=torch.uint8, device=dev)
        res = []
        for i, (sp, pt) in enumerate(((spans_dev, span_ptr_dev), (rev, rev_ptr))):
            cap = max_groups if max_groups is not None else max(16, 4 * tiles + 16)
            groups = torch.zeros((cap, ctypes.sizeof(abi.SpanGroup)), dtype=torch.uint8, device=dev)
            gptr = torch.zeros(tiles + 1, **i32)
            check(L.tsa_group_attention_device(length, _ptr(sp), _ptr(pt), cap, _ptr(groups), _ptr(gptr), _ptr(counts[1 + i]),
                                               _ptr(gws), gws.numel(), _stream()))
            res += [groups, gptr]
        c = counts.cpu().numpy()
        if c[:, 1].any():
            raise RuntimeError("from_spans_device: capacity too small (needed %d transposed spans, %d / %d groups)" % (c[0, 0], c[1, 0], c[2, 0]))
        m = cls(length, None, None, None, None)
        m._dev[str(dev)] = (res[0][:int(c[1, 0])], res[1], res[2][:int(c[2, 0])], res[3])
        m.rev_spans_dev, m.rev_span_ptr_dev, m.counts = rev[:int(c[0, 0])], rev_ptr, c
        return m

    def dev(self, device):
        key = str(device)
        if key not in self._dev:
            self._dev[key] = tuple(torch.from_numpy(np.ascontiguousarray(a)).to(device)
                                   for a in (self.groups, self.group_ptr, self.rev_groups, self.rev_group_ptr))
        return self._dev[key]


def quant_rows(src, kind, dst, tile, vec_scale=0.0, length=None):
    """Per-row, per-tile quantiser.  kind 'rms' | 'absmax'; dst 'i8' | 'e4m3'.
    Returns (bytes uint8 [rows][x], scale f32 [x/tile][rows])."""
    rows, xs = src.shape
    length = rows if length is None else length
    out = torch.empty((rows, xs), dtype=torch.uint8, device=src.device)
    scale = torch.empty((xs // tile, rows), dtype=torch.float32, device=src.device)
    check(abi.lib().tsa_quant_rows(abi.TSA_QUANT_RMS if kind == "rms" else abi.TSA_QUANT_ABSMAX, _DT[src.dtype], _DT[dst],
                                   vec_scale, p2d(src), p2d(out), p2d(scale), length, tile, _stream()))
    return out, scale


def norm_rope_quant(src, rope, dst, heads, head_dim, vec_scale=1.0, direction=1.0, length=None):
    """Per-head RMS normalise, rope (None: no rotation), quantise.  Returns (bytes uint8 [rows][H*D], scale f32 [H][rows])."""
    rows = src.shape[0]
    length = rows if length is None else length
    out = torch.empty((rows, heads * head_dim), dtype=torch.uint8, device=src.device)
    scale = torch.empty((heads, rows), dtype=torch.float32, device=src.device)
    check(abi.lib().tsa_norm_rope_quant(_DT[src.dtype], _DT[dst], vec_scale, p2d(src), p2d(rope),
                                        _DT[rope.dtype] if rope is not None else abi.TSA_F32, direction, p2d(out), p2d(scale),
                                        heads, head_dim, length, _stream()))
    return out, scale


def matmul_norm_rope_quant(x, w, rope, dst, heads, head_dim, vec_scale=1.0, src_scale=1.0, direction=1.0, length=None, status=None, src="i8"):
    """The projection x @ w^T fused with norm_rope_quant: x [rows][dim], w [H*D][dim] both int8 (exact int32 products) or both
    e4m3 bytes (src="e4m3", f32 accumulation), rope f32 [rows][D] or None; dst "i8" / "e4m3" (quantised bytes) or torch.float16 /
    torch.bfloat16 (the normalised, rotated values).  Returns (out [rows][H*D], scale f32 [H][rows])."""
    rows = x.shape[0]
    length = rows if length is None else length
    out = torch.empty((rows, heads * head_dim), dtype=torch.uint8 if isinstance(dst, str) else dst, device=x.device)
    scale = torch.empty((heads, rows), dtype=torch.float32, device=x.device)
    check(abi.lib().tsa_matmul_norm_rope_quant(_DT[src], _DT[dst], vec_scale, src_scale, p2d(x), p2d(w), p2d(rope), direction, p2d(out), p2d(scale),
                                               heads, head_dim, length, _ptr(status), _stream()))
    return out, scale


def rope_norm_bwd(src, grad, rope, heads, head_dim, direction=1.0):
    """Gradient with respect to the raw projections given the gradient with respect to the roped unit-RMS vectors."""
    out = torch.empty_like(grad)
    check(abi.lib().tsa_rope_norm_bwd(_DT[src.dtype], _DT[grad.dtype], p2d(src), p2d(grad), p2d(rope),
                                      _DT[rope.dtype] if rope is not None else abi.TSA_F32, direction, p2d(out), heads, head_dim,
                                      src.shape[0], _stream()))
    return out


def kv_product(k, val, heads, head_dim, kv_mult=1.0, out_dtype=None, out=None):
    """Combiner input [rows][H*D*4] from k and the attention output."""
    out_dtype = (k.dtype if out is None else out.dtype) if out_dtype is None else out_dtype
    if out is None:
        out = torch.empty((k.shape[0], heads * head_dim * 4), dtype=out_dtype, device=k.device)
    check(abi.lib().tsa_kv_product(_DT[k.dtype], _DT[out_dtype], p2d(k), p2d(val), kv_mult, p2d(out), heads, head_dim, k.shape[0], _stream()))
    return out


def kv_product_bwd(k, val, dkv, heads, head_dim):
    """Returns (dK, dVal [rows][H*D] of dkv's dtype, dScale f32 [H][rows])."""
    rows = k.shape[0]
    dk = torch.empty((rows, heads * head_dim), dtype=dkv.dtype, device=k.device)
    dv = torch.empty_like(dk)
    ds = torch.empty((heads, rows), dtype=torch.float32, device=k.device)
    check(abi.lib().tsa_kv_product_bwd(_DT[k.dtype], _DT[dkv.dtype], p2d(k), p2d(val), p2d(dkv), p2d(dk), p2d(dv), p2d(ds),
                                       heads, head_dim, rows, _stream()))
    return dk, dv, ds


def make_cfg(qk_dtype, v_dtype, head_dim_qk, head_dim_v, out_dtype=torch.bfloat16, grad_dtype=torch.bfloat16,
             qk_vec_scale=1.0, v_vec_scale=1.0, force_generic=False):
    return abi.AttCfg(_DT[qk_dtype], _DT[v_dtype], _DT[out_dtype], _DT[grad_dtype], head_dim_qk, head_dim_v,
                      qk_vec_scale, v_vec_scale, abi.TSA_FLAG_FORCE_GENERIC if force_generic else 0)


def att_fwd(cfg, qk, qv, v, qv_scale, mask, slope, heads, qk_scale=None, v_scale=None, global_scale=None,
            out=None, lse=None, workspace=None, status=None, out_copies=None, combiner_k=None, kv_mult=1.0, kv=None):
    """Forward.  Returns (out [len][H*Dv], sumWeightLog f32 [H][len]).  out_copies: further destinations of the output rows,
    either tensors or (data_ptr, stride_bytes) pairs for buffers of other GPUs mapped into this process (tsa_att_fwd_to).
    combiner_k (bf16 [len][H*D]): the kernel also forms the combiner input kv (bf16 [len][4*H*D], tsa_att_fwd_kv) and the
    call returns (out, sumWeightLog, kv)."""
    L = abi.lib()
    dev = qk.device
    rows = qk.shape[0]
    out_t = {abi.TSA_F16: torch.float16, abi.TSA_BF16: torch.bfloat16, abi.TSA_F32: torch.float32}[cfg.out_dtype]
    if out is None:
        out = torch.empty((rows, heads * cfg.head_dim_v), dtype=out_t, device=dev)
    if lse is None:
        lse = torch.empty((heads, rows), dtype=torch.float32, device=dev)
    if workspace is None:
        workspace = torch.empty(max(1, L.tsa_att_fwd_workspace_bytes(ctypes.byref(cfg), heads, rows)), dtype=torch.uint8, device=dev)
    groups, gptr, _, _ = mask.dev(dev)
    if combiner_k is not None:
        if out_copies:
            raise ValueError("att_fwd: out_copies and combiner_k exclude each other")
        if kv is None:
            kv = torch.empty((rows, 4 * heads * cfg.head_dim_v), dtype=torch.bfloat16, device=dev)
        check(L.tsa_att_fwd_kv(ctypes.byref(cfg), _ptr(global_scale), p2d(qk), p2d(qv), p2d(qk_scale), p2d(qv_scale),
                               p2d(v), p2d(v_scale), _ptr(groups), _ptr(gptr), slope, p2d(out), p2d(lse), p2d(combiner_k),
                               kv_mult, p2d(kv), heads, mask.len_att_tiles, _ptr(workspace), workspace.numel(), _ptr(status),
                               _stream()))
        return out, lse, kv
    if out_copies:
        outs = (Ptr2D * (1 + len(out_copies)))()
        outs[0] = p2d(out)
        for i, c in enumerate(out_copies):
            outs[1 + i] = p2d(c) if isinstance(c, torch.Tensor) else Ptr2D(int(c[0]), int(c[1]), out.shape[1], out.shape[0])
        check(L.tsa_att_fwd_to(ctypes.byref(cfg), _ptr(global_scale), p2d(qk), p2d(qv), p2d(qk_scale), p2d(qv_scale),
                               p2d(v), p2d(v_scale), _ptr(groups), _ptr(gptr), slope, outs, len(outs), p2d(lse), heads,
                               mask.len_att_tiles, _ptr(workspace), workspace.numel(), _ptr(status), _stream()))
        return out, lse
    check(L.tsa_att_fwd(ctypes.byref(cfg), _ptr(global_scale), p2d(qk), p2d(qv), p2d(qk_scale), p2d(qv_scale),
                        p2d(v), p2d(v_scale), _ptr(groups), _ptr(gptr), slope, p2d(out), p2d(lse), heads,
                        mask.len_att_tiles, _ptr(workspace), workspace.numel(), _ptr(status), _stream()))
    return out, lse


def att_fwd_host(cfg, qk, qv, v, qv_scale, mask, slope, heads, out, lse=None, qk_scale=None, v_scale=None, global_scale=None,
                 slices=4, staging=None, status=None, device=None, out_device=None):
    """Forward on page-locked HOST tensors (qk, qv, v, the scale planes, out and lse on the CPU, pinned): head slices are
    copied in, computed and copied out concurrently by the library.  Asynchronous: synchronise the current stream before
    reading `out`.  out_device: optional CUDA tensor [len][H*Dv] that also keeps the result.  Returns the staging tensor
    so that the caller can pass it again."""
    L = abi.lib()
    dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
    rows = qk.shape[0]
    need = L.tsa_att_fwd_host_staging_bytes(ctypes.byref(cfg), heads, rows, slices)
    if staging is None:
        staging = torch.empty(need, dtype=torch.uint8, device=dev)
    groups, gptr, _, _ = mask.dev(dev)
    check(L.tsa_att_fwd_host(ctypes.byref(cfg), _ptr(global_scale), p2d(qk), p2d(qv), p2d(qk_scale), p2d(qv_scale),
                             p2d(v), p2d(v_scale), _ptr(groups), _ptr(gptr), slope, p2d(out), p2d(lse), p2d(out_device),
                             heads, mask.len_att_tiles, slices, _ptr(staging), staging.numel(), _ptr(status), _stream()))
    return staging


def att_bwd(cfg, qk, qv, v, qv_scale, d_out, out, lse, mask, slope, heads, qk_scale=None, v_scale=None,
            global_scale=None, d_scale=None, grad_mult=1.0, workspace=None, status=None):
    """Backward.  Returns (dQK, dQV, dV) with respect to the true-scale vectors."""
    L = abi.lib()
    dev = qk.device
    rows = qk.shape[0]
    gt = {abi.TSA_F16: torch.float16, abi.TSA_BF16: torch.bfloat16, abi.TSA_F32: torch.float32}[cfg.grad_dtype]
    dq = torch.empty((rows, heads * cfg.head_dim_qk), dtype=gt, device=dev)
    dk = torch.empty((rows, heads * cfg.head_dim_qk), dtype=gt, device=dev)
    dv = torch.empty((rows, heads * cfg.head_dim_v), dtype=gt, device=dev)
    if workspace is None:
        workspace = torch.empty(max(1, L.tsa_att_bwd_workspace_bytes(ctypes.byref(cfg), heads, rows)), dtype=torch.uint8, device=dev)
    groups, gptr, rgroups, rgptr = mask.dev(dev)
    check(L.tsa_att_bwd(ctypes.byref(cfg), _ptr(global_scale), p2d(qk), p2d(qv), p2d(qk_scale), p2d(qv_scale),
                        p2d(v), p2d(v_scale), p2d(d_out), p2d(out), p2d(d_scale), p2d(lse),
                        _ptr(groups), _ptr(gptr), _ptr(rgroups), _ptr(rgptr), slope, grad_mult,
                        p2d(dq), p2d(dk), p2d(dv), heads, mask.len_att_tiles,
                        _ptr(workspace), workspace.numel(), _ptr(status), _stream()))
    return dq, dk, dv


def calc_dscale(out, d_out, heads, head_dim_v):
    rows = out.shape[0]
    res = torch.empty((heads, rows), dtype=torch.float32, device=out.device)
    check(abi.lib().tsa_calc_dscale(_DT[out.dtype], _DT[d_out.dtype], p2d(out), p2d(d_out), p2d(res), heads, head_dim_v,
                                    rows, _stream()))
    return res


def qk_scores_i32(qk, qv, heads, head_dim, status=None):
    """Raw int32 QK^T scores [H][lenQ][lenK] from the tcgen05 kind::i8 path."""
    len_q, len_k = qk.shape[0], qv.shape[0]
    res = torch.empty((heads, len_q, len_k), dtype=torch.int32, device=qk.device)
    check(abi.lib().tsa_qk_scores_i32(p2d(qk), p2d(qv), heads, head_dim, len_q, len_k, _ptr(res), _ptr(status), _stream()))
    return res


class KVCache:
    """Caller-owned int8 KV cache of nSeq sequences (the reference's TAttentionVecHistory,
    code/gpt/train/cpu_infer.cpp:397-410), one contiguous [capacity][H*D] block per sequence."""

    def __init__(self, n_seq, capacity, heads, head_dim, device, scale_dtype=torch.float16, out_dtype=torch.float32,
                 qk_vec_scale=1.0):
        self.n_seq, self.capacity, self.heads, self.head_dim = n_seq, capacity, heads, head_dim
        row = heads * head_dim
        self.k = torch.zeros((n_seq, capacity, row), dtype=torch.int8, device=device)
        self.v = torch.zeros((n_seq, capacity, row), dtype=torch.int8, device=device)
        self.k_scale = torch.zeros((n_seq, capacity, heads), dtype=scale_dtype, device=device)
        self.v_scale = torch.zeros((n_seq, capacity, heads), dtype=scale_dtype, device=device)
        self.ctx_lens = torch.zeros(n_seq, dtype=torch.int32, device=device)
        table = np.zeros((n_seq, 4), dtype=np.uint64)
        for s in range(n_seq):
            table[s] = (self.k[s].data_ptr(), self.v[s].data_ptr(), self.k_scale[s].data_ptr(), self.v_scale[s].data_ptr())
        self.seqs = torch.from_numpy(table.view(np.int64)).to(device)
        self.cfg = abi.DecodeCfg(head_dim, _DT[scale_dtype], _DT[out_dtype], qk_vec_scale)
        self.out_dtype = out_dtype
        self.workspace = None
        self.max_ctx = 0

    def append(self, k_new, k_scale_new, v_new, v_scale_new, status=None):
        check(abi.lib().tsa_kv_append(ctypes.byref(self.cfg), _ptr(self.seqs), _ptr(self.ctx_lens), self.n_seq, self.capacity,
                                      p2d(k_new), p2d(k_scale_new), p2d(v_new), p2d(v_scale_new), self.heads,
                                      _ptr(status), _stream()))
        self.max_ctx = min(self.capacity, self.max_ctx + 1)

    def decode(self, q, q_scale, window, slope, out=None, status=None):
        L = abi.lib()
        if out is None:
            out = torch.empty((self.n_seq, self.heads * self.head_dim), dtype=self.out_dtype, device=q.device)
        need = L.tsa_att_decode_workspace_bytes(ctypes.byref(self.cfg), self.n_seq, self.heads, self.capacity)
        if self.workspace is None or self.workspace.numel() < need:
            self.workspace = torch.empty(max(1, need), dtype=torch.uint8, device=q.device)
        check(L.tsa_att_decode(ctypes.byref(self.cfg), _ptr(self.seqs), _ptr(self.ctx_lens), self.n_seq, self.max_ctx,
                               p2d(q), p2d(q_scale), window, slope, p2d(out), self.heads,
                               _ptr(self.workspace), self.workspace.numel(), _ptr(status), _stream()))
        return out

    def decode_static(self, q, q_scale, window, slope, out=None, status=None):
        """The same step through tsa_att_decode_static: no workspace, the library's built-in scratch array."""
        if out is None:
            out = torch.empty((self.n_seq, self.heads * self.head_dim), dtype=self.out_dtype, device=q.device)
        check(abi.lib().tsa_att_decode_static(ctypes.byref(self.cfg), _ptr(self.seqs), _ptr(self.ctx_lens), self.n_seq,
                                              self.max_ctx, p2d(q), p2d(q_scale), window, slope, p2d(out), self.heads,
                                              _ptr(status), _stream()))
        return out
