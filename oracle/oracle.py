"""TEST INFRASTRUCTURE, NOT PRODUCT CODE.

ctypes front-end of the CPU oracle (oracle/libtsa_oracle.so, our restatement of TScale's
attention path) and, when it has been built from a reference checkout, of the reference's own
CPU code (oracle/_ref/libtsa_ref.so).  Only tests/, __graft_entry__.smoke() and the CPU-baseline
legs of bench.py import this module.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_ORACLE_SO = os.path.join(_HERE, "libtsa_oracle.so")
_REF_SO = os.path.join(_HERE, "_ref", "libtsa_ref.so")
_REF_FAST_SO = os.path.join(_HERE, "_ref", "libtsa_ref_fast.so")
_REF_GPU_SO = os.path.join(_HERE, "_ref", "libtsa_ref_gpu.so")

c_int = ctypes.c_int
c_float = ctypes.c_float
_fp = ctypes.POINTER(ctypes.c_float)
_ip = ctypes.POINTER(ctypes.c_int)
_bp = ctypes.POINTER(ctypes.c_int8)


def build(reference=True):
    """Compile the oracle and, when the Makefile finds a reference checkout (its REF variable, which the environment
    may override), the two builds of the reference's own CPU code."""
    subprocess.run(["make", "-C", _HERE, "oracle"], check=True, stdout=subprocess.DEVNULL)
    if reference:
        subprocess.run(["make", "-C", _HERE, "ref", "ref_fast", "ref_gpu", "-j8"], check=True, stdout=subprocess.DEVNULL)


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(_fp)


def _i(a):
    a = np.ascontiguousarray(a, dtype=np.int32)
    return a, a.ctypes.data_as(_ip)


def _b(a):
    a = np.ascontiguousarray(a).view(np.int8)
    return a, a.ctypes.data_as(_bp)


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_ORACLE_SO):
            build(reference=False)
        _lib = ctypes.CDLL(_ORACLE_SO)
        _lib.oracle_e4m3_to_f32.restype = c_float
        _lib.oracle_e4m3_to_f32.argtypes = [c_int]
        _lib.oracle_f32_to_e4m3.argtypes = [c_float]
        _lib.oracle_f32_to_i8.argtypes = [c_float]
    return _lib


def _cpu_has(*flags):
    try:
        txt = open("/proc/cpuinfo").read()
    except OSError:
        return False
    line = next((l for l in txt.splitlines() if l.startswith("flags")), "")
    have = set(line.split())
    return all(f in have for f in flags)


_ref = {}


def ref(fast=False):
    """The reference's own CPU attention, or None when it was not built or this CPU cannot run it
    (the decode path uses AVX-VNNI intrinsics).  fast: the -O3 build with fused multiply-adds that the CPU
    baseline times (results differ from the parity build in the last bits)."""
    if fast not in _ref:
        path = _REF_FAST_SO if fast else _REF_SO
        if not os.path.exists(path) or not _cpu_has("avx2", "fma", "avx_vnni"):
            _ref[fast] = False
        else:
            r = ctypes.CDLL(path)
            r.ref_vec_scale.restype = c_float
            r.ref_e4m3_to_float.restype = c_float
            r.ref_float2i8.argtypes = [c_float]
            _ref[fast] = r
    return _ref[fast] or None


_ref_gpu = None


def ref_gpu():
    """The reference's own GPU attention kernel behind its finite harness (oracle/_ref/libtsa_ref_gpu.so), or None when
    it was not built.  Needs a GPU."""
    global _ref_gpu
    if _ref_gpu is None:
        if not os.path.exists(_REF_GPU_SO):
            _ref_gpu = False
        else:
            r = ctypes.CDLL(_REF_GPU_SO)
            vp = ctypes.c_void_p
            r.ref_gpu_fp8_att.argtypes = [vp, vp, c_int, vp, c_int, vp, c_int, vp, c_int, vp, c_int, vp, c_float,
                                          vp, c_int, vp, c_int, c_int, c_int, c_int, ctypes.POINTER(c_float), vp]
            _ref_gpu = r
    return _ref_gpu or None


def ref_gpu_fp8_att(global_scale, qk, qv, qv_scale, v_t, groups, group_ptr, slope, out, sum_weight_log, heads, length, reps=1):
    """Launches the reference's Fp8Att `reps` times on CUDA tensors (torch): qk, qv uint8 e4m3 [len][H*128]; qv_scale f32
    [H][len]; v_t uint8 [H*128][len] (V transposed); groups / group_ptr the grouped spans on the device; out float16
    [len][H*128]; sum_weight_log f32 [H][len]; global_scale f32 [1] on the device.  len must be a multiple of 128.
    Returns the mean milliseconds per launch.  The query scale is the harness constant 1/32 and the result is in
    stored-V units, as in the reference's own kernel test (code/gpt/compute/gpt_att.cu:21-25)."""
    assert length % 128 == 0
    ms = c_float(0)
    sb = lambda t: t.stride(0) * t.element_size()
    rc = ref_gpu().ref_gpu_fp8_att(global_scale.data_ptr(), qk.data_ptr(), sb(qk), qv.data_ptr(), sb(qv), qv_scale.data_ptr(), sb(qv_scale),
                                   v_t.data_ptr(), sb(v_t), groups.data_ptr(), groups.shape[0], group_ptr.data_ptr(), c_float(slope),
                                   out.data_ptr(), sb(out), sum_weight_log.data_ptr(), sb(sum_weight_log), heads, length, reps,
                                   ctypes.byref(ms), None)
    if rc != 0:
        raise RuntimeError("reference GPU kernel: CUDA error %d" % rc)
    return float(ms.value)


def set_threads(n):
    lib().oracle_set_threads(int(n))


# ------------------------------------------------------------------------------------------------
# 8-bit formats
E4M3_TABLE = None


def e4m3_table():
    """float value of each of the 256 e4m3 bytes (0x7f/0xff are NaN codes and map to +-480 here
    only so that the table stays finite; the quantisers never emit them)."""
    global E4M3_TABLE
    if E4M3_TABLE is None:
        E4M3_TABLE = np.array([lib().oracle_e4m3_to_f32(i) for i in range(256)], dtype=np.float32)
    return E4M3_TABLE


def e4m3_to_f32(a):
    return e4m3_table()[np.asarray(a).view(np.uint8)]


def dequant(a8, dtype):
    if dtype == "i8":
        return np.asarray(a8).view(np.int8).astype(np.float32)
    if dtype == "e4m3":
        return e4m3_to_f32(a8)
    raise ValueError(dtype)


def quant_rows(kind, dst, vec_scale, src, tile):
    """kind: 'rms' | 'absmax' | 'rms_clamp127'; dst: 'i8' | 'e4m3'.
    Returns (bytes [len][x] int8, scale [x/tile][len] f32)."""
    src, sp = _f(src)
    ln, xs = src.shape
    out = np.zeros((ln, xs), dtype=np.int8)
    scale = np.zeros((xs // tile, ln), dtype=np.float32)
    lib().oracle_quant_rows(
        {"rms": 0, "absmax": 1, "rms_clamp127": 2}[kind], {"i8": 0, "e4m3": 1}[dst], c_float(vec_scale),
        ln, xs, tile, sp, out.ctypes.data_as(_bp), scale.ctypes.data_as(_fp))
    return out, scale


# ------------------------------------------------------------------------------------------------
# producer of the attention inputs: normalise per head, rope, quantise
def fill_rope(width, max_len, use_ref=False):
    """Rope table [max_len][width] (rope.cpp:4-24): per 64-element block 32 cosines then 32 sines."""
    out = np.zeros((max_len, width), dtype=np.float32)
    (ref() if use_ref else lib()).__getattr__("ref_fill_rope" if use_ref else "oracle_fill_rope")(
        width, max_len, out.ctypes.data_as(_fp))
    return out


def apply_rope(rope, data, direction=1.0, use_ref=False):
    """Rotates a copy of data [len][dim] with rope [len][headDim] (rope.cpp:28-61)."""
    rope, rp = _f(rope)
    data = np.array(data, dtype=np.float32, order="C", copy=True)
    ln, dim = data.shape
    fn = ref().ref_apply_rope if use_ref else lib().oracle_apply_rope
    fn(rope.shape[1], ln, dim, c_float(direction), rp, data.ctypes.data_as(_fp))
    return data


def normalize_state_ref(src, heads):
    """The reference's fp32 NormalizeState (gpt_cpu.cpp:297-324): every head scaled to unit RMS."""
    src, sp = _f(src)
    out = np.zeros_like(src)
    ref().ref_normalize_state_f32(src.shape[0], src.shape[1], heads, sp, out.ctypes.data_as(_fp))
    return out


def norm_rope_quant(dst, vec_scale, src, rope, head_dim, direction=1.0):
    """Per-head RMS normalise, rope (None: no rotation), quantise.
    Returns (bytes [len][dim] int8, scale [dim/head_dim][len] f32, roped fp32 [len][dim])."""
    src, sp = _f(src)
    ln, dim = src.shape
    out = np.zeros((ln, dim), dtype=np.int8)
    scale = np.zeros((dim // head_dim, ln), dtype=np.float32)
    roped = np.zeros((ln, dim), dtype=np.float32)
    rp = None
    if rope is not None:
        rope, rp = _f(rope)
    lib().oracle_norm_rope_quant({"i8": 0, "e4m3": 1}[dst], c_float(vec_scale), ln, dim, head_dim, c_float(direction), sp, rp,
                                 out.ctypes.data_as(_bp), scale.ctypes.data_as(_fp), roped.ctypes.data_as(_fp))
    return out, scale, roped


def normalize_state_backward_ref(src, d_norm, heads):
    """The reference's NormalizeStateBackward (gpt_cpu.cpp:329-360)."""
    src, sp = _f(src)
    d_norm, dp = _f(d_norm)
    out = np.zeros_like(src)
    ref().ref_normalize_state_backward_f32(src.shape[0], src.shape[1], heads, sp, dp, out.ctypes.data_as(_fp))
    return out


def rope_norm_bwd(src, d_roped, rope, head_dim, direction=1.0):
    """Gradient with respect to the raw projections, given the gradient with respect to the roped unit-RMS vectors."""
    src, sp = _f(src)
    d_roped, dp = _f(d_roped)
    ln, dim = src.shape
    out = np.zeros((ln, dim), dtype=np.float32)
    rp = None
    if rope is not None:
        rope, rp = _f(rope)
    lib().oracle_rope_norm_bwd(ln, dim, head_dim, c_float(direction), sp, dp, rp, out.ctypes.data_as(_fp))
    return out

def kv_product(k, val, heads, use_ref=False):
    """Combiner input (gpt_cpu.cpp:191-216): [len][H*D*4]."""
    k, kp = _f(k)
    val, vp = _f(val)
    ln, dim = k.shape
    out = np.zeros((ln, dim * 4), dtype=np.float32)
    fn = ref().ref_kv_product if use_ref else lib().oracle_kv_product
    fn(ln, heads, dim // heads, kp, vp, out.ctypes.data_as(_fp))
    return out


def kv_product_bwd(k, val, dkv, heads, use_ref=False):
    """Back-propagation of kv_product: returns (dK, dVal [len][H*D], dScale [H][len])."""
    k, kp = _f(k)
    val, vp = _f(val)
    dkv, dp = _f(dkv)
    ln, dim = k.shape
    dk = np.zeros((ln, dim), dtype=np.float32)
    dv = np.zeros((ln, dim), dtype=np.float32)
    ds = np.zeros((heads, ln), dtype=np.float32)
    fn = ref().ref_kv_product_backprop if use_ref else lib().oracle_kv_product_bwd
    fn(ln, heads, dim // heads, kp, vp, dp, dk.ctypes.data_as(_fp), dv.ctypes.data_as(_fp), ds.ctypes.data_as(_fp))
    return dk, dv, ds

# ------------------------------------------------------------------------------------------------
# spans
def window_spans(frag_lens, window):
    """Causal window spans of TScale (att/sliding_window.cpp:80-87,211-222): row i of a fragment
    starting at f0 attends [max(f0, i - window), i - 1]; the row itself is excluded; the first row
    of a fragment has no span.  window <= 0 or None means the whole fragment prefix."""
    spans, ptr = [], [0]
    base = 0
    for fl in frag_lens:
        for i in range(base, base + fl):
            lo = base if not window or window <= 0 else max(base, i - window)
            if i - 1 >= lo:
                spans.append((lo, i - 1))
            ptr.append(len(spans))
        base += fl
    return np.array(spans, dtype=np.int32).reshape(-1, 2), np.array(ptr, dtype=np.int32)


def transpose_attention(spans, span_ptr, use_ref=False):
    spans, sp = _i(spans)
    span_ptr, pp = _i(span_ptr)
    ln = len(span_ptr) - 1
    fn = ref().ref_transpose_attention if use_ref else lib().oracle_transpose_attention
    cap = max(16, 2 * len(spans) + ln)
    while True:
        res = np.zeros((cap, 2), dtype=np.int32)
        rptr = np.zeros(ln + 1, dtype=np.int32)
        n = fn(ln, sp, pp, cap, res.ctypes.data_as(_ip), rptr.ctypes.data_as(_ip))
        if n >= 0:
            return res[:n].copy(), rptr
        cap = -n


def group_attention(spans, span_ptr, use_ref=False):
    """GroupAttention<64,128>: returns (groups [n][130] int32, group_ptr [ceil(len/64)+1])."""
    spans, sp = _i(spans)
    span_ptr, pp = _i(span_ptr)
    ln = len(span_ptr) - 1
    fn = ref().ref_group_attention_64_128 if use_ref else lib().oracle_group_attention_64_128
    cap = max(16, (ln + 63) // 64 * 2)
    while True:
        groups = np.zeros((cap, 130), dtype=np.int32)
        gptr = np.zeros((ln + 63) // 64 + 1, dtype=np.int32)
        n = fn(ln, sp, pp, cap, groups.ctypes.data_as(_ip), gptr.ctypes.data_as(_ip))
        if n >= 0:
            return groups[:n].copy(), gptr
        cap = -n


# ------------------------------------------------------------------------------------------------
# attention
def att_fwd(q, k, v, spans, span_ptr, heads, slope, global_scale=1.0, use_ref=False):
    """fp32 forward on true-scale vectors q,k [len][H*Dq], v [len][H*Dv].
    Returns dict(out, sum_weight [H][len], max_dp [H][len], lse [H][len])."""
    q, qp = _f(q)
    k, kp = _f(k)
    v, vp = _f(v)
    spans, sp = _i(spans)
    span_ptr, pp = _i(span_ptr)
    ln = q.shape[0]
    dq, dv = q.shape[1] // heads, v.shape[1] // heads
    out = np.zeros_like(v)
    sw = np.zeros((heads, ln), dtype=np.float32)
    mx = np.zeros((heads, ln), dtype=np.float32)
    if use_ref:
        # use_ref == "fast": the -O3 build that the CPU baseline times
        assert global_scale == 1.0
        ref(fast=(use_ref == "fast")).ref_att_fwd(ln, heads, dq, dv, c_float(slope), qp, kp, vp, sp, pp,
                          out.ctypes.data_as(_fp), sw.ctypes.data_as(_fp), mx.ctypes.data_as(_fp))
        lse = mx + np.log2(sw)
    else:
        lse = np.zeros((heads, ln), dtype=np.float32)
        lib().oracle_att_fwd(ln, heads, dq, dv, c_float(global_scale), c_float(slope), qp, kp, vp, sp, pp,
                             out.ctypes.data_as(_fp), sw.ctypes.data_as(_fp), mx.ctypes.data_as(_fp),
                             lse.ctypes.data_as(_fp))
    return dict(out=out, sum_weight=sw, max_dp=mx, lse=lse)


def dscale(out, d_out, heads):
    out, op = _f(out)
    d_out, dp = _f(d_out)
    ln = out.shape[0]
    res = np.zeros((heads, ln), dtype=np.float32)
    lib().oracle_dscale(ln, heads, out.shape[1] // heads, op, dp, res.ctypes.data_as(_fp))
    return res


def att_bwd(q, k, v, d_out, spans, span_ptr, heads, slope, global_scale=1.0, use_ref=False, fwd=None,
            rev=None):
    """fp32 backward.  Returns dict(dq, dk, dv, dscale)."""
    q, qp = _f(q)
    k, kp = _f(k)
    v, vp = _f(v)
    d_out, dop = _f(d_out)
    spans, sp = _i(spans)
    span_ptr, pp = _i(span_ptr)
    ln = q.shape[0]
    dq_, dv_ = q.shape[1] // heads, v.shape[1] // heads
    if fwd is None:
        fwd = att_fwd(q, k, v, spans, span_ptr, heads, slope, global_scale, use_ref=use_ref)
    ds = dscale(fwd["out"], d_out, heads)
    if rev is None:
        rev = transpose_attention(spans, span_ptr)
    rs, rsp = _i(rev[0])
    rp, rpp = _i(rev[1])
    dq = np.zeros_like(q)
    dk = np.zeros_like(k)
    dv = np.zeros_like(v)
    if use_ref:
        assert global_scale == 1.0
        ref().ref_att_bwd(ln, heads, dq_, dv_, c_float(slope), qp, kp, vp, dop, ds.ctypes.data_as(_fp),
                          sp, pp, rsp, rpp, dq.ctypes.data_as(_fp), dk.ctypes.data_as(_fp),
                          dv.ctypes.data_as(_fp))
    else:
        sw, swp = _f(fwd["sum_weight"])
        mx, mxp = _f(fwd["max_dp"])
        lib().oracle_att_bwd(ln, heads, dq_, dv_, c_float(global_scale), c_float(slope), qp, kp, vp, dop,
                             ds.ctypes.data_as(_fp), swp, mxp, sp, pp, rsp, rpp,
                             dq.ctypes.data_as(_fp), dk.ctypes.data_as(_fp), dv.ctypes.data_as(_fp))
    return dict(dq=dq, dk=dk, dv=dv, dscale=ds)


def qk_int32(q8, k8, heads):
    q8, qp = _b(q8)
    k8, kp = _b(k8)
    lq, lk = q8.shape[0], k8.shape[0]
    d = q8.shape[1] // heads
    s = np.zeros((heads, lq, lk), dtype=np.int32)
    lib().oracle_qk_int32(lq, lk, heads, d, qp, kp, s.ctypes.data_as(_ip))
    return s


def decode_step(k_cache, k_scale, v_cache, v_scale, q8, q_scale, heads, width, slope, exp_mode="exact",
                use_ref=False):
    """One decode step of one sequence; the cache already holds the new token (see tsa_oracle.cpp).
    k_cache, v_cache int8 [ctx][H*D]; k_scale, v_scale f32 [ctx][H]; q8 int8 [H*D]; q_scale f32 [H]."""
    k_cache, kp = _b(k_cache)
    v_cache, vp = _b(v_cache)
    k_scale, ksp = _f(k_scale)
    q8, qp = _b(q8)
    k_cache = k_cache.reshape(k_cache.shape[0], -1)
    ctx = k_cache.shape[0]
    d = k_cache.shape[1] // heads
    out = np.zeros(heads * d, dtype=np.float32)
    if use_ref:
        # the reference has constant q and v scales (VEC_SCALE)
        ref().ref_decode_step(ctx, heads, d, width, c_float(slope), kp, ksp, vp, qp, out.ctypes.data_as(_fp))
        return out
    v_scale, vsp = _f(v_scale)
    q_scale, qsp = _f(q_scale)
    lib().oracle_decode_step(ctx, heads, d, width, c_float(slope), 0 if exp_mode == "poly" else 1,
                             kp, ksp, vp, vsp, qp, qsp, out.ctypes.data_as(_fp))
    return out


# ------------------------------------------------------------------------------------------------
# one-token inference through the int8 model (cpu_infer.cpp:466-560)
def make_infer_model(seed, dim, head_dim, heads, relu_mult, vocab, label_count, widths_slopes):
    """Seeded random int8 model in the form of TCPUModelParams (cpu_infer.cpp:59-84): a dict of numpy arrays.
    widths_slopes: one (attention width, ALiBi slope) pair per layer."""
    rng = np.random.default_rng(seed)
    hs, relu_dim = heads * head_dim, heads * 128 * relu_mult

    def mat(rows, cols):
        return np.clip(np.rint(rng.standard_normal((rows, cols)) * 32), -127, 127).astype(np.int8)

    def scale():
        return np.float32(rng.uniform(0.5, 1.5) / 32)

    layers = []
    for width, slope in widths_slopes:
        layers.append(dict(qk=mat(hs, dim), qv=mat(hs, dim), k=mat(hs, dim), v=mat(hs, dim), combiner=mat(dim, hs * 4),
                           expand=mat(relu_dim, dim), contract=mat(dim, relu_dim), qv_scale=scale(), combiner_scale=scale(),
                           contract_scale=scale(), width=int(width), slope=float(slope)))
    return dict(dim=dim, head_dim=head_dim, heads=heads, relu_mult=relu_mult, vocab=vocab, label_count=label_count, layers=layers,
                label_embed=mat(label_count, dim), label_embed_scale=scale(), final_layer=mat(vocab, dim), final_layer_scale=scale(),
                bias=(rng.standard_normal(vocab) * 0.5).astype(np.float32))


class InferOracle:
    """One sequence stepping through the model: the restated oracle (use_ref=False) or the reference's own
    NCPUInfer::ComputePrediction (use_ref=True).  rope_len bounds the number of steps."""

    def __init__(self, model, rope_len, use_ref=False, exp_mode="exact"):
        self.model = model          # keeps the weight arrays alive: the C side holds pointers into them
        self.use_ref = use_ref
        self.vocab = model["vocab"]
        self._l = ref() if use_ref else lib()
        pre = "ref_infer_" if use_ref else "oracle_infer_"
        create = getattr(self._l, pre + "create")
        create.restype = ctypes.c_void_p
        self._step = getattr(self._l, pre + "step")
        self._free = getattr(self._l, pre + "free")
        names = ("qk", "qv", "k", "v", "combiner", "expand", "contract")
        n = len(model["layers"])
        mats = (ctypes.c_void_p * (7 * n))()
        for i, layer in enumerate(model["layers"]):
            for j, nm in enumerate(names):
                assert layer[nm].dtype == np.int8 and layer[nm].flags["C_CONTIGUOUS"]
                mats[i * 7 + j] = layer[nm].ctypes.data
        self._scalars = np.array([[l["qv_scale"], l["combiner_scale"], l["contract_scale"], l["width"], l["slope"]] for l in model["layers"]],
                                 dtype=np.float32)
        self._mats = mats
        self._h = ctypes.c_void_p(create(
            model["dim"], model["head_dim"], model["heads"], model["relu_mult"], model["vocab"], model["label_count"], n, int(rope_len),
            mats, self._scalars.ctypes.data_as(_fp), model["label_embed"].ctypes.data_as(_bp), c_float(model["label_embed_scale"]),
            model["final_layer"].ctypes.data_as(_bp), c_float(model["final_layer_scale"]), model["bias"].ctypes.data_as(_fp)))
        if not use_ref:
            self._l.oracle_infer_set_exp(self._h, 0 if exp_mode == "poly" else 1)

    def step(self, labels, want_logits=False):
        labels, lp = _i(labels)
        pred = np.zeros(self.vocab, dtype=np.float32)
        if self.use_ref:
            self._step(self._h, lp, len(labels), pred.ctypes.data_as(_fp))
            return pred
        logits = np.zeros(self.vocab, dtype=np.float32)
        self._step(self._h, lp, len(labels), pred.ctypes.data_as(_fp), logits.ctypes.data_as(_fp))
        return (pred, logits) if want_logits else pred

    def __del__(self):
        if getattr(self, "_h", None):
            self._free(self._h)
            self._h = None
