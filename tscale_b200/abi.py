"""ctypes binding of the C ABI in include/tsa.h (libtsa_b200.so).

The shared library is the product; this module only declares its entry points for Python callers
(tests, bench.py).  There is no Python or CPU implementation behind it: if the library has not been
built, importing this module raises.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# TSA_B200_LIB selects another build of the same ABI (the bounds-check build of the tests)
LIB_PATH = os.environ.get("TSA_B200_LIB") or os.path.join(_HERE, "libtsa_b200.so")

TSA_OK, TSA_BAD_ARG, TSA_UNSUPPORTED, TSA_CUDA_ERROR, TSA_TIMEOUT = range(5)
TSA_I8, TSA_E4M3, TSA_F16, TSA_BF16, TSA_F32 = range(5)
TSA_QUANT_RMS, TSA_QUANT_ABSMAX = 0, 1
TSA_FLAG_FORCE_GENERIC = 1
ATT_GROUP = 64
ATT_ALIGN = 128

c_int, c_float, c_void_p, c_size_t = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t
c_int_p = ctypes.POINTER(ctypes.c_int)


class Ptr2D(ctypes.Structure):
    """tsa_ptr2d"""
    _fields_ = [("data", c_void_p), ("stride_bytes", c_int), ("xsize", c_int), ("ysize", c_int)]


class SpanGroup(ctypes.Structure):
    """tsa_span_group"""
    _fields_ = [("Start", c_int), ("Finish", c_int), ("SpanStart", c_int * ATT_GROUP), ("SpanFinish", c_int * ATT_GROUP)]


class AttCfg(ctypes.Structure):
    """tsa_att_cfg"""
    _fields_ = [("qk_dtype", c_int), ("v_dtype", c_int), ("out_dtype", c_int), ("grad_dtype", c_int),
                ("head_dim_qk", c_int), ("head_dim_v", c_int), ("qk_vec_scale", c_float), ("v_vec_scale", c_float),
                ("flags", c_int)]


class KvSeq(ctypes.Structure):
    """tsa_kv_seq"""
    _fields_ = [("k", c_void_p), ("v", c_void_p), ("kScale", c_void_p), ("vScale", c_void_p)]


class DecodeCfg(ctypes.Structure):
    """tsa_decode_cfg"""
    _fields_ = [("head_dim", c_int), ("scale_dtype", c_int), ("out_dtype", c_int), ("qk_vec_scale", c_float)]


class InferDims(ctypes.Structure):
    """tsa_infer_dims"""
    _fields_ = [("dim", c_int), ("head_dim", c_int), ("head_count", c_int), ("relu_dim", c_int), ("vocab_size", c_int),
                ("label_count", c_int), ("layer_count", c_int)]


class InferLayer(ctypes.Structure):
    """tsa_infer_layer"""
    _fields_ = [("qk", c_void_p), ("qv", c_void_p), ("k", c_void_p), ("v", c_void_p), ("combiner", c_void_p),
                ("expand", c_void_p), ("contract", c_void_p), ("qv_scale", c_float), ("combiner_scale", c_float),
                ("contract_scale", c_float), ("attention_width", c_int), ("alibi_slope", c_float)]


class InferModel(ctypes.Structure):
    """tsa_infer_model"""
    _fields_ = [("dims", InferDims), ("layers", ctypes.POINTER(InferLayer)), ("label_embed", c_void_p),
                ("label_embed_scale", c_float), ("final_layer", c_void_p), ("final_layer_scale", c_float),
                ("bias", c_void_p), ("rope", c_void_p), ("rope_len", c_int)]


EXPORTS = [
    "tsa_version", "tsa_last_error", "tsa_att_fwd", "tsa_att_fwd_workspace_bytes", "tsa_att_bwd",
    "tsa_att_bwd_workspace_bytes", "tsa_calc_dscale", "tsa_qk_scores_i32", "tsa_quant_rows", "tsa_kv_append",
    "tsa_att_decode", "tsa_att_decode_workspace_bytes", "tsa_make_window_spans", "tsa_transpose_attention",
    "tsa_group_attention", "tsa_group_window_spans", "tsa_att_decode_static", "tsa_att_decode_static_capacity_bytes",
    "tsa_norm_rope_quant", "tsa_rope_norm_bwd", "tsa_group_window_spans_device", "tsa_kv_product", "tsa_kv_product_bwd",
    "tsa_infer_workspace_bytes", "tsa_infer_step", "tsa_matmul_norm_rope_quant", "tsa_att_fwd_set_score_dump", "tsa_shard_range", "tsa_shard_rects", "tsa_status_from_word", "tsa_selftest_bounded_wait",
    "tsa_selftest_fwd_withhold_copy", "tsa_att_fwd_host", "tsa_att_fwd_host_staging_bytes",
    "tsa_bounds_check_hits", "tsa_selftest_bounds_check",
    "tsa_att_fwd_to", "tsa_att_fwd_kv", "tsa_peer_scatter",
    "tsa_transpose_attention_device", "tsa_transpose_attention_device_workspace_bytes", "tsa_group_attention_device",
    "tsa_group_attention_device_workspace_bytes",
]


def _declare(lib):
    P = Ptr2D
    lib.tsa_version.restype = ctypes.c_char_p
    lib.tsa_last_error.restype = ctypes.c_char_p
    lib.tsa_att_fwd.argtypes = [ctypes.POINTER(AttCfg), c_void_p, P, P, P, P, P, P, c_void_p, c_void_p, c_float,
                                P, P, c_int, c_int, c_void_p, c_size_t, c_void_p, c_void_p]
    lib.tsa_att_fwd_to.argtypes = [ctypes.POINTER(AttCfg), c_void_p, P, P, P, P, P, P, c_void_p, c_void_p, c_float,
                                   ctypes.POINTER(P), c_int, P, c_int, c_int, c_void_p, c_size_t, c_void_p, c_void_p]
    lib.tsa_att_fwd_kv.argtypes = [ctypes.POINTER(AttCfg), c_void_p, P, P, P, P, P, P, c_void_p, c_void_p, c_float,
                                   P, P, P, c_float, P, c_int, c_int, c_void_p, c_size_t, c_void_p, c_void_p]
    lib.tsa_peer_scatter.argtypes = [P, ctypes.POINTER(P), c_int, c_int, c_int, c_int, c_void_p]
    lib.tsa_att_fwd_host.argtypes = [ctypes.POINTER(AttCfg), c_void_p, P, P, P, P, P, P, c_void_p, c_void_p, c_float,
                                     P, P, P, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p, c_void_p]
    lib.tsa_att_fwd_host_staging_bytes.restype = c_size_t
    lib.tsa_att_fwd_host_staging_bytes.argtypes = [ctypes.POINTER(AttCfg), c_int, c_int, c_int]
    lib.tsa_att_fwd_workspace_bytes.restype = c_size_t
    lib.tsa_att_fwd_workspace_bytes.argtypes = [ctypes.POINTER(AttCfg), c_int, c_int]
    lib.tsa_att_bwd.argtypes = [ctypes.POINTER(AttCfg), c_void_p, P, P, P, P, P, P, P, P, P, P,
                                c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_float, P, P, P, c_int, c_int,
                                c_void_p, c_size_t, c_void_p, c_void_p]
    lib.tsa_att_bwd_workspace_bytes.restype = c_size_t
    lib.tsa_att_bwd_workspace_bytes.argtypes = [ctypes.POINTER(AttCfg), c_int, c_int]
    lib.tsa_calc_dscale.argtypes = [c_int, c_int, P, P, P, c_int, c_int, c_int, c_void_p]
    lib.tsa_qk_scores_i32.argtypes = [P, P, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]
    lib.tsa_transpose_attention_device.argtypes = [c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]
    lib.tsa_transpose_attention_device_workspace_bytes.restype = c_size_t
    lib.tsa_transpose_attention_device_workspace_bytes.argtypes = [c_int, c_int]
    lib.tsa_group_attention_device.argtypes = [c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]
    lib.tsa_group_attention_device_workspace_bytes.restype = c_size_t
    lib.tsa_group_attention_device_workspace_bytes.argtypes = [c_int]
    lib.tsa_bounds_check_hits.argtypes = [c_int]
    lib.tsa_selftest_bounds_check.argtypes = [c_void_p, c_void_p]
    lib.tsa_status_from_word.argtypes = [c_int]
    lib.tsa_selftest_bounded_wait.argtypes = [ctypes.c_longlong, c_void_p, c_void_p]
    lib.tsa_selftest_fwd_withhold_copy.argtypes = [ctypes.c_longlong, c_int]
    lib.tsa_shard_range.argtypes = [c_int, c_int, c_int, c_int_p, c_int_p]
    lib.tsa_shard_rects.argtypes = [c_int, c_int, c_int, c_void_p]
    lib.tsa_att_fwd_set_score_dump.argtypes = [c_void_p, c_int, c_int, c_int]
    lib.tsa_quant_rows.argtypes = [c_int, c_int, c_int, c_float, P, P, P, c_int, c_int, c_void_p]
    lib.tsa_norm_rope_quant.argtypes = [c_int, c_int, c_float, P, P, c_int, c_float, P, P, c_int, c_int, c_int, c_void_p]
    lib.tsa_rope_norm_bwd.argtypes = [c_int, c_int, P, P, P, c_int, c_float, P, c_int, c_int, c_int, c_void_p]
    lib.tsa_group_window_spans_device.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]
    lib.tsa_kv_product.argtypes = [c_int, c_int, P, P, c_float, P, c_int, c_int, c_int, c_void_p]
    lib.tsa_kv_product_bwd.argtypes = [c_int, c_int, P, P, P, P, P, P, c_int, c_int, c_int, c_void_p]
    lib.tsa_kv_append.argtypes = [ctypes.POINTER(DecodeCfg), c_void_p, c_void_p, c_int, c_int, P, P, P, P, c_int,
                                  c_void_p, c_void_p]
    lib.tsa_att_decode.argtypes = [ctypes.POINTER(DecodeCfg), c_void_p, c_void_p, c_int, c_int, P, P, c_int, c_float,
                                   P, c_int, c_void_p, c_size_t, c_void_p, c_void_p]
    lib.tsa_att_decode_workspace_bytes.restype = c_size_t
    lib.tsa_att_decode_workspace_bytes.argtypes = [ctypes.POINTER(DecodeCfg), c_int, c_int, c_int]
    lib.tsa_att_decode_static.argtypes = [ctypes.POINTER(DecodeCfg), c_void_p, c_void_p, c_int, c_int, P, P, c_int, c_float,
                                          P, c_int, c_void_p, c_void_p]
    lib.tsa_att_decode_static_capacity_bytes.restype = c_size_t
    lib.tsa_att_decode_static_capacity_bytes.argtypes = []
    lib.tsa_matmul_norm_rope_quant.argtypes = [c_int, c_int, c_float, c_float, P, P, P, c_float, P, P, c_int, c_int, c_int, c_void_p, c_void_p]
    lib.tsa_infer_workspace_bytes.restype = c_size_t
    lib.tsa_infer_workspace_bytes.argtypes = [ctypes.POINTER(InferModel), c_int, c_int]
    lib.tsa_infer_step.argtypes = [ctypes.POINTER(InferModel), ctypes.POINTER(c_void_p), c_void_p, c_int, c_void_p, c_int, c_int,
                                   c_int, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]
    lib.tsa_make_window_spans.argtypes = [c_int, c_int_p, c_int, c_int, c_int_p, c_int_p]
    lib.tsa_transpose_attention.argtypes = [c_int, c_int_p, c_int_p, c_int, c_int_p, c_int_p]
    lib.tsa_group_attention.argtypes = [c_int, c_int_p, c_int_p, c_int, c_void_p, c_int_p]
    lib.tsa_group_window_spans.argtypes = [c_int, c_int_p, c_int, c_int, c_int, c_void_p, c_int_p]


_lib = None


def lib():
    """The loaded shared library.  Raises if it has not been built (no fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                "tscale_b200: %s is missing; build it with `make -C tscale_b200/csrc` "
                "(or __graft_entry__.build()).  There is no CPU fallback." % LIB_PATH)
        _lib = ctypes.CDLL(LIB_PATH)
        _declare(_lib)
    return _lib


class TsaError(RuntimeError):
    def __init__(self, code, text):
        RuntimeError.__init__(self, "tsa status %d: %s" % (code, text))
        self.code = code


def check(code):
    if code != TSA_OK:
        raise TsaError(code, lib().tsa_last_error().decode())
