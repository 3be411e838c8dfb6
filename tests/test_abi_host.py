"""CPU-side checks of the shared library: it loads, exports every entry point include/tsa.h declares,
rejects bad arguments with status codes (no GPU needed: validation comes before any CUDA call), and its
host span helpers agree with the reference's preprocessing (golden files) and with the oracle."""
import ctypes
import os
import re

import numpy as np
import pytest

from oracle import oracle as O
from tscale_b200 import abi, ops

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    text = open(os.path.join(ROOT, "include", "tsa.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    declared = set(re.findall(r"\b(tsa_[a-z0-9_]+)\s*\(", text))
    assert declared, "no declarations found"
    lib = abi.lib()
    for name in sorted(declared):
        assert hasattr(lib, name), "libtsa_b200.so does not export %s" % name
    assert declared == set(abi.EXPORTS)
    assert b"sm_100a" in lib.tsa_version()


def test_struct_layouts_match_header():
    assert ctypes.sizeof(abi.SpanGroup) == 130 * 4          # TAttentionSpanGroup<64>: 2 + 64 + 64 ints
    assert ctypes.sizeof(abi.Ptr2D) == 24
    assert ctypes.sizeof(abi.KvSeq) == 32
    assert ctypes.sizeof(abi.AttCfg) == 36


def test_bad_arguments_return_status_not_abort():
    lib = abi.lib()
    null = abi.Ptr2D(None, 0, 0, 0)
    assert lib.tsa_quant_rows(7, abi.TSA_F32, abi.TSA_I8, 0.0, null, null, null, 0, 128, None) == abi.TSA_BAD_ARG
    assert b"kind" in lib.tsa_last_error()
    fake = abi.Ptr2D(4096, 96 * 4, 96, 8)  # never dereferenced: validation comes first
    assert lib.tsa_norm_rope_quant(abi.TSA_F32, abi.TSA_I8, 1.0, fake, null, abi.TSA_F32, 1.0, fake, null, 1, 96, 8, None) == abi.TSA_BAD_ARG
    assert b"head size" in lib.tsa_last_error()
    assert lib.tsa_norm_rope_quant(abi.TSA_F32, abi.TSA_F16, 1.0, fake, null, abi.TSA_F32, 1.0, fake, null, 1, 64, 8, None) == abi.TSA_BAD_ARG
    assert lib.tsa_rope_norm_bwd(abi.TSA_F32, abi.TSA_F32, null, fake, null, abi.TSA_F32, 1.0, fake, 1, 64, 8, None) == abi.TSA_BAD_ARG
    assert lib.tsa_rope_norm_bwd(abi.TSA_F16, abi.TSA_F32, fake, fake, null, abi.TSA_F32, 1.0, fake, 1, 64, 8, None) == abi.TSA_UNSUPPORTED
    assert lib.tsa_quant_rows(0, abi.TSA_F32, abi.TSA_F16, 0.0, null, null, null, 0, 128, None) == abi.TSA_BAD_ARG
    cfg = ops.make_cfg("e4m3", "e4m3", 64, 64)
    rc = lib.tsa_att_fwd(ctypes.byref(cfg), None, null, null, null, null, null, null, None, None, 0.0, null, null, 2, 1,
                         None, 0, None, None)
    assert rc == abi.TSA_BAD_ARG and b"null" in lib.tsa_last_error()
    cfg.head_dim_qk = 1000
    rc = lib.tsa_att_fwd(ctypes.byref(cfg), None, null, null, null, null, null, null, None, None, 0.0, null, null, 2, 1,
                         None, 0, None, None)
    assert rc == abi.TSA_BAD_ARG
    dcfg = abi.DecodeCfg(96, abi.TSA_F16, abi.TSA_F32, 1.0)
    assert lib.tsa_att_decode(ctypes.byref(dcfg), None, None, 1, 1, null, null, 0, 0.0, null, 1, None, 0, None, None) == abi.TSA_BAD_ARG
    assert lib.tsa_att_decode_workspace_bytes(ctypes.byref(abi.DecodeCfg(128, abi.TSA_F16, abi.TSA_F32, 1.0)), 64, 16, 8192) > 0
    # fused projection: validation before any tensor map is made
    fx = abi.Ptr2D(4096, 200, 200, 8)
    assert lib.tsa_matmul_norm_rope_quant(abi.TSA_I8, abi.TSA_I8, 1.0, 1.0, fx, fx, null, 1.0, fake, null, 1, 64, 8, None, None) == abi.TSA_BAD_ARG
    assert b"multiples of 64" in lib.tsa_last_error()
    assert lib.tsa_matmul_norm_rope_quant(abi.TSA_I8, abi.TSA_F32, 1.0, 1.0, fx, fx, null, 1.0, fake, null, 1, 64, 8, None, None) == abi.TSA_BAD_ARG
    # inference step: sizes are checked before anything is dereferenced or launched
    im = abi.InferModel()
    im.dims = abi.InferDims(768, 64, 12, 1536, 50000, 50100, 0)
    assert lib.tsa_infer_workspace_bytes(ctypes.byref(im), 64, 8192) > 64 * 50000 * 4
    assert lib.tsa_infer_workspace_bytes(ctypes.byref(im), 65, 8192) == 0          # at most 64 sequences per step
    assert lib.tsa_infer_step(ctypes.byref(im), None, None, 16, None, 1, 4, 8, None, None, None, 0, None, None) == abi.TSA_BAD_ARG
    im.dims.head_dim = 96
    assert lib.tsa_infer_workspace_bytes(ctypes.byref(im), 4, 16) == 0
    assert lib.tsa_infer_step(ctypes.byref(im), None, None, 16, None, 1, 4, 8, None, None, None, 0, None, None) == abi.TSA_BAD_ARG
    assert b"head_dim" in lib.tsa_last_error()
    assert ctypes.sizeof(abi.InferLayer) == 80 and ctypes.sizeof(abi.InferDims) == 28


@pytest.mark.parametrize("name", ["att_w64_slope05", "att_full_slope0", "att_w1_d32", "att_handmade"])
def test_span_helpers_match_reference_fixtures(golden_dir, name):
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    m = ops.Mask.from_spans(z["spans"], z["span_ptr"])
    assert np.array_equal(m.rev_spans, z["rev_spans"]) and np.array_equal(m.rev_span_ptr, z["rev_span_ptr"])
    assert np.array_equal(m.groups, z["groups"]) and np.array_equal(m.group_ptr, z["group_ptr"])
    assert np.array_equal(m.rev_groups, z["rev_groups"]) and np.array_equal(m.rev_group_ptr, z["rev_group_ptr"])


@pytest.mark.parametrize("frag_lens,window", [([160, 96], 64), ([130, 62, 1, 300], 0), ([40], 1), ([4096, 100], 256), ([5], 64)])
def test_window_closed_form_equals_general_path(frag_lens, window):
    lib = abi.lib()
    fl = np.array(frag_lens, dtype=np.int32)
    length = int(fl.sum())
    spans = np.zeros((length, 2), dtype=np.int32)
    ptr = np.zeros(length + 1, dtype=np.int32)
    n = lib.tsa_make_window_spans(len(fl), fl.ctypes.data_as(abi.c_int_p), window, length, spans.ctypes.data_as(abi.c_int_p),
                                  ptr.ctypes.data_as(abi.c_int_p))
    want_spans, want_ptr = O.window_spans(frag_lens, window)
    assert n == len(want_spans) and np.array_equal(spans[:n], want_spans) and np.array_equal(ptr, want_ptr)
    closed = ops.Mask.window(frag_lens, window)
    general = ops.Mask.from_spans(want_spans, want_ptr)
    for a, b in ((closed.groups, general.groups), (closed.group_ptr, general.group_ptr),
                 (closed.rev_groups, general.rev_groups), (closed.rev_group_ptr, general.rev_group_ptr)):
        assert np.array_equal(a, b)


def test_span_helpers_report_needed_capacity():
    lib = abi.lib()
    fl = np.array([100], dtype=np.int32)
    ptr = np.zeros(101, dtype=np.int32)
    spans = np.zeros((4, 2), dtype=np.int32)
    n = lib.tsa_make_window_spans(1, fl.ctypes.data_as(abi.c_int_p), 8, 4, spans.ctypes.data_as(abi.c_int_p), ptr.ctypes.data_as(abi.c_int_p))
    assert n == -99


def test_empty_mask():
    m = ops.Mask.from_spans(np.zeros((0, 2), dtype=np.int32), np.zeros(65, dtype=np.int32))
    assert m.groups.shape[0] == 0 and np.all(m.group_ptr == 0) and m.len_att_tiles == 1


def test_header_is_plain_c_and_links(tmp_path):
    """include/tsa.h compiles as C11 without warnings, and a C program bound against the shared library the way a host
    in another language would (plain pointers and sizes) resolves every declared entry point and runs the host-side ones."""
    import shutil
    import subprocess
    cc = shutil.which("gcc")
    if cc is None:
        pytest.skip("no C compiler")
    text = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", "tsa.h")).read(), flags=re.S)
    names = sorted(set(re.findall(r"\b(tsa_[a-z0-9_]+)\s*\(", text)))
    src = tmp_path / "bind.c"
    src.write_text(
        '#include <stdio.h>\n#include <string.h>\n#include "tsa.h"\n'
        "typedef void (*fn_t)(void);\n"
        "int main(void) {\n"
        "    fn_t table[] = {" + ", ".join("(fn_t)%s" % n for n in names) + "};\n"
        "    int lens[2] = {5, 3}, spans[64], ptr[9];\n"
        "    int n = tsa_make_window_spans(2, lens, 2, 32, spans, ptr);\n"
        "    if (n != ptr[8] || strstr(tsa_version(), \"sm_100a\") == NULL) return 1;\n"
        "    printf(\"%d %d\\n\", (int)(sizeof(table) / sizeof(table[0])), n);\n"
        "    return 0;\n}\n")
    exe = tmp_path / "bind"
    lib_dir = os.path.dirname(abi.LIB_PATH)
    subprocess.run([cc, "-std=c11", "-Wall", "-Wextra", "-Werror", "-pedantic", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe),
                    "-L", lib_dir, "-ltsa_b200", "-Wl,-rpath," + lib_dir], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    assert int(out[0]) == len(names) == len(abi.EXPORTS)
    assert int(out[1]) == 4 + 2      # one span per row that has keys: rows 1..4 of the first fragment, rows 1..2 of the second
