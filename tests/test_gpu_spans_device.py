"""Device-side transpose and grouping of arbitrary span lists against the host helpers (which are checked against the
reference's TransposeAttention / GroupAttention on fixtures): bit-identical records, and the same attention results."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import util

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _csr(rows):
    spans, ptr = [], [0]
    for r in rows:
        spans.extend(r)
        ptr.append(len(spans))
    return np.array(spans, dtype=np.int32).reshape(-1, 2), np.array(ptr, dtype=np.int32)


def _masks():
    res = {}
    for name, (frags, window) in {"window64": ([300, 212], 64), "full": ([257, 130], 0), "window1": ([70], 1)}.items():
        res[name] = O.window_spans(frags, window)
    # ragged: empty rows, rows of two spans, a span that sticks out past the end and one that starts before 0
    length = 300
    rows = []
    for i in range(length):
        if i % 7 == 0:
            rows.append([])
        elif i > 140 and i % 5 == 0:
            rows.append([(3, 40), (i - 20, i - 1)])
        elif i == 33:
            rows.append([(-5, 10), (20, 500)])
        else:
            rows.append([(max(0, i - 90), i - 1)] if i > 0 else [])
    res["ragged"] = _csr(rows)
    # documents with a shared prefix: every row attends 16 "global" keys and its own document up to itself
    rng = np.random.default_rng(11)
    bounds = [0] + sorted(set(int(x) for x in rng.integers(40, 1000, 9))) + [1000]
    rows = []
    for d0, d1 in zip(bounds[:-1], bounds[1:]):
        for i in range(d0, d1):
            r = []
            if i > 0:
                if d0 > 16:
                    r.append((0, 15))
                    if i > d0:
                        r.append((d0, i - 1))
                else:
                    r.append((0, i - 1))
            rows.append(r)
    res["documents"] = _csr(rows)
    # random sorted disjoint spans, up to four per row, not causal
    rows = []
    for i in range(450):
        cuts = sorted(set(int(x) for x in rng.integers(0, 450, int(rng.integers(0, 9)))))
        r = [(cuts[k], cuts[k + 1] - 1) for k in range(0, len(cuts) - 1, 2) if cuts[k + 1] - 1 >= cuts[k]]
        # keep them disjoint and non-adjacent as written: finish < next start
        rows.append(r)
    res["random"] = _csr(rows)
    return res


@pytest.mark.parametrize("name", ["window64", "full", "window1", "ragged", "documents", "random"])
def test_device_transpose_and_grouping_equal_host(name):
    from tscale_b200 import ops
    spans, ptr = _masks()[name]
    host = ops.Mask.from_spans(spans, ptr)
    sd = torch.from_numpy(np.ascontiguousarray(spans)).to(DEV)
    pd = torch.from_numpy(ptr).to(DEV)
    length = len(ptr) - 1
    dev = ops.Mask.from_spans_device(sd, pd, max_rev_spans=length * length // 2 + 16, max_groups=8192)
    torch.cuda.synchronize()
    assert np.array_equal(dev.rev_span_ptr_dev.cpu().numpy(), host.rev_span_ptr)
    assert np.array_equal(dev.rev_spans_dev.cpu().numpy(), host.rev_spans.reshape(-1, 2))
    g, gp, rg, rgp = dev.dev(DEV)
    as_i32 = lambda t: t.cpu().numpy().view(np.int32).reshape(-1, 130)
    assert np.array_equal(gp.cpu().numpy(), host.group_ptr)
    assert np.array_equal(rgp.cpu().numpy(), host.rev_group_ptr)
    assert np.array_equal(as_i32(g), host.groups.reshape(-1, 130))
    assert np.array_equal(as_i32(rg), host.rev_groups.reshape(-1, 130))


def test_device_capacity_overflow_is_reported():
    from tscale_b200 import ops
    spans, ptr = _masks()["documents"]
    sd = torch.from_numpy(np.ascontiguousarray(spans)).to(DEV)
    pd = torch.from_numpy(ptr).to(DEV)
    with pytest.raises(RuntimeError):
        ops.Mask.from_spans_device(sd, pd, max_rev_spans=8)
    with pytest.raises(RuntimeError):
        ops.Mask.from_spans_device(sd, pd, max_groups=2)


@pytest.mark.parametrize("d", [64, 128])
def test_attention_with_device_built_mask(d):
    """Forward and backward through a mask transposed and grouped on the GPU give the bits of the host-built mask."""
    from tscale_b200 import ops
    spans, ptr = _masks()["documents"]
    length, heads = len(ptr) - 1, 2
    q, k, v = util.make_qkv(5, length, heads, d, d, 0.5)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    q8, sq, _ = util.quantize(q, "i8", d)
    k8, sk, _ = util.quantize(k, "i8", d)
    v8, sv, _ = util.quantize(v, "e4m3", d)
    g = dict(q=t(q8.view(np.uint8)), k=t(k8.view(np.uint8)), v=t(v8.view(np.uint8)), sq=t(sq), sk=t(sk), sv=t(sv))
    cfg = ops.make_cfg("i8", "e4m3", d, d, out_dtype=torch.float32, grad_dtype=torch.float32)
    masks = [ops.Mask.from_spans(spans, ptr), ops.Mask.from_spans_device(t(spans), t(ptr))]
    gen = torch.Generator(device=DEV)
    gen.manual_seed(2)
    d_out = torch.randn((length, heads * d), generator=gen, device=DEV) * 1e-2
    res = []
    for m in masks:
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        out, lse = ops.att_fwd(cfg, g["q"], g["k"], g["v"], g["sk"], m, 0.0, heads, qk_scale=g["sq"], v_scale=g["sv"], status=status)
        grads = ops.att_bwd(cfg, g["q"], g["k"], g["v"], g["sk"], d_out, out, lse, m, 0.0, heads, qk_scale=g["sq"], v_scale=g["sv"],
                            status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        res.append((out, lse) + tuple(grads))
    for a, b in zip(res[0], res[1]):
        assert torch.equal(a, b)
