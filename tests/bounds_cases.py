"""Small forward / backward / decode / quantiser / combiner calls against whatever build of the library TSA_B200_LIB names,
followed by the count of out-of-range row lookups that build caught.  Run as a module by test_gpu_bounds_check.py with the
bounds-check build; prints one JSON line."""
import json

import numpy as np
import torch

from tscale_b200 import abi, ops


def main():
    dev = torch.device("cuda:0")
    L = abi.lib()
    plane = torch.zeros(1, dtype=torch.float32, device=dev)
    sink = torch.zeros(1, dtype=torch.float32, device=dev)
    selftest = L.tsa_selftest_bounds_check(plane.data_ptr(), sink.data_ptr())
    L.tsa_bounds_check_hits(1)
    gen = torch.Generator(device=dev)
    gen.manual_seed(5)
    cases = 0
    for d, heads, frag_lens, window, qk, v in ((64, 3, [200, 120], 64, "e4m3", "e4m3"), (128, 2, [256, 130], 0, "i8", "e4m3"),
                                               (64, 2, [129], 0, "i8", "i8"), (96, 2, [100, 60], 32, "i8", "i8")):
        rows = sum(frag_lens)
        t = {}
        for n, dt in (("q", qk), ("k", qk), ("v", v)):
            x = torch.randn((rows, heads * d), generator=gen, device=dev) * 0.5
            t[n], t["s" + n] = ops.quant_rows(x, "absmax", dt, d)
        mask = ops.Mask.window(frag_lens, window)
        cfg = ops.make_cfg(qk, v, d, d, out_dtype=torch.float32, grad_dtype=torch.float32)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        out, lse = ops.att_fwd(cfg, t["q"], t["k"], t["v"], t["sk"], mask, 0.25, heads, qk_scale=t["sq"], v_scale=t["sv"], status=status)
        d_out = torch.randn((rows, heads * d), generator=gen, device=dev) * 1e-2
        ops.att_bwd(cfg, t["q"], t["k"], t["v"], t["sk"], d_out, out, lse, mask, 0.25, heads, qk_scale=t["sq"], v_scale=t["sv"], status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0, "device status %#x" % int(status.item())
        assert bool(torch.isfinite(out).all())
        cases += 1
    # decode step over a short int8 cache
    ctx, dh, hh = 300, 128, 4
    cache = ops.KVCache(2, ctx + 1, hh, dh, dev, scale_dtype=torch.float16, out_dtype=torch.float32)
    rng = np.random.default_rng(3)
    for step in range(3):
        kn = torch.from_numpy(rng.integers(-127, 128, (2, hh * dh), dtype=np.int8)).to(dev)
        vn = torch.from_numpy(rng.integers(-127, 128, (2, hh * dh), dtype=np.int8)).to(dev)
        ks = torch.rand((2, hh), device=dev).to(torch.float16)
        vs = torch.rand((2, hh), device=dev).to(torch.float16)
        cache.append(kn, ks, vn, vs)
        q = torch.from_numpy(rng.integers(-127, 128, (2, hh * dh), dtype=np.int8)).to(dev)
        qs = torch.rand((2, hh), device=dev).to(torch.float16)
        cache.decode(q, qs, 0, 0.0)
        cases += 1
    torch.cuda.synchronize()
    hits = L.tsa_bounds_check_hits(0)
    print(json.dumps({"selftest_caught": selftest, "hits": hits, "cases": cases}))


if __name__ == "__main__":
    main()
