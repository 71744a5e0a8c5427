"""Runs the REFERENCE's CUDA operators (built by oracle/build_ref.py into oracle/_ref/) in a
process of their own -- they register the same torch.ops names as the product -- on inputs
read from an .npz, and writes their outputs (and CUDA-event timings) to another .npz.

    python tests/ref_cuda_runner.py in.npz out.npz
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref")


def _t(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.view(dtype)


def _time(fn, iters=20):
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3   # us


def main(inp, outp):
    torch.ops.load_library(os.path.join(REF, "wkv_cuda_ref.so"))
    torch.ops.load_library(os.path.join(REF, "rwkv5_ref.so"))
    torch.ops.load_library(os.path.join(REF, "rwkv6_ref.so"))
    d = np.load(inp)
    out = {}
    h = torch.float16
    for name in sorted({k.split("/")[1] for k in d.files if k.startswith("mm8/")}):
        g = lambda s: d[f"mm8/{name}/{s}"]
        w = _t(g("w"))
        mx, rx, my, ry = _t(g("mx"), h), _t(g("rx"), h), _t(g("my"), h), _t(g("ry"), h)
        N, M = w.shape
        x1 = _t(g("x1"), h)
        y = torch.zeros(M, dtype=torch.float32, device="cuda")
        torch.ops.rwkv.mm8_one(N, M, x1, w, mx, rx, my, ry, y)
        out[f"mm8/{name}/y1"] = y.cpu().numpy()
        yy = torch.zeros(M, dtype=torch.float32, device="cuda")
        out[f"mm8/{name}/t_one_us"] = np.float64(_time(lambda: torch.ops.rwkv.mm8_one(N, M, x1, w, mx, rx, my, ry, yy)))
        xs = _t(g("xs"), h)
        B = xs.shape[0]
        ys = torch.empty((B, M), dtype=h, device="cuda")
        torch.ops.rwkv.mm8_seq(B, N, M, xs, w, mx, rx, my, ry, ys)
        out[f"mm8/{name}/ys"] = ys.view(torch.int16).cpu().numpy()
        out[f"mm8/{name}/t_seq_us"] = np.float64(_time(lambda: torch.ops.rwkv.mm8_seq(B, N, M, xs, w, mx, rx, my, ry, ys), 5))
    if "wkv4/k" in d.files:
        k, v = _t(d["wkv4/k"]), _t(d["wkv4/v"])
        T, C = k.shape
        w, u = _t(d["wkv4/w"]), _t(d["wkv4/u"])
        aa, bb, pp = _t(d["wkv4/aa"]), _t(d["wkv4/bb"]), _t(d["wkv4/pp"])
        y = torch.empty_like(k)
        torch.ops.rwkv.wkv_forward(1, T, C, w, u, k, v, y, aa, bb, pp)
        out["wkv4/y"], out["wkv4/aa"], out["wkv4/bb"], out["wkv4/pp"] = (t.cpu().numpy() for t in (y, aa, bb, pp))
        out["wkv4/t_us"] = np.float64(_time(lambda: torch.ops.rwkv.wkv_forward(1, T, C, w, u, k, v, y, aa, bb, pp), 5))
    for which in (5, 6):
        p = f"wkv{which}"
        if f"{p}/r" not in d.files:
            continue
        r, k, v, w, u, s = (_t(d[f"{p}/{n}"]) for n in ("r", "k", "v", "w", "u", "state"))
        T, C = r.shape
        H = s.shape[0]
        y = torch.empty_like(r)
        fn = getattr(torch.ops, f"rwkv{which}").forward_fp32
        fn(1, T, C, H, s, r, k, v, w, u, y)
        out[f"{p}/y"], out[f"{p}/state"] = y.cpu().numpy(), s.cpu().numpy()
        s2 = s.clone()
        out[f"{p}/t_us"] = np.float64(_time(lambda: fn(1, T, C, H, s2, r, k, v, w, u, y), 5))
    # timing only, at the 7B width (64 heads of 64, 2048 steps): what the product's kernels are compared with
    if "time/wkv_T" in d.files:
        T, C, H = int(d["time/wkv_T"]), 4096, 64
        g = torch.Generator(device="cuda").manual_seed(3001)
        k, v, r = (torch.randn(T, C, generator=g, device="cuda") for _ in range(3))
        w6 = torch.exp(-torch.exp(torch.rand(T, C, generator=g, device="cuda") * 6 - 5))
        w4 = -torch.exp(torch.rand(C, generator=g, device="cuda") * 6 - 5)
        u = torch.rand(C, generator=g, device="cuda") * 2 - 1
        y = torch.empty(T, C, device="cuda")
        aa, bb, pp = torch.zeros(C, device="cuda"), torch.zeros(C, device="cuda"), torch.full((C,), -1e30, device="cuda")
        S = torch.zeros(H, C // H, C // H, device="cuda")
        out["time/wkv4_us"] = np.float64(_time(lambda: torch.ops.rwkv.wkv_forward(1, T, C, w4, u, k, v, y, aa, bb, pp), 5))
        out["time/wkv5_us"] = np.float64(_time(lambda: torch.ops.rwkv5.forward_fp32(1, T, C, H, S, r, k, v, w6[0].contiguous(), u, y), 5))
        out["time/wkv6_us"] = np.float64(_time(lambda: torch.ops.rwkv6.forward_fp32(1, T, C, H, S, r, k, v, w6, u, y), 5))
    np.savez(outp, **out)


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2])
