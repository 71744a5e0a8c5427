"""The product's operators against the REFERENCE's own CUDA kernels, both run on this GPU on
the same seeded inputs.  The reference kernels come prebuilt from oracle/_ref/ (see
oracle/build_ref.py) and run in a child process; the test is skipped when they are absent."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from oracle import rwkv_oracle as orc

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref")


def _i16(t):
    return t.contiguous().view(torch.int16).numpy()


@pytest.fixture(scope="module")
def ref_outputs(tmp_path_factory):
    if not all(os.path.exists(os.path.join(REF, n)) for n in ("wkv_cuda_ref.so", "rwkv5_ref.so", "rwkv6_ref.so")):
        pytest.skip("oracle/_ref not built")
    tmp = tmp_path_factory.mktemp("refcuda")
    g = torch.Generator().manual_seed(3000)
    inp = {}
    cases = {"a": (4096, 4096, 16), "b": (768, 3072, 5), "c": (3072, 768, 33)}
    for name, (N, M, B) in cases.items():
        w = (torch.randn(N, M, generator=g) * 0.02).half().float()
        q, mx, rx, my, ry = orc.quantize_weight(w, torch.float16)
        inp[f"mm8/{name}/w"] = q.numpy()
        for n, t in (("mx", mx), ("rx", rx), ("my", my), ("ry", ry)):
            inp[f"mm8/{name}/{n}"] = _i16(t)
        inp[f"mm8/{name}/x1"] = _i16(torch.randn(N, generator=g).half())
        inp[f"mm8/{name}/xs"] = _i16(torch.randn(B, N, generator=g).half())
    T, C = 64, 768
    inp["wkv4/k"] = torch.randn(T, C, generator=g).numpy()
    inp["wkv4/v"] = torch.randn(T, C, generator=g).numpy()
    inp["wkv4/w"] = (-torch.exp(torch.empty(C).uniform_(-5, 1, generator=g))).numpy()
    inp["wkv4/u"] = torch.empty(C).uniform_(-1, 1, generator=g).numpy()
    inp["wkv4/aa"], inp["wkv4/bb"] = np.zeros(C, np.float32), np.zeros(C, np.float32)
    inp["wkv4/pp"] = np.full(C, -1e30, np.float32)
    H, N64, T56 = 4, 64, 48
    for which in (5, 6):
        p = f"wkv{which}"
        Cc = H * N64
        inp[f"{p}/r"] = torch.randn(T56, Cc, generator=g).numpy()
        inp[f"{p}/k"] = (torch.randn(T56, Cc, generator=g) * 0.5).numpy()
        inp[f"{p}/v"] = torch.randn(T56, Cc, generator=g).numpy()
        shape = (T56, Cc) if which == 6 else (Cc,)
        inp[f"{p}/w"] = torch.exp(-torch.exp(torch.empty(shape).uniform_(-5, 1, generator=g))).numpy()
        inp[f"{p}/u"] = torch.empty(Cc).uniform_(-1, 1, generator=g).numpy()
        inp[f"{p}/state"] = (torch.randn(H, N64, N64, generator=g) * 0.1).numpy()
    inp["time/wkv_T"] = np.int64(2048)
    fin, fout = str(tmp / "in.npz"), str(tmp / "out.npz")
    np.savez(fin, **inp)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "ref_cuda_runner.py"), fin, fout],
                       capture_output=True, text=True, timeout=600)
    if r.returncode != 0:
        pytest.fail("reference CUDA runner failed:\n" + r.stdout[-2000:] + r.stderr[-4000:])
    return inp, dict(np.load(fout))


def _cu(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.view(dtype)


def test_mm8_against_reference_kernels(ref_outputs):
    from chatrwkv_b200 import ops  # noqa: F401
    inp, out = ref_outputs
    h = torch.float16
    report = {}
    for name in ("a", "b", "c"):
        g = lambda s: inp[f"mm8/{name}/{s}"]
        w = _cu(g("w"))
        mx, rx, my, ry = (_cu(g(n), h) for n in ("mx", "rx", "my", "ry"))
        N, M = w.shape
        y = torch.zeros(M, dtype=torch.float32, device="cuda")
        torch.ops.rwkv.mm8_one(N, M, _cu(g("x1"), h), w, mx, rx, my, ry, y)
        ref = torch.from_numpy(out[f"mm8/{name}/y1"])
        # the reference sums with atomics in arbitrary order: compare at fp32 round-off scale
        assert (y.cpu() - ref).abs().max().item() <= 1e-4 * max(1.0, ref.abs().max().item())
        xs = _cu(g("xs"), h)
        ys = torch.empty((xs.shape[0], M), dtype=h, device="cuda")
        torch.ops.rwkv.mm8_seq(xs.shape[0], N, M, xs, w, mx, rx, my, ry, ys)
        refs = torch.from_numpy(out[f"mm8/{name}/ys"]).view(h)
        d = (ys.cpu().float() - refs.float()).abs()
        assert (d <= refs.float().abs() * 2 ** -9 + 2e-4).all(), d.max().item()
        report[name] = {"N": N, "M": M, "ref_mm8_one_us": float(out[f"mm8/{name}/t_one_us"]),
                        "ref_mm8_seq_us": float(out[f"mm8/{name}/t_seq_us"]), "seq_rows": int(xs.shape[0]),
                        "mismatch_frac_fp16_seq": float((ys.cpu() != refs).float().mean())}
    for name in ("wkv4", "wkv5", "wkv6"):
        report[f"ref_{name}_T2048_C4096_us"] = float(out[f"time/{name}_us"])
    rdir = os.environ.get("RWKV_B200_REPORT_DIR")          # the reference kernels' times on this GPU, for the record
    if rdir:
        os.makedirs(rdir, exist_ok=True)
        with open(os.path.join(rdir, "reference_cuda_ops.json"), "w") as f:
            json.dump(report, f, indent=1)


def test_wkv_against_reference_kernels(ref_outputs):
    from chatrwkv_b200 import ops  # noqa: F401
    inp, out = ref_outputs
    k, v = _cu(inp["wkv4/k"]), _cu(inp["wkv4/v"])
    T, C = k.shape
    aa, bb, pp = _cu(inp["wkv4/aa"]), _cu(inp["wkv4/bb"]), _cu(inp["wkv4/pp"])
    y = torch.empty_like(k)
    torch.ops.rwkv.wkv_forward(1, T, C, _cu(inp["wkv4/w"]), _cu(inp["wkv4/u"]), k, v, y, aa, bb, pp)
    # the reference kernel is built with --use_fast_math (approximate exp and division)
    torch.testing.assert_close(y.cpu(), torch.from_numpy(out["wkv4/y"]), rtol=2e-4, atol=2e-4)
    torch.testing.assert_close(aa.cpu(), torch.from_numpy(out["wkv4/aa"]), rtol=2e-4, atol=2e-4)
    torch.testing.assert_close(pp.cpu(), torch.from_numpy(out["wkv4/pp"]), rtol=1e-5, atol=1e-5)
    for which in (5, 6):
        p = f"wkv{which}"
        r, kk, vv, w, u, s = (_cu(inp[f"{p}/{n}"]) for n in ("r", "k", "v", "w", "u", "state"))
        T, C = r.shape
        y = torch.empty_like(r)
        getattr(torch.ops, f"rwkv{which}").forward_fp32(1, T, C, s.shape[0], s, r, kk, vv, w, u, y)
        torch.testing.assert_close(y.cpu(), torch.from_numpy(out[f"{p}/y"]), rtol=1e-4, atol=1e-4)
        torch.testing.assert_close(s.cpu(), torch.from_numpy(out[f"{p}/state"]), rtol=1e-4, atol=1e-4)
