"""Runs the REFERENCE's own runtime -- `RWKV(path, 'cuda fp16i8').forward` of
rwkv_pip_package/src/rwkv/model.py:612-1677 with RWKV_CUDA_ON=1, i.e. its CUDA operators
mm8_seq / mm8_one / wkv_forward / rwkv5 / rwkv6 -- in a process of its own (it registers the
same torch.ops names as the product) on a pre-converted checkpoint, and stores what it
computed:

    python tests/ref_model_runner.py converted.pth job.json out.npz

job.json: {"prompt": [token ids], "decode": n greedy steps, "repeat": 0 | 1}

out.npz:  logits_prefill fp32 [V]; logits_steps fp16 [n, V] (the reference's logits are
fp16 values widened to fp32, model.py:1677, so nothing is lost); tokens int64 [n] (greedy:
torch.argmax); prefill_ms (second run of the prompt, CUDA events), decode_tok_s (median step
time over the greedy loop, device synchronised per step); with "repeat": 1 the whole protocol
runs a second time, teacher-forced on the first run's tokens, and `noise_max` holds the
largest |logit difference| between the two runs (the reference's mm8_one adds its 24 partial
sums with atomics in arbitrary order, operators.cu:230).

The runtime and its prebuilt operators are staged by oracle/build_ref.py under oracle/_ref/;
`torch.utils.cpp_extension.load`, which the reference calls at import (model.py:31-38,
907, 940), is redirected to those prebuilt files so that nothing is compiled here.
"""
import json
import os
import statistics
import sys
import time
import types

import numpy as np

os.environ["RWKV_CUDA_ON"] = "1"
os.environ.setdefault("RWKV_JIT_ON", "1")

import torch  # noqa: E402
import torch.utils.cpp_extension as cpp_ext  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref")


def _prebuilt_load(name, sources=None, **kw):
    so = {"wkv_cuda": "wkv_cuda_ref.so", "rwkv5": "rwkv5_ref.so", "rwkv6": "rwkv6_ref.so"}[name]
    torch.ops.load_library(os.path.join(REF, so))
    if name == "wkv_cuda":
        return None
    ns = getattr(torch.ops, name)           # rwkv5_op.cpp:30-34 / rwkv6_op.cpp:30-34 register these too
    return types.SimpleNamespace(forward_bf16=ns.forward_bf16, forward_fp16=ns.forward_fp16,
                                 forward_fp32=ns.forward_fp32)


def main(ckpt, job_path, outp):
    cpp_ext.load = _prebuilt_load
    sys.path.insert(0, os.path.join(REF, "pkg"))
    from rwkv.model import RWKV

    with open(job_path) as f:
        job = json.load(f)
    prompt, n = job["prompt"], int(job["decode"])
    t0 = time.perf_counter()
    model = RWKV(ckpt, job.get("strategy", "cuda fp16i8"), verbose=False)
    load_s = time.perf_counter() - t0
    out = {"load_s": np.float64(load_s)}

    def run(forced=None):
        logits, state = model.forward(prompt, None)
        lp = logits.float().cpu()
        steps = torch.empty((n, lp.numel()), dtype=torch.float16)
        toks, dts = [], []
        tok = int(torch.argmax(logits))
        for i in range(n):
            toks.append(tok)
            torch.cuda.synchronize()
            t = time.perf_counter()
            logits, state = model.forward([tok if forced is None else int(forced[i])], state)
            torch.cuda.synchronize()
            dts.append(time.perf_counter() - t)
            steps[i] = logits.to(torch.float16).cpu()
            tok = int(torch.argmax(logits))
        return lp, steps, toks, dts

    lp, steps, toks, dts = run()
    out["logits_prefill"] = lp.numpy()
    out["logits_steps"] = steps.view(torch.int16).numpy()
    out["tokens"] = np.asarray(toks, dtype=np.int64)
    out["decode_tok_s"] = np.float64(1.0 / statistics.median(dts[len(dts) // 4:])) if dts else np.float64(0)
    # prefill time: the prompt once more (TorchScript and the kernels are warm now)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    model.forward(prompt, None)
    e1.record()
    torch.cuda.synchronize()
    out["prefill_ms"] = np.float64(e0.elapsed_time(e1))
    if job.get("repeat"):
        lp2, steps2, _, _ = run(forced=toks)
        noise = (lp2 - lp).abs().max().item()
        if n:
            noise = max(noise, (steps2.float() - steps.float()).abs().max().item())
        out["noise_max"] = np.float64(noise)
    np.savez(outp, **out)


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2], sys.argv[3])
