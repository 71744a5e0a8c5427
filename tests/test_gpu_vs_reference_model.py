"""RWKV.forward of this package against the REFERENCE's own `RWKV(path, 'cuda fp16i8')` with
RWKV_CUDA_ON=1 (rwkv_pip_package/src/rwkv/model.py:612-1677 on its CUDA operators), both on
this GPU, on byte-identical weights: the product packs a seeded random-init checkpoint, writes it
in the reference's pre-converted format (model.py:646-656, 894-903) and the reference loads
that file in a child process (tests/ref_model_runner.py; staged by oracle/build_ref.py).

Gate, per configuration (prompt + greedy steps as named): logits within max-abs 2e-2 of the
reference's after the prompt and at EVERY decode step (the product is teacher-forced on the
reference's greedy tokens), and the product's arg-max equal to the reference's next token at
every step; a step whose arg-max differs is forgiven only when the reference's own top-2
margin is below twice the logit difference observed at that step, and the number of forgiven
steps is recorded.  Every decode path of the runtime is run.  The reference's decode rate and
prefill time on the same GPU are recorded next to the product's.

The reference is not bit-stable: its mm8_one adds partial sums with atomics in arbitrary order
(operators.cu:230), a different fp32 sum flips fp16 roundings, and the flips random-walk through
the layers.  The runner therefore repeats the whole protocol and reports the reference's own
run-to-run difference (`noise_max`).  Measured on a B200: 0.003 at the 169M shape, 0.022 at the
7B shape, 0.025 at 14B, 0.042 for RWKV-6 7B -- above 2e-2 from 7B on.  The bound asserted is
therefore max(2e-2, 1.5 x noise_max): 2e-2 wherever the reference itself can meet it, and
"indistinguishable from a second run of the reference" where it cannot.

Reports go to $RWKV_B200_REPORT_DIR/reference_model_<config>.json when that variable is set.
"""
import copy
import json
import os
import subprocess
import sys
import time

import numpy as np
import pytest
import torch

from chatrwkv_b200 import synth

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref")
TOL = 2e-2

# name: (version, shape name, checkpoint seed, prompt tokens, greedy steps, measure noise floor)
CONFIGS = {
    "config0_v4_169m": (4, "v4-169m", 1000, 64, 128, True),
    "config2_v4_7b": (4, "v4-7b", 1002, 1024, 256, True),
    "config3_v6_7b": (6, "v6-7b", 1003, 2048, 512, True),
    "config4_v4_14b": (4, "v4-14b", 1004, 256, 512, True),
}


def _reference_ready():
    return all(os.path.exists(os.path.join(REF, n)) for n in
               ("wkv_cuda_ref.so", "rwkv5_ref.so", "rwkv6_ref.so", os.path.join("pkg", "rwkv", "model.py")))


def _run_reference(tmp, converted, prompt, n, repeat, strategy="cuda fp16i8"):
    ck, job, out = str(tmp / "converted.pth"), str(tmp / "job.json"), str(tmp / "ref.npz")
    torch.save(converted, ck)
    with open(job, "w") as f:
        json.dump({"prompt": prompt, "decode": n, "repeat": int(repeat), "strategy": strategy}, f)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "ref_model_runner.py"), ck, job, out],
                       capture_output=True, text=True, timeout=1500)
    os.remove(ck)
    if r.returncode != 0:
        pytest.fail("reference model runner failed:\n" + r.stdout[-2000:] + r.stderr[-4000:])
    return dict(np.load(out))


def _decode(model, state, ref_tokens, ref_steps):
    """Teacher-forced on the reference's tokens; returns (worst |dlogit|, mismatching steps, forgiven steps,
    smallest reference top-2 margin, tok/s)."""
    worst, mismatch, forgiven, min_margin = 0.0, 0, 0, float("inf")
    n = len(ref_tokens)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = []
    for i in range(n):
        logits, state = model.forward([int(ref_tokens[i])], state)
        outs.append(logits)
    torch.cuda.synchronize()
    rate = n / (time.perf_counter() - t0)
    for i in range(n):
        ref = torch.from_numpy(ref_steps[i]).view(torch.float16).float().cuda()
        err = (outs[i] - ref).abs().max().item()
        worst = max(worst, err)
        top2 = torch.topk(ref, 2).values
        margin = (top2[0] - top2[1]).item()
        min_margin = min(min_margin, margin)
        if i + 1 < n and int(torch.argmax(outs[i])) != int(ref_tokens[i + 1]):
            mismatch += 1
            if margin < 2 * err:
                forgiven += 1
    return worst, mismatch, forgiven, min_margin, rate


@pytest.mark.parametrize("name", list(CONFIGS))
def test_logits_and_greedy_tokens_match_reference_cuda_path(name, tmp_path):
    if not _reference_ready():
        pytest.skip("oracle/_ref (reference operators + staged runtime) not built")
    from chatrwkv_b200 import _lib
    from chatrwkv_b200.model import RWKV
    version, shape, seed, n_prompt, n_steps, noise = CONFIGS[name]
    L, D, Fn, V = synth.SHAPES[shape]
    if torch.cuda.get_device_properties(0).total_memory < 60e9 and D >= 4096:
        pytest.skip("needs a large-memory GPU")
    dev = torch.device("cuda", 0)
    ck = synth.make_checkpoint(version, L, D, Fn, V, seed=seed, device=dev)
    model = RWKV(ck, "cuda fp16i8", verbose=False)
    del ck
    torch.cuda.empty_cache()
    converted = model.export_converted()
    if version == 6:
        # the reference's loader takes the head count from a `time_faaaa` key (model.py:678-679) and renames
        # it to `time_first` itself (model.py:767-769)
        converted = {k.replace(".time_first", ".time_faaaa"): v for k, v in converted.items()}
    prompt = synth.make_tokens(n_prompt, V, 2000)
    ref = _run_reference(tmp_path, converted, prompt, n_steps, noise)
    del converted

    logits, state = model.forward(prompt, None)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    logits, state = model.forward(prompt, None)
    torch.cuda.synchronize()
    prefill_ms = (time.perf_counter() - t0) * 1e3
    ref_p = torch.from_numpy(ref["logits_prefill"]).cuda()
    err_p = (logits - ref_p).abs().max().item()
    tokens = ref["tokens"]
    top2 = torch.topk(ref_p, 2).values
    first_ok = int(torch.argmax(logits)) == int(tokens[0]) or (top2[0] - top2[1]).item() < 2 * err_p
    snapshot = copy.deepcopy(state)

    report = {"config": name, "prompt": n_prompt, "steps": n_steps, "prefill_max_abs": err_p,
              "reference": {"decode_tok_s": float(ref["decode_tok_s"]), "prefill_ms": float(ref["prefill_ms"]),
                            "noise_max": float(ref["noise_max"]) if "noise_max" in ref else None},
              "product": {"prefill_ms": prefill_ms}}
    # every decode path of the runtime: a launch per group of matmuls with 16-bit fixed-point activations (the
    # default), the same with fp32 arithmetic, and for RWKV-4 the persistent weight-stream kernel
    paths = [("launch", False, 0), ("launch_fp32", False, 8)]
    if version == 4:
        paths.insert(0, ("stream", True, 0))
    try:
        for label, use_stream, variant in paths:
            _lib.lib().rwkv_mm8_one_set_variant(variant)
            model.set_decode_path("stream" if use_stream and version == 4 else "launch")   # drops the captured graphs
            st = copy.deepcopy(snapshot)
            worst, mismatch, forgiven, min_margin, rate = _decode(model, st, tokens, ref["logits_steps"])
            report["product"][label] = {"max_abs": worst, "argmax_mismatch_steps": mismatch, "forgiven_steps": forgiven,
                                        "min_reference_top2_margin": min_margin, "decode_tok_s_host_loop": rate}
    finally:
        _lib.lib().rwkv_mm8_one_set_variant(0)
    tol = max(TOL, 1.5 * float(ref["noise_max"])) if "noise_max" in ref else TOL
    report["tolerance"] = tol
    rdir = os.environ.get("RWKV_B200_REPORT_DIR")
    if rdir:
        os.makedirs(rdir, exist_ok=True)
        with open(os.path.join(rdir, f"reference_model_{name}.json"), "w") as f:
            json.dump(report, f, indent=1)
    print(json.dumps(report))
    assert err_p <= tol and first_ok, report
    for label, _, _ in paths:
        r = report["product"][label]
        assert r["max_abs"] <= tol, report
        assert r["argmax_mismatch_steps"] == r["forgiven_steps"], report


@pytest.mark.parametrize("strategy", ["cuda fp16", "cuda fp16i8 *6 -> cuda fp16"])
def test_plain_and_mixed_strategies_match_reference_cuda_path(strategy, tmp_path):
    """The 169M shape under the strategies with plain fp16 layers: the reference runs its cuBLAS GEMM operator for
    them (model.py:143-167), this runtime a library GEMM too; logits after the prompt and at every teacher-forced step."""
    if not _reference_ready():
        pytest.skip("oracle/_ref (reference operators + staged runtime) not built")
    from chatrwkv_b200.model import RWKV
    L, D, Fn, V = synth.SHAPES["v4-169m"]
    ck = synth.make_checkpoint(4, L, D, Fn, V, seed=1000, device=torch.device("cuda", 0))
    model = RWKV(ck, strategy, verbose=False)
    del ck
    prompt = synth.make_tokens(64, V, 2000)
    ref = _run_reference(tmp_path, model.export_converted(), prompt, 64, True, strategy)
    logits, state = model.forward(prompt, None)
    err_p = (logits - torch.from_numpy(ref["logits_prefill"]).cuda()).abs().max().item()
    worst, mismatch, forgiven, _, _ = _decode(model, state, ref["tokens"], ref["logits_steps"])
    tol = max(TOL, 1.5 * float(ref["noise_max"]))
    print(json.dumps({"strategy": strategy, "prefill_max_abs": err_p, "decode_max_abs": worst, "mismatch": mismatch,
                      "forgiven": forgiven, "reference_noise": float(ref["noise_max"])}))
    assert err_p <= tol and worst <= tol and mismatch == forgiven
