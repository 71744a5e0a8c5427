"""Times the REFERENCE's own CPU implementation of the hot path -- `RWKV(path, 'cpu fp32i8')` of
rwkv_pip_package/src/rwkv/model.py (loader with its inline int8 packing, torch_mm8_one / torch_mm8_seq
at model.py:91-97, att_one / ffn_one at model.py:984-1055) -- on this machine's host cores.  Test
and benchmark infrastructure only: the product never imports this module.

    python -m oracle.ref_cpu_bench config0 [--steps K] [--warmup W]
    python -m oracle.ref_cpu_bench token7b [--steps K] [--warmup W] [--shape v4-7b]

config0  the whole 169M-shape model (12 x 768, ffn 3072, vocab 50277, seeded random init): the 64-token
         prompt as one call, then greedy one-token steps; prints tokens/s of the steps.
token7b  a bounded sample of one decode token at a large shape: the reference cannot finish a 32-layer
         7B-shape model in minutes on host cores (every step dequantises 7.2 G codes), so two models of
         that WIDTH are timed, with one and with two layers (embedding and head included), and the
         step time of the full depth is extrapolated as t1 + (L - 1) * (t2 - t1): the per-layer work
         is identical in every layer.  Prints the extrapolated tokens/s and the sample it came from.

One JSON line on stdout.  The runtime is taken from oracle/_ref/pkg (staged by oracle/build_ref.py); it
runs with RWKV_CUDA_ON=0 and all host threads.
"""
import argparse
import json
import os
import statistics
import sys
import tempfile
import time

os.environ["RWKV_CUDA_ON"] = "0"
os.environ.setdefault("RWKV_JIT_ON", "1")

import torch  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
PKG = os.path.join(HERE, "_ref", "pkg")


def available():
    return os.path.exists(os.path.join(PKG, "rwkv", "model.py"))


def _threads():
    try:
        n = len(os.sched_getaffinity(0))
    except (AttributeError, OSError):
        n = os.cpu_count() or 1
    torch.set_num_threads(n)
    return n


def _model(version, L, D, Fn, V, seed, tmp):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, PKG)
    from chatrwkv_b200 import synth
    from rwkv.model import RWKV
    ck = synth.make_checkpoint(version, L, D, Fn, V, seed=seed)
    path = os.path.join(tmp, f"raw_{L}_{D}.pth")
    torch.save(ck, path)
    del ck
    t0 = time.perf_counter()
    m = RWKV(path, "cpu fp32i8", verbose=False)
    os.remove(path)
    return m, time.perf_counter() - t0


def _steps(model, state, tok, steps, warmup):
    dts = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        logits, state = model.forward([tok], state)
        tok = int(torch.argmax(logits))
        if i >= warmup:
            dts.append(time.perf_counter() - t0)
    return dts


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("mode", choices=["config0", "token7b"])
    ap.add_argument("--steps", type=int, default=16)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--shape", default="v4-7b")
    a = ap.parse_args()
    cores = _threads()
    sys.path.insert(0, ROOT)
    from chatrwkv_b200 import synth
    with tempfile.TemporaryDirectory() as tmp:
        if a.mode == "config0":
            L, D, Fn, V = synth.SHAPES["v4-169m"]
            model, load_s = _model(4, L, D, Fn, V, 1000, tmp)
            prompt = synth.make_tokens(64, V, 2000)
            t0 = time.perf_counter()
            logits, state = model.forward(prompt, None)
            prefill_s = time.perf_counter() - t0
            dts = _steps(model, state, int(torch.argmax(logits)), a.steps, a.warmup)
            out = {"kind": "reference", "mode": "config0", "cores": cores, "value": len(dts) / sum(dts), "unit": "tokens/s",
                   "ms_per_step": statistics.mean(dts) * 1e3, "load_and_pack_s": load_s, "prefill_64_tokens_s": prefill_s,
                   "sample": f"reference RWKV('cpu fp32i8') on the 169M shape: 64-token prompt, {len(dts)} greedy steps timed"}
        else:
            Lfull, D, Fn, V = synth.SHAPES[a.shape]
            version = 6 if a.shape.startswith("v6") else 4
            per = {}
            for L in (1, 2):
                model, _ = _model(version, L, D, Fn, V, 1002, tmp)
                logits, state = model.forward([1, 2, 3], None)
                dts = _steps(model, state, int(torch.argmax(logits)), a.steps, a.warmup)
                per[L] = dts
                del model
            t1, t2 = statistics.mean(per[1]), statistics.mean(per[2])
            step = [t1_ + (Lfull - 1) * max(t2_ - t1_, 0.0) for t1_, t2_ in zip(per[1], per[2])]
            full = t1 + (Lfull - 1) * max(t2 - t1, 0.0)
            out = {"kind": "reference", "mode": "token7b", "cores": cores, "value": 1.0 / full, "unit": "tokens/s",
                   "ms_per_step": full * 1e3, "ms_per_step_samples": [s * 1e3 for s in step],
                   "sample": f"reference RWKV('cpu fp32i8') at the {a.shape} width with 1 and 2 layers (+ embedding and head), "
                             f"{len(per[1])} one-token steps each: {t1 * 1e3:.0f} ms and {t2 * 1e3:.0f} ms per step; a "
                             f"{Lfull}-layer token extrapolated as t1 + {Lfull - 1} x (t2 - t1)"}
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
