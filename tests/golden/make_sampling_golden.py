"""Writes tests/golden/sampling_reference.npz by RUNNING THE REFERENCE's PIPELINE.sample_logits
(rwkv_pip_package/src/rwkv/utils.py:55-75, its CPU branch) on seeded logits, with `np.random.choice` replaced
by a recorder so that the probabilities it would draw from are kept.  Needs the reference tree:

    RWKV_REFERENCE_ROOT=<path to the ChatRWKV checkout> python tests/golden/make_sampling_golden.py
"""
import os
import sys

import numpy as np
import torch


def main():
    root = os.environ["RWKV_REFERENCE_ROOT"]
    sys.path.insert(0, os.path.join(root, "rwkv_pip_package", "src"))
    from rwkv import utils as ref_utils

    recorded = []

    def recorder(a, p):
        recorded.append(np.array(p, dtype=np.float64))
        return 0

    ref_utils.np.random.choice = recorder
    cases = []
    g = torch.Generator().manual_seed(4000)
    V = 3000
    settings = [(1.0, 0.85, 0), (1.0, 0.5, 0), (0.7, 0.9, 0), (1.5, 0.3, 0), (1.0, 0.95, 40), (0.8, 0.999, 5),
                (0.0, 0.85, 0), (1.0, 0.0, 0), (1.0, 0.2, 1), (2.0, 0.6, 200)]
    for i, (temperature, top_p, top_k) in enumerate(settings):
        scale = (0.5, 2.0, 6.0)[i % 3]              # flat, medium and peaked distributions
        logits = (torch.randn(V, generator=g) * scale).float()
        if i == 4:
            logits[100:110] = logits[100]           # ties
        ref_utils.PIPELINE.sample_logits(None, logits.clone(), temperature=temperature, top_p=top_p, top_k=top_k)
        cases.append((logits.numpy(), temperature, top_p, top_k, recorded[-1]))
    out = {}
    for i, (lg, t, p, k, pr) in enumerate(cases):
        out[f"logits_{i}"] = lg
        out[f"params_{i}"] = np.array([t, p, k], dtype=np.float64)
        out[f"probs_{i}"] = pr
    out["n"] = np.array(len(cases))
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "sampling_reference.npz"), **out)
    print("wrote", len(cases), "cases")


if __name__ == "__main__":
    main()
