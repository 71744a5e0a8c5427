"""The sampling oracle (oracle/sampling_oracle.py) against what the reference's own PIPELINE.sample_logits
computed (tests/golden/sampling_reference.npz, recorded by tests/golden/make_sampling_golden.py)."""
import os

import numpy as np

from oracle import sampling_oracle as so

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "sampling_reference.npz")


def test_filtered_probs_match_the_reference():
    g = np.load(GOLD)
    for i in range(int(g["n"])):
        t, p, k = g[f"params_{i}"]
        mine = so.filtered_probs(g[f"logits_{i}"], t, p, int(k))
        ref = g[f"probs_{i}"]
        assert np.array_equal(mine > 0, ref > 0), i
        assert np.allclose(mine, ref, rtol=1e-5, atol=1e-9), i


def test_occurrence_bookkeeping():
    occ = so.Occurrence(alpha_presence=0.3, alpha_frequency=0.1, alpha_decay=0.5, token_ban=[2])
    x = np.zeros(5, dtype=np.float32)
    assert np.isneginf(occ.apply(x)[2])
    occ.update(1)
    occ.update(1)          # 1 * 0.5 + 1
    occ.update(3)          # token 1 decays to 0.75
    y = occ.apply(x)
    assert np.isclose(y[1], -(0.3 + 0.75 * 0.1)) and np.isclose(y[3], -(0.3 + 1 * 0.1)) and y[0] == 0


def test_inverse_cdf():
    p = np.array([0.0, 0.25, 0.0, 0.75])
    assert so.inverse_cdf(p, 0.0) == 1 and so.inverse_cdf(p, 0.24) == 1 and so.inverse_cdf(p, 0.26) == 3 and so.inverse_cdf(p, 0.999) == 3
