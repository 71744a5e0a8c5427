"""CPU restatement of the reference's sampler, for tests only (the product never imports this).

`filtered_probs` follows the CPU branch of PIPELINE.sample_logits (rwkv_pip_package/src/rwkv/utils.py:55-75)
up to the draw and returns the distribution `np.random.choice` is given; `Occurrence` follows the penalty
bookkeeping of PIPELINE.generate (utils.py:97-100, 111-122).  Pinned against the reference itself by
tests/golden/sampling_reference.npz (made by tests/golden/make_sampling_golden.py, which runs the reference's
function with `np.random.choice` replaced by a recorder)."""
import numpy as np


def softmax_f32(logits):
    x = np.asarray(logits, dtype=np.float32)
    m = np.max(x)
    if not np.isfinite(m):
        m = np.float32(0.0)
    e = np.exp(x - m, dtype=np.float32)
    return e / np.sum(e, dtype=np.float32)


def filtered_probs(logits, temperature=1.0, top_p=0.85, top_k=0):
    """utils.py:55-75: the normalised probabilities the token is drawn from."""
    if temperature == 0:
        temperature = 1.0
        top_p = 0
    probs = softmax_f32(logits)
    top_k = int(top_k)
    sorted_ids = np.argsort(probs)
    sorted_probs = probs[sorted_ids][::-1]
    cumulative_probs = np.cumsum(sorted_probs)
    cutoff = float(sorted_probs[np.argmax(cumulative_probs >= top_p)])
    probs[probs < cutoff] = 0
    if top_k < len(probs) and top_k > 0:
        probs[sorted_ids[:-top_k]] = 0
    if temperature != 1.0:
        probs = probs ** (1.0 / temperature)
    return probs / np.sum(probs)


def inverse_cdf(probs, u):
    """The id an inverse-CDF walk in id order picks for the uniform number u (how the product draws)."""
    c = np.cumsum(np.asarray(probs, dtype=np.float64))
    return int(min(np.searchsorted(c, u * c[-1], side="right"), len(probs) - 1))


class Occurrence:
    """utils.py:97-100 (apply) and 111-122 (update)."""

    def __init__(self, alpha_presence=0.2, alpha_frequency=0.2, alpha_decay=0.996, token_ban=(), token_weight=None):
        self.ap, self.af, self.ad = alpha_presence, alpha_frequency, alpha_decay
        self.ban = list(token_ban)
        self.weight = token_weight
        self.occurrence = {}

    def apply(self, logits):
        out = np.array(logits, dtype=np.float32, copy=True)
        for n in self.ban:
            out[n] = -np.inf
        for n, c in self.occurrence.items():
            out[n] -= np.float32(self.ap + c * self.af)
        return out

    def update(self, token):
        for k in self.occurrence:
            self.occurrence[k] *= self.ad
        w = 1 if self.weight is None else self.weight[token]
        self.occurrence[token] = self.occurrence.get(token, 0) + w
