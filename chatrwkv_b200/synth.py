"""Seeded random-init RWKV checkpoints with the key names and shapes the loader expects.

There is no network for trained checkpoints, so every parity case and benchmark uses
weights drawn from fixed distributions: matrices N(0, 0.02) fp32, LayerNorm weight 1 /
bias 0, time_decay U(-5, 1), time_first / time_faaaa U(-1, 1), time_mix_* / time_maa_*
U(0, 1), RWKV-6 LoRA matrices N(0, 0.01).

The key layout follows what `RWKV.__init__` sniffs in the reference loader
(rwkv_pip_package/src/rwkv/model.py:658-680): `ln_x` -> v5, `gate.weight` -> v5.1,
2-D `att.time_decay` with a second dimension > 1 -> v5.2, `time_maa` -> v6,
`time_faaaa` -> n_head.
"""
from __future__ import annotations

import torch

SHAPES = {
    # name: (n_layer, n_embd, n_ffn, vocab)
    "v4-169m": (12, 768, 3072, 50277),
    "v4-7b": (32, 4096, 16384, 50277),
    "v4-14b": (40, 5120, 20480, 50277),
    "v6-7b": (32, 4096, 14336, 65536),
}

# RWKV-6 LoRA ranks of the random-init 7B-shape model (the loader is shape-agnostic).
V6_MAA_RANK = 32
V6_DECAY_RANK = 64


def _normal(gen, shape, std, device, dtype):
    return torch.empty(shape, device=device, dtype=dtype).normal_(0.0, std, generator=gen)


def _uniform(gen, shape, lo, hi, device, dtype):
    return torch.empty(shape, device=device, dtype=dtype).uniform_(lo, hi, generator=gen)


def make_checkpoint(version, n_layer, n_embd, n_ffn, vocab, seed, *, head_size=64,
                    maa_rank=V6_MAA_RANK, decay_rank=V6_DECAY_RANK,
                    device="cpu", dtype=torch.float32):
    """Return a raw (un-converted) checkpoint dict for RWKV `version` in {4, 5.2, 6}.

    Matrices are stored `[out_features, in_features]` like `nn.Linear.weight`; the loader
    transposes them (model.py:793-794).
    """
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    D, F_, V = n_embd, n_ffn, vocab
    kw = dict(device=device, dtype=dtype)
    w = {}
    w["emb.weight"] = _normal(gen, (V, D), 0.02, **kw)
    w["blocks.0.ln0.weight"] = torch.ones(D, **kw)
    w["blocks.0.ln0.bias"] = torch.zeros(D, **kw)
    H = D // head_size
    for i in range(n_layer):
        b = f"blocks.{i}."
        w[b + "ln1.weight"] = torch.ones(D, **kw)
        w[b + "ln1.bias"] = torch.zeros(D, **kw)
        w[b + "ln2.weight"] = torch.ones(D, **kw)
        w[b + "ln2.bias"] = torch.zeros(D, **kw)
        a = b + "att."
        if version == 4:
            w[a + "time_decay"] = _uniform(gen, (D,), -5.0, 1.0, **kw)
            w[a + "time_first"] = _uniform(gen, (D,), -1.0, 1.0, **kw)
            for n in ("k", "v", "r"):
                w[a + f"time_mix_{n}"] = _uniform(gen, (1, 1, D), 0.0, 1.0, **kw)
        elif version == 5.2:
            for n in ("k", "v", "r", "g"):
                w[a + f"time_mix_{n}"] = _uniform(gen, (1, 1, D), 0.0, 1.0, **kw)
            w[a + "ln_x.weight"] = torch.ones(D, **kw)
            w[a + "ln_x.bias"] = torch.zeros(D, **kw)
            w[a + "time_decay"] = _uniform(gen, (H, head_size), -5.0, 1.0, **kw)
            w[a + "time_faaaa"] = _uniform(gen, (H, head_size), -1.0, 1.0, **kw)
        elif version == 6:
            for n in ("x", "w", "k", "v", "r", "g"):
                w[a + f"time_maa_{n}"] = _uniform(gen, (1, 1, D), 0.0, 1.0, **kw)
            w[a + "time_maa_w1"] = _normal(gen, (D, 5 * maa_rank), 0.01, **kw)
            w[a + "time_maa_w2"] = _normal(gen, (5, maa_rank, D), 0.01, **kw)
            w[a + "time_decay_w1"] = _normal(gen, (D, decay_rank), 0.01, **kw)
            w[a + "time_decay_w2"] = _normal(gen, (decay_rank, D), 0.01, **kw)
            w[a + "time_decay"] = _uniform(gen, (1, 1, D), -5.0, 1.0, **kw)
            w[a + "time_faaaa"] = _uniform(gen, (H, head_size), -1.0, 1.0, **kw)
            w[a + "ln_x.weight"] = torch.ones(D, **kw)
            w[a + "ln_x.bias"] = torch.zeros(D, **kw)
        else:
            raise ValueError(f"unsupported version {version}")
        for n in ("key", "value", "receptance", "output"):
            w[a + n + ".weight"] = _normal(gen, (D, D), 0.02, **kw)
        if version != 4:
            w[a + "gate.weight"] = _normal(gen, (D, D), 0.02, **kw)
        f = b + "ffn."
        if version == 6:
            w[f + "time_maa_k"] = _uniform(gen, (1, 1, D), 0.0, 1.0, **kw)
            w[f + "time_maa_r"] = _uniform(gen, (1, 1, D), 0.0, 1.0, **kw)
        else:
            w[f + "time_mix_k"] = _uniform(gen, (1, 1, D), 0.0, 1.0, **kw)
            w[f + "time_mix_r"] = _uniform(gen, (1, 1, D), 0.0, 1.0, **kw)
        w[f + "key.weight"] = _normal(gen, (F_, D), 0.02, **kw)
        w[f + "receptance.weight"] = _normal(gen, (D, D), 0.02, **kw)
        w[f + "value.weight"] = _normal(gen, (D, F_), 0.02, **kw)
    w["ln_out.weight"] = torch.ones(D, **kw)
    w["ln_out.bias"] = torch.zeros(D, **kw)
    w["head.weight"] = _normal(gen, (V, D), 0.02, **kw)
    return w


def make_tokens(n, vocab, seed):
    """`n` seeded uniform token ids in [0, vocab) as a Python list."""
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=gen).tolist()
