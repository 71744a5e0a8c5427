"""rwkv_sample_logits / chatrwkv_b200.pipeline against the reference's sampler: the distributions recorded from
PIPELINE.sample_logits itself (tests/golden/sampling_reference.npz) and, at the vocabulary sizes of the models,
the CPU restatement (oracle/sampling_oracle.py).  Probabilities within 1e-4 relative (fp32 sums in another order);
the kept set may differ from the reference's by the single value on which a cumulative sum hinges."""
import os

import numpy as np
import pytest
import torch

from oracle import sampling_oracle as so

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "sampling_reference.npz")


def _gpu_probs(logits, t, p, k, u=0.5, sampler=None, penalties=False):
    from chatrwkv_b200.pipeline import PIPELINE_ARGS, Sampler
    lg = torch.as_tensor(logits, dtype=torch.float32).cuda().contiguous()
    s = sampler or Sampler(lg.numel(), "cuda", PIPELINE_ARGS())
    out = torch.full((lg.numel(),), -1.0, dtype=torch.float32, device="cuda")
    un = torch.tensor([u], dtype=torch.float32, device="cuda")
    tok = s.sample(lg, probs_out=out, penalties=penalties, temperature=t, top_p=p, top_k=k, uniforms=un)
    return out.cpu().numpy().astype(np.float64), int(tok.item())


def _same_distribution(mine, ref, what):
    differ = np.flatnonzero((mine > 0) != (ref > 0))
    assert len(differ) <= 1, f"{what}: kept sets differ at {differ[:8]}"
    if len(differ) == 1:        # the value the cutoff hinged on: renormalise both over the common support
        keep = (mine > 0) & (ref > 0)
        mine, ref = np.where(keep, mine, 0), np.where(keep, ref, 0)
        mine, ref = mine / mine.sum(), ref / ref.sum()
    assert np.allclose(mine, ref, rtol=1e-4, atol=1e-9), what


def test_distributions_recorded_from_the_reference():
    g = np.load(GOLD)
    for i in range(int(g["n"])):
        t, p, k = g[f"params_{i}"]
        mine, tok = _gpu_probs(g[f"logits_{i}"], float(t), float(p), int(k))
        if i == 4:              # ties at the top-k boundary are kept by lowest id here, by sort order there: compare the sorted values
            assert np.allclose(np.sort(mine), np.sort(g[f"probs_{i}"]), rtol=1e-4, atol=1e-9)
        else:
            _same_distribution(mine, g[f"probs_{i}"], f"case {i}")
        assert mine[tok] > 0 and abs(mine.sum() - 1) < 1e-5


@pytest.mark.parametrize("V", [50277, 65536, 1000, 17])
@pytest.mark.parametrize("t,p,k", [(1.0, 0.85, 0), (0.7, 0.5, 0), (1.3, 0.95, 50), (1.0, 0.999, 3)])
def test_model_vocabularies_against_the_oracle(V, t, p, k):
    g = torch.Generator().manual_seed(V + k)
    logits = (torch.randn(V, generator=g) * 3.0).float().numpy()
    ref = so.filtered_probs(logits, t, p, k)
    for u in (0.0, 0.37, 0.999):
        mine, tok = _gpu_probs(logits, t, p, k, u)
        _same_distribution(mine, ref, f"V={V}")
        want = so.inverse_cdf(mine, u)
        kept = np.flatnonzero(mine > 0)
        pos = {int(v): j for j, v in enumerate(kept)}
        assert abs(pos[tok] - pos[want]) <= 1          # a boundary of the CDF may round either way


def test_greedy_and_bans():
    from chatrwkv_b200.pipeline import PIPELINE_ARGS, Sampler
    g = torch.Generator().manual_seed(5)
    logits = torch.randn(50277, generator=g).float()
    best = int(logits.argmax())
    mine, tok = _gpu_probs(logits.numpy(), 0.0, 0.85, 0, u=0.0)
    assert tok == best and mine[best] == 1.0
    s = Sampler(50277, "cuda", PIPELINE_ARGS(token_ban=[best]))
    mine, tok = _gpu_probs(logits.numpy(), 0.0, 0.85, 0, u=0.0, sampler=s)
    assert tok != best and mine[best] == 0.0 and tok == int(torch.topk(logits, 2).indices[1])


def test_penalties_follow_the_reference_bookkeeping():
    from chatrwkv_b200.pipeline import PIPELINE_ARGS, Sampler
    V = 2000
    args = PIPELINE_ARGS(temperature=1.0, top_p=0.9, top_k=0, alpha_frequency=0.4, alpha_presence=0.3, alpha_decay=0.9, token_ban=[7])
    weight = torch.ones(V)
    weight[::5] = 0.0
    s = Sampler(V, "cuda", args, seed=3, token_weight=weight)
    occ = so.Occurrence(0.3, 0.4, 0.9, [7], weight.numpy())
    g = torch.Generator().manual_seed(11)
    base = torch.randn(V, generator=g).float() * 4.0
    for step in range(12):
        logits = base + 0.01 * step
        u = float(torch.rand(1, generator=g))
        mine, tok = _gpu_probs(logits.numpy(), 1.0, 0.9, 0, u, sampler=s, penalties=True)
        ref = so.filtered_probs(occ.apply(logits.numpy()), 1.0, 0.9, 0)
        _same_distribution(mine, ref, f"step {step}")
        assert mine[7] == 0.0
        occ.update(tok)
    table = s.occurrence.cpu().numpy()
    for k, v in occ.occurrence.items():
        assert abs(table[k] - v) < 1e-5 and int(s.seen[k]) == 1
    assert int(s.seen.sum()) == len(occ.occurrence)


def test_vocabulary_limit():
    from chatrwkv_b200 import _lib
    lg = torch.zeros(70000, device="cuda")
    tok = torch.zeros(1, dtype=torch.int64, device="cuda")
    rc = _lib.lib().rwkv_sample_logits(70000, lg.data_ptr(), 1.0, 0.85, 0, None, None, None, None, 0.0, 0.0, 1.0, None, 0, None,
                                       tok.data_ptr(), None, torch.cuda.current_stream().cuda_stream)
    assert rc == _lib.ERR_UNSUPPORTED


def test_generation_loops_agree():
    """`generate` (token to the host every step) and `generate_tokens` (token stays on the device) produce the same
    ids from the same seed; stop tokens cut the result; banned tokens never appear."""
    from chatrwkv_b200 import synth
    from chatrwkv_b200.model import RWKV
    from chatrwkv_b200.pipeline import PIPELINE, PIPELINE_ARGS
    ck = synth.make_checkpoint(4, 2, 256, 1024, 500, seed=77, device="cuda")
    model = RWKV(ck, "cuda fp16i8", verbose=False)
    prompt = synth.make_tokens(40, 500, 3)
    args = PIPELINE_ARGS(temperature=1.2, top_p=0.9, top_k=60, token_ban=[1, 2, 3], chunk_len=16)
    a = PIPELINE(model, seed=9).generate(prompt, 24, args)
    b, _ = PIPELINE(model, seed=9).generate_tokens(prompt, 24, args)
    assert a == b and len(a) == 24 and not (set(a) & {1, 2, 3})
    c = PIPELINE(model, seed=10).generate(prompt, 24, args)
    assert c != a
    args.token_stop = [a[5]]
    first = a.index(a[5])
    d = PIPELINE(model, seed=9).generate(prompt, 24, args)
    e, _ = PIPELINE(model, seed=9).generate_tokens(prompt, 24, args)
    assert d == a[:first] and e == a[:first]
    g = PIPELINE(model, seed=9)
    assert g.sample_logits(torch.tensor([0.0, 5.0, 1.0]), temperature=0.0, u=0.0) == 1
