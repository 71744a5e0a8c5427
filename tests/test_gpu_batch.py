"""Batched decode (RWKV.forward_batch: B independent sequences, one token each per call) against the same
sequences decoded one by one with RWKV.forward and against the CPU oracle.  Tolerance on logits: max-abs 2e-2."""
import copy

import pytest
import torch

from chatrwkv_b200 import synth
from oracle import rwkv_oracle as orc
from tests.golden.make_golden import TOY

pytestmark = pytest.mark.gpu
TOL = 2e-2


@pytest.mark.parametrize("B", [3, 9])
@pytest.mark.parametrize("name", ["v4", "v5", "v6"])
def test_forward_batch_matches_per_sequence_decode(name, B):
    """B = 3 runs the CUDA-core mm8_seq kernel, B = 9 the tensor-core one.  Sequences start from different prompts
    (stack_states of B prefills), decode 6 tokens each."""
    from chatrwkv_b200.model import RWKV
    ck = synth.make_checkpoint(**TOY[name])
    V = TOY[name]["vocab"]
    model = RWKV(copy.deepcopy(ck), "cuda fp16i8", verbose=False)
    oracle = orc.OracleRWKV(ck, atype=torch.float16)
    prompts = [synth.make_tokens(3 + b % 4, V, 100 + b) for b in range(B)]
    steps = [synth.make_tokens(6, V, 200 + b) for b in range(B)]
    states, ostates = [], []
    for p in prompts:
        _, s = model.forward(p, None)
        states.append(copy.deepcopy(s))
        _, so = oracle.forward(p, None)
        ostates.append(so)
    bstate = model.stack_states(states)
    for t in range(6):
        toks = [steps[b][t] for b in range(B)]
        logits, bstate = model.forward_batch(toks, bstate)
        assert logits.shape == (B, V) and logits.dtype == torch.float32
        for b in range(B):
            lo, ostates[b] = oracle.forward([toks[b]], ostates[b])
            assert (logits[b].cpu() - lo).abs().max().item() < TOL, (t, b)
            l1, states[b] = model.forward([toks[b]], states[b])
            states[b] = copy.deepcopy(states[b])
            assert (logits[b] - l1).abs().max().item() < TOL, (t, b)
    # the batch state splits back into ordinary state lists
    per_seq = model.unstack_states(bstate)
    for b in range(B):
        for j, (x, y) in enumerate(zip(per_seq[b], ostates[b])):
            x, y = x.float().cpu(), y.float()
            m = y > -1e29
            assert (x[m] - y[m].contiguous()).abs().max().item() <= 2e-2 * max(1.0, y[m].abs().max().item()), (b, j)


def test_forward_batch_from_zero_state():
    from chatrwkv_b200.model import RWKV
    ck = synth.make_checkpoint(**TOY["v4"])
    model = RWKV(copy.deepcopy(ck), "cuda fp16i8", verbose=False)
    oracle = orc.OracleRWKV(ck, atype=torch.float16)
    toks = [5, 17, 5, 250]
    logits, st = model.forward_batch(toks, None)
    for b, t in enumerate(toks):
        lo, _ = oracle.forward([t], None)
        assert (logits[b].cpu() - lo).abs().max().item() < TOL
    assert torch.equal(logits[0], logits[2])


def test_forward_batch_graph_and_eager_agree(monkeypatch):
    """The CUDA-graph replay (default) and direct launches give the same bits; a state list from another source
    (a snapshot) can be passed back in."""
    from chatrwkv_b200.model import RWKV
    ck = synth.make_checkpoint(**TOY["v6"])
    mg = RWKV(copy.deepcopy(ck), "cuda fp16i8", verbose=False)
    monkeypatch.setenv("RWKV_B200_BATCH_GRAPH", "0")
    me = RWKV(copy.deepcopy(ck), "cuda fp16i8", verbose=False)
    monkeypatch.setenv("RWKV_B200_BATCH_GRAPH", "1")
    sg = se = None
    toks = [[3, 9, 27, 81, 243, 1, 2, 4, 8], [5, 25, 125, 7, 49, 11, 121, 13, 169]]
    snap = None
    for step in range(4):
        t = toks[step % 2]
        lg, sg = mg.forward_batch(t, sg)
        le, se = me.forward_batch(t, se)
        assert torch.equal(lg, le), step
        if step == 1:
            snap = copy.deepcopy(sg)
            keep = lg.clone()
    l2, _ = mg.forward_batch(toks[1], copy.deepcopy(snap))      # not the graph's own output list: copied in
    l3, _ = me.forward_batch(toks[1], copy.deepcopy(snap))
    assert torch.equal(l2, l3)
