"""The strategies without int8, 'cuda fp16' and the per-layer split 'cuda fp16i8 *K -> cuda fp16'
(rwkv_pip_package/src/rwkv/model.py:684-749, 143-167): plain fp16 layers run as library GEMMs plus the reference's
pointwise ops, int8 layers on the kernels of this library.  Checked against the oracle with the same per-layer weight
types (pinned to the reference by tests/golden/reference_cpu_plain.npz); logits max-abs 2e-2 as everywhere."""
import copy

import pytest
import torch

from chatrwkv_b200 import synth
from oracle import rwkv_oracle as orc
from tests.golden.make_golden import TOY

pytestmark = pytest.mark.gpu
TOL = 2e-2


@pytest.mark.parametrize("name", ["v4", "v6", "v5"])
@pytest.mark.parametrize("strategy,k", [("cuda fp16", 0), ("cuda fp16i8 *2 -> cuda fp16", 2)])
def test_plain_and_mixed_strategies(name, strategy, k):
    from chatrwkv_b200.model import RWKV
    ck = synth.make_checkpoint(**TOY[name])
    tokens = synth.make_tokens(14, TOY[name]["vocab"], 21)
    oracle = orc.OracleRWKV(copy.deepcopy(ck), atype=torch.float16, i8_layers=k)
    model = RWKV(copy.deepcopy(ck), strategy, verbose=False)
    L = model.args.n_layer
    assert [s.wtype for s in model.strategy] == [torch.uint8] * k + [torch.float16] * (L + 1 - k)
    assert model.w["head.weight"].dtype == torch.float16
    assert (model.w["blocks.0.att.key.weight"].dtype == torch.uint8) == (k > 0)
    lo, so = oracle.forward(tokens[:9], None)
    lg, sg = model.forward(tokens[:9], None)
    assert (lg.cpu() - lo).abs().max().item() < TOL
    for t in tokens[9:]:
        lo, so = oracle.forward([t], so)
        lg, sg = model.forward([t], sg)
        assert (lg.cpu() - lo).abs().max().item() < TOL
    full_o, _ = oracle.forward(tokens, None, full_output=True)
    full_g, _ = model.forward(tokens, None, full_output=True)
    assert full_g.shape == full_o.shape and (full_g.cpu() - full_o).abs().max().item() < TOL
    for a, b in zip(sg, so):
        scale = max(1.0, b.float().abs().max().item()) if b.float().abs().max().item() < 1e20 else 1e30
        assert (a.float().cpu() - b.float()).abs().max().item() <= 2e-2 * scale


def test_converted_fp16_checkpoint_round_trip(tmp_path):
    """A model loaded as 'cuda fp16' exports the reference's pre-converted format and loads it back unchanged."""
    from chatrwkv_b200.model import RWKV
    ck = synth.make_checkpoint(**TOY["v4"])
    tokens = synth.make_tokens(6, TOY["v4"]["vocab"], 5)
    a = RWKV(copy.deepcopy(ck), "cuda fp16", verbose=False)
    path = str(tmp_path / "conv.pth")
    torch.save(a.export_converted(), path)
    b = RWKV(path, "cuda fp16", verbose=False)
    la, _ = a.forward(tokens, None)
    lb, _ = b.forward(tokens, None)
    assert torch.equal(la, lb)


def test_other_strategies_still_refused():
    from chatrwkv_b200.model import RWKV
    ck = synth.make_checkpoint(**TOY["v4"])
    for s in ("cpu fp32", "cuda fp32", "cuda bf16", "cuda:0 fp16i8 -> cuda:1 fp16", "cuda fp16i8 *4+"):
        with pytest.raises(NotImplementedError):
            RWKV(copy.deepcopy(ck), s, verbose=False)
