"""Pins the CPU oracle to outputs of the reference executed on CPU (tests/golden)."""
import numpy as np
import pytest
import torch

from chatrwkv_b200 import synth
from oracle import rwkv_oracle as orc
from tests.golden.make_golden import TOY, TOKENS


def _t(a, f16=False):
    t = torch.from_numpy(np.ascontiguousarray(a))
    return t.view(torch.float16) if f16 else t


@pytest.mark.parametrize("tag,atype,rescale", [("f32", torch.float32, 0), ("f16", torch.float16, 6)])
def test_packing_bit_exact(golden, tag, atype, rescale):
    ck = synth.make_checkpoint(**TOY["v4"])
    for key in ("blocks.0.att.key.weight", "blocks.7.att.output.weight",
                "blocks.0.ffn.key.weight", "blocks.7.ffn.value.weight", "head.weight"):
        w = ck[key]
        layer = int(key.split(".")[1]) if key.startswith("blocks.") else 0
        if rescale and ("att.output" in key or "ffn.value" in key):
            w = w / (2 ** (layer // rescale))
        q, mx, rx, my, ry = orc.quantize_weight(w.t(), atype)
        f16 = atype == torch.float16
        assert torch.equal(q, _t(golden[f"pack/{tag}/{key}"])), key
        for name, v in (("_mx", mx), ("_rx", rx), ("_my", my), ("_ry", ry)):
            ref = _t(golden[f"pack/{tag}/{key}{name}"], f16)
            assert v.shape == ref.shape, (key, name)
            a = v.view(torch.int16) if f16 else v.view(torch.int32)
            b = ref.view(torch.int16) if f16 else ref.view(torch.int32)
            assert torch.equal(a, b), (key, name)


def test_mm8_spec(golden):
    ck = synth.make_checkpoint(**TOY["v4"])
    for key in ("blocks.0.ffn.key.weight", "blocks.0.ffn.value.weight", "head.weight"):
        q, mx, rx, my, ry = orc.quantize_weight(ck[key].t(), torch.float32)
        x1, xs = _t(golden[f"mm8/{key}/x1"]), _t(golden[f"mm8/{key}/xs"])
        y1, ys = _t(golden[f"mm8/{key}/y1"]), _t(golden[f"mm8/{key}/ys"])
        assert torch.equal(orc.mm8_spec(x1, q, mx, rx, my, ry), y1)
        assert torch.equal(orc.mm8_spec(xs, q, mx, rx, my, ry), ys)
        # the kernel-arithmetic restatement agrees with the spec to fp32 round-off
        torch.testing.assert_close(orc.mm8_kernel(x1, q, mx, rx, my, ry), y1, rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(orc.mm8_kernel(xs, q, mx, rx, my, ry), ys, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("name", ["v4", "v5", "v6"])
def test_model_logits_and_state(golden, name):
    ck = synth.make_checkpoint(**TOY[name])
    m = orc.OracleRWKV(ck, atype=torch.float32)
    tol = dict(rtol=2e-4, atol=2e-5)
    full, st = m.forward(TOKENS, None, full_output=True)
    torch.testing.assert_close(full, _t(golden[f"model/{name}/full"]), **tol)
    for j, s in enumerate(st):
        torch.testing.assert_close(s.float().contiguous(), _t(golden[f"model/{name}/state_full/{j}"]), **tol)
    o, st = m.forward(TOKENS[:5], None)
    torch.testing.assert_close(o, _t(golden[f"model/{name}/split_a"]), **tol)
    o, st = m.forward(TOKENS[5:6], st)
    torch.testing.assert_close(o, _t(golden[f"model/{name}/split_b"]), **tol)
    o, st = m.forward(TOKENS[6:], st)
    torch.testing.assert_close(o, _t(golden[f"model/{name}/split_c"]), **tol)
    st = None
    for i, t in enumerate(TOKENS):
        o, st = m.forward([t], st)
        torch.testing.assert_close(o, _t(golden[f"model/{name}/one"][i]), **tol)
    for j, s in enumerate(st):
        torch.testing.assert_close(s.float().contiguous(), _t(golden[f"model/{name}/state_one/{j}"]), **tol)


def test_fp16_path_tracks_fp32_path():
    """The fp16 ('cuda fp16i8' arithmetic) oracle stays close to the fp32 one on a toy model:
    guards the rounding-point emulation against gross mistakes (rescale, state dtypes)."""
    for name in ("v4", "v6"):
        ck = synth.make_checkpoint(**TOY[name])
        a = orc.OracleRWKV(ck, atype=torch.float32)
        b = orc.OracleRWKV(ck, atype=torch.float16)
        la, _ = a.forward(TOKENS, None)
        lb, _ = b.forward(TOKENS, None)
        assert (la - lb).abs().max() < 2e-2


def test_reference_converted_checkpoint_matches_oracle_packing():
    """Every packed matrix (and its four scale vectors) in the checkpoint the reference's own loader
    converted for 'cuda fp16i8' equals the oracle's packing of the raw checkpoint, bit for bit."""
    import os
    path = os.path.join(os.path.dirname(__file__), "golden", "ref_converted_v4.pth")
    conv = torch.load(path, map_location="cpu")
    assert conv["_strategy"] == "cuda fp16i8" and conv["_rescale_layer"] == 6
    ck = synth.make_checkpoint(**TOY["v4"])
    n = 0
    for key, t in conv.items():
        if not (torch.is_tensor(t) and t.dtype == torch.uint8):
            continue
        w = ck[key].float()
        layer = int(key.split(".")[1]) if key.startswith("blocks.") else 0
        if "att.output" in key or "ffn.value" in key:
            w = w / (2 ** (layer // 6))
        q, mx, rx, my, ry = orc.quantize_weight(w.t(), torch.float16)
        assert torch.equal(q, t), key
        for name, v in (("_mx", mx), ("_rx", rx), ("_my", my), ("_ry", ry)):
            ref = conv[key + name]
            assert v.shape == ref.shape and torch.equal(v.view(torch.int16), ref.view(torch.int16)), (key, name)
        n += 1
    assert n == 8 * 7 + 1


def test_plain_and_mixed_strategies_match_the_reference():
    """Unquantised layers ('cpu fp32') and the per-layer split of 'cpu fp32i8 *2 -> cpu fp32', against logits the
    reference produced (tests/golden/reference_cpu_plain.npz, made by tests/golden/make_plain_golden.py)."""
    import os
    import numpy as np
    from chatrwkv_b200 import synth
    from tests.golden.make_golden import TOKENS, TOY
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_cpu_plain.npz"))
    for name in ("v4", "v6"):
        for tag, k in (("plain", 0), ("mixed", 2)):
            m = orc.OracleRWKV(synth.make_checkpoint(**TOY[name]), atype=torch.float32, i8_layers=k)
            full, _ = m.forward(TOKENS, None, full_output=True)
            assert torch.allclose(full, torch.from_numpy(g[f"{name}/{tag}/full"]), rtol=2e-4, atol=2e-5), (name, tag)
            st = None
            for i, t in enumerate(TOKENS):
                o, st = m.forward([t], st)
                assert torch.allclose(o, torch.from_numpy(g[f"{name}/{tag}/one"][i]), rtol=2e-4, atol=2e-5), (name, tag, i)
