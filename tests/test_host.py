"""CPU-side checks: the C-ABI library loads and exports every declared symbol, the
operators are registered with the reference's signatures, and the host logic rejects what it
does not implement.  No kernel is launched here."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "rwkv_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rwkv_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from chatrwkv_b200 import _lib
    if not os.path.exists(_lib.LIB_PATH):
        from chatrwkv_b200.build import build_library
        build_library()
    handle = ctypes.CDLL(_lib.LIB_PATH)
    names = _declared_symbols()
    assert len(names) >= 14
    for n in names:
        assert hasattr(handle, n), n
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert _lib.lib().rwkv_b200_version() >= 1000
    assert b"workspace" in _lib.lib().rwkv_b200_error_string(-3)


def test_argument_errors_without_gpu():
    """Argument validation happens before any CUDA call."""
    from chatrwkv_b200 import _lib
    L = _lib.lib()
    assert L.rwkv_mm8_one(0, 16, None, None, 16, None, None, None, None, _lib.F16, None, None, 0, None) == -1
    assert L.rwkv_mm8_seq(1, 16, 16, None, 16, None, 16, None, None, None, None, _lib.F16, None, 16, None, 0, None) == -1
    assert L.rwkv_wkv6_forward(2, 1, 64, 1, None, None, None, None, None, None, None, _lib.F32, None) == -1
    assert L.rwkv_quantize_weight_workspace_bytes(4096, 4096) > 0
    assert L.rwkv_mm8_one_workspace_bytes(4096, 50277) >= 64 * 50688 * 4


def test_ops_registered_with_reference_signatures():
    from chatrwkv_b200 import ops  # noqa: F401
    s = str(torch.ops.rwkv.mm8_one.default._schema)
    assert re.match(r"rwkv::mm8_one\(int N, int M, Tensor x, Tensor w, Tensor mx, Tensor rx, Tensor my, Tensor ry, Tensor\(a!\) y\) -> \(\)", s), s
    s = str(torch.ops.rwkv.mm8_seq.default._schema)
    assert s.startswith("rwkv::mm8_seq(int B, int N, int M, Tensor x, Tensor w, Tensor mx, Tensor rx, Tensor my, Tensor ry"), s
    s = str(torch.ops.rwkv.wkv_forward.default._schema)
    assert s.startswith("rwkv::wkv_forward(int B, int T, int C, Tensor w, Tensor u, Tensor k, Tensor v"), s
    for which in (5, 6):
        for suf in ("bf16", "fp16", "fp32"):
            s = str(getattr(getattr(torch.ops, f"rwkv{which}"), f"forward_{suf}").default._schema)
            assert s.startswith(f"rwkv{which}::forward_{suf}(int B, int T, int C, int H, Tensor(a!) state, Tensor r, Tensor k, Tensor v, Tensor w, Tensor u"), s


def test_strategy_validation():
    from chatrwkv_b200.model import RWKV
    with pytest.raises(ValueError):
        RWKV({}, "gpu fp16", verbose=False)
    for s in ("cpu fp32i8", "cuda fp16", "cuda fp16i8 *10 -> cpu fp32", "cuda:0 fp16i8 *4+"):
        with pytest.raises(NotImplementedError):
            RWKV({}, s, verbose=False)


def test_synth_checkpoint_schema():
    from chatrwkv_b200 import synth
    w = synth.make_checkpoint(6, 2, 64, 224, 100, seed=1, head_size=16, maa_rank=8, decay_rank=16)
    assert w["blocks.1.att.time_maa_w2"].shape == (5, 8, 64)
    assert w["blocks.0.att.time_faaaa"].shape == (4, 16)
    assert w["blocks.1.ffn.key.weight"].shape == (224, 64)
    w2 = synth.make_checkpoint(6, 2, 64, 224, 100, seed=1, head_size=16, maa_rank=8, decay_rank=16)
    assert all(torch.equal(w[k], w2[k]) for k in w)
    assert synth.make_tokens(5, 100, 3) == synth.make_tokens(5, 100, 3)
