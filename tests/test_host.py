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
    for s in ("cpu fp32i8", "cuda fp32", "cuda bf16", "cuda fp16i8 *10 -> cpu fp32", "cuda:0 fp16i8 *4+",
              "cuda:0 fp16i8 *4 -> cuda:1 fp16"):
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


def test_peer_region_launch_numbering_without_gpu():
    """The exchange descriptors of a token: launch j publishes j and waits for j - 1 (0 = no wait), every
    rank addresses the others' arrival word for itself, and the numbering restarts with each token (the
    device-side base is advanced instead)."""
    from chatrwkv_b200 import shard
    import torch
    pr = shard.PeerRegion.__new__(shard.PeerRegion)
    pr.world, pr.rank = 4, 2
    pr.others = [0, 1, 3]
    pr.bases = [0x10000000 * (r + 1) for r in range(4)]
    pr.base = pr.bases[2]
    pr.offsets = {"x": (0, torch.float16, 64), "fk": (256, torch.float16, 256)}
    pr.flag_off = 1024
    pr._rel, pr._n = 0, 3
    e1 = pr.exchange([("x", 16)], wait=False)
    e2 = pr.exchange([("fk", 128), ("x", 16)], wait=True)
    e3 = pr.exchange([("x", 16)], wait=True)
    assert (e1.wait_seq, e1.signal_seq) == (0, 1) and (e2.wait_seq, e2.signal_seq) == (1, 2) and (e3.wait_seq, e3.signal_seq) == (2, 3)
    assert e2.world == 4 and e2.rank == 2
    # problem 0 of launch 2 is fk at element 128 on ranks 0, 1, 3; problem 1 is x at element 16
    assert [e2.peer_y[0][i] for i in range(3)] == [pr.bases[r] + 256 + 2 * 128 for r in (0, 1, 3)]
    assert [e2.peer_y[1][i] for i in range(3)] == [pr.bases[r] + 0 + 2 * 16 for r in (0, 1, 3)]
    # this rank's words, and on every other rank the word that belongs to this rank (index 2)
    assert e2.arrived == pr.bases[2] + 1024
    assert [e2.peer_arrived[i] for i in range(3)] == [pr.bases[r] + 1024 + 4 * 2 for r in (0, 1, 3)]
    assert e2.seq_base == pr.bases[2] + 1024 + 4 * (shard.PeerRegion.FLAG_WORDS - 3)
