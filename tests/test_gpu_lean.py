"""The decode kernel cut down to its critical path (csrc/mm8_lean.cuh) against the general cluster kernel
(csrc/mm8_cluster.cuh) on the same launches.  The integer dot products are exact in both; what differs is the
order of a few fp32 additions (rows are dealt to threads differently, panels may have another width) and the
one-pass LayerNorm statistics: ulps of fp32 before the fp16 rounding.  The oracle comparisons of
test_gpu_model*.py and test_gpu_model_widths.py run on this kernel by default."""
import copy

import pytest
import torch

from chatrwkv_b200 import synth
from oracle import rwkv_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture()
def lean_switch():
    from chatrwkv_b200 import _lib
    lib = _lib.lib()
    yield lib.rwkv_mm8_one_set_lean
    lib.rwkv_mm8_one_set_lean(-1)


def _take_error():
    import ctypes as C
    from chatrwkv_b200 import _lib
    e = C.c_int(-1)
    _lib.check(_lib.lib().rwkv_mm8_one_take_error(torch.cuda.current_stream().cuda_stream, C.byref(e)), "take_error")
    return e.value


@pytest.mark.parametrize("N,M", [(4096, 4096), (4096, 16384), (16384, 4096), (20480, 5120), (4096, 50277), (1024, 1000)])
def test_mm8_one_operator_agrees_between_the_kernels(lean_switch, N, M):
    from chatrwkv_b200 import ops  # noqa: F401  (registers torch.ops.rwkv)
    from tests.util import packed_case
    cpu, dev = packed_case(N, M, seed=N + 3 * M)
    g = torch.Generator().manual_seed(M)
    x = torch.randn(N, generator=g).half()
    ys = []
    for on in (1, 0):
        lean_switch(on)
        y = torch.zeros(M, dtype=torch.float32, device="cuda")
        torch.ops.rwkv.mm8_one(N, M, x.cuda(), *dev, y)
        ys.append(y)
    ref = orc.mm8_kernel(x, *cpu)
    assert (ys[0] - ys[1]).abs().max().item() <= 2e-6 * max(1.0, ref.abs().max().item())
    lean_switch(1)
    y2 = torch.zeros(M, dtype=torch.float32, device="cuda")
    torch.ops.rwkv.mm8_one(N, M, x.cuda(), *dev, y2)
    assert torch.equal(ys[0], y2)                 # the same kernel twice: bit-identical
    assert (ys[0].cpu() - ref).abs().max().item() <= 2.5e-4 * max(1.0, ref.abs().max().item())
    # accumulate semantics of the operator (the reference adds into y, pkg/cuda/operators.cu:229-231)
    lean_switch(1)
    torch.ops.rwkv.mm8_one(N, M, x.cuda(), *dev, ys[0])
    assert (ys[0].cpu() - 2 * ref).abs().max().item() <= 5e-4 * max(1.0, ref.abs().max().item())
    assert _take_error() == 0


@pytest.mark.parametrize("case", [dict(version=4, n_layer=2, n_embd=4096, n_ffn=16384, vocab=2048, seed=41),
                                  dict(version=4, n_layer=2, n_embd=5120, n_ffn=20480, vocab=2048, seed=42),
                                  dict(version=6, n_layer=2, n_embd=4096, n_ffn=14336, vocab=2048, seed=43),
                                  dict(version=4, n_layer=3, n_embd=768, n_ffn=3072, vocab=1000, seed=44)])
def test_decode_steps_agree_between_the_kernels(lean_switch, case):
    from chatrwkv_b200.model import RWKV
    ck = synth.make_checkpoint(**case, device="cuda")
    model = RWKV(ck, "cuda fp16i8", verbose=False)
    tokens = synth.make_tokens(14, case["vocab"], 9)
    _, st0 = model.forward(tokens[:8], None)
    st0 = copy.deepcopy(st0)
    runs = []
    for on in (1, 0):
        lean_switch(on)
        model.set_decode_path("launch")          # drops the captured graphs: the kernel choice is part of a capture
        st, outs = copy.deepcopy(st0), []
        for t in tokens[8:]:
            lg, st = model.forward([t], st)
            outs.append(lg.clone())
        runs.append((outs, copy.deepcopy(st)))
    # an fp32 sum taken in another order flips an fp16 rounding here and there, and the flips travel through the
    # layers (two runs of the reference differ the same way): a few fp16 ulps of the logits
    for a, b in zip(runs[0][0], runs[1][0]):
        assert (a - b).abs().max().item() < 1.6e-2
        assert (a - b).abs().mean().item() < 4e-3
    for a, b in zip(runs[0][1], runs[1][1]):
        scale = max(1.0, b.float().abs().max().item()) if b.float().abs().max().item() < 1e20 else 1e30
        assert (a.float() - b.float()).abs().max().item() <= 4e-3 * scale
    assert _take_error() == 0
