"""mm8_one with more than 16384 in-features (the 14B shape's ffn.value: 20480): the cluster kernel's
build with 2560 rows per CTA (taken per launch; rwkv_mm8_one_batch_flags can ask for it on other launches too)."""
import pytest
import torch

from oracle import rwkv_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("N,M", [(20480, 1024), (20480, 5120)])
def test_mm8_one_20480_in_features(N, M):
    from chatrwkv_b200 import ops  # noqa: F401  (registers torch.ops.rwkv)
    from tests.util import packed_case
    cpu, dev = packed_case(N, M, seed=N + M)
    g = torch.Generator().manual_seed(N)
    x = (torch.randn(N, generator=g).clamp(min=0) ** 2).half()       # what ffn.value sees: relu(k)^2
    ref = orc.mm8_kernel(x, *cpu)
    y = torch.zeros(M, dtype=torch.float32, device="cuda")
    torch.ops.rwkv.mm8_one(N, M, x.cuda(), *dev, y)
    y2 = torch.zeros(M, dtype=torch.float32, device="cuda")
    torch.ops.rwkv.mm8_one(N, M, x.cuda(), *dev, y2)
    assert (y.cpu() - ref).abs().max().item() <= 2.5e-4 * ref.abs().max().item()
    assert torch.equal(y, y2)
    # a matrix of ordinary size afterwards runs on the ordinary build again
    cpu2, dev2 = packed_case(4096, 4096, seed=5)
    x2 = torch.randn(4096, generator=g).half()
    ref2 = orc.mm8_kernel(x2, *cpu2)
    y3 = torch.zeros(4096, dtype=torch.float32, device="cuda")
    torch.ops.rwkv.mm8_one(4096, 4096, x2.cuda(), *dev2, y3)
    assert (y3.cpu() - ref2).abs().max().item() <= 2.5e-4 * max(1.0, ref2.abs().max().item())
