"""Parity at the shapes the benchmark measures: the operator sweep's (N, M) pairs, the 7B / 14B
matrices and the head.  Same oracle and tolerances as tests/test_gpu_ops.py; packing stays
bit-exact."""
import pytest
import torch

from oracle import rwkv_oracle as orc

pytestmark = pytest.mark.gpu

SWEEP = [(4096, 4096), (4096, 16384), (16384, 4096), (5120, 20480)]


def _bits(t):
    return t.contiguous().view(torch.int16 if t.dtype == torch.float16 else torch.int32)


@pytest.fixture(scope="module")
def packed():
    """Each shape packed once by the oracle on the CPU (seconds per shape), shared by the tests below."""
    from tests.util import packed_case
    cache = {}

    def get(N, M):
        if (N, M) not in cache:
            cache[(N, M)] = packed_case(N, M, seed=N + 7 * M)
        return cache[(N, M)]
    return get


@pytest.mark.parametrize("N,M", [(4096, 16384), (16384, 4096), (5120, 20480)])
def test_quantize_weight_bit_exact_at_model_shapes(N, M):
    """Both branch orders of the packer (N > M subtracts the row minimum first, model.py:822-838)."""
    from chatrwkv_b200 import ops
    g = torch.Generator().manual_seed(N * 131 + M)
    src = torch.randn(M, N, generator=g) * 0.02               # nn.Linear layout [out, in]
    ref = orc.quantize_weight(src.t(), torch.float16)
    got = ops.quantize_weight(src.cuda().t(), torch.float16)
    assert torch.equal(got[0].cpu(), ref[0])
    for a, b, name in zip(got[1:], ref[1:], ("mx", "rx", "my", "ry")):
        assert torch.equal(_bits(a.cpu()), _bits(b)), name


@pytest.mark.parametrize("variant,tol", [(0, 2.5e-4), (8, 2e-5)])
@pytest.mark.parametrize("N,M", SWEEP[1:] + [(4096, 50277)])
def test_mm8_one_at_sweep_shapes(packed, N, M, variant, tol):
    from chatrwkv_b200 import ops  # noqa: F401
    from chatrwkv_b200._lib import lib
    cpu, dev = packed(N, M)
    g = torch.Generator().manual_seed(3000 + N)
    x = torch.randn(N, generator=g).half()
    ref = orc.mm8_kernel(x, *cpu)
    lib().rwkv_mm8_one_set_variant(variant)
    try:
        y = torch.zeros(M, dtype=torch.float32, device="cuda")
        torch.ops.rwkv.mm8_one(N, M, x.cuda(), *dev, y)
        torch.cuda.synchronize()
    finally:
        lib().rwkv_mm8_one_set_variant(0)
    assert (y.cpu() - ref).abs().max().item() <= tol * max(ref.abs().max().item(), 1.0)


@pytest.mark.parametrize("T", [16, 128, 1024])
@pytest.mark.parametrize("N,M", SWEEP)
def test_mm8_seq_at_sweep_shapes(packed, T, N, M):
    """Checked on a seeded sample of 96 output columns per shape and T (the fp64 oracle product over all
    columns of a 1024-row case would take minutes on the host): the kernel's column tiles are
    independent, the sample spans the first, interior and last tiles."""
    from chatrwkv_b200 import ops  # noqa: F401
    cpu, dev = packed(N, M)
    g = torch.Generator().manual_seed(3000 + T)
    x = torch.randn(T, N, generator=g).half()
    y = torch.empty((T, M), dtype=torch.float16, device="cuda")
    torch.ops.rwkv.mm8_seq(T, N, M, x.cuda(), *dev, y)
    torch.cuda.synchronize()
    cols = torch.cat([torch.arange(0, 32), torch.randint(32, M - 32, (32,), generator=g), torch.arange(M - 32, M)])
    q, mx, rx, my, ry = cpu
    ref = orc.mm8_kernel(x, q[:, cols], mx[cols], rx[cols], my, ry)
    got = y[:, cols.cuda()].float().cpu()
    # one fp16 rounding of an fp32-accumulated sum over up to 20480 terms: one fp16 ulp
    assert ((got - ref).abs() <= ref.abs() * 2 ** -9 + 2e-4).all(), (got - ref).abs().max().item()
    assert (got.half() != ref.half()).float().mean().item() < (0.08 if N < 16384 else 0.2)   # fp32 sums of 16384+ terms
    assert torch.isfinite(y).all()


def test_bounded_peer_wait_runs_out_and_reports():
    """rwkv_peer_wait on an arrival word that nothing writes: the wait gives up after its poll limit,
    the kernel returns, the error word reads 1 and the context stays usable.  Nothing faults."""
    from chatrwkv_b200 import _lib
    L = _lib.lib()
    arrived = torch.zeros(8, dtype=torch.int32, device="cuda")
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert L.rwkv_peer_wait(arrived.data_ptr(), 2, 1, None, error.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert error.item() == 1
    # a word that has arrived passes without touching the error word
    error.zero_()
    arrived.fill_(5)
    assert L.rwkv_peer_wait(arrived.data_ptr(), 2, 5, None, error.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert error.item() == 0
    assert torch.ones(4, device="cuda").sum().item() == 4.0
