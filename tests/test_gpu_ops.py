"""GPU parity: every CUDA entry point against the CPU oracle on the same seeded inputs."""
import numpy as np
import pytest
import torch

from oracle import rwkv_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from chatrwkv_b200 import ops as o
    return o


def _bits(t):
    return t.contiguous().view(torch.int16 if t.dtype == torch.float16 else torch.int32)


# ------------------------------------------------------------------------------------ packing
@pytest.mark.parametrize("N,M", [(64, 300), (300, 64), (64, 64), (768, 768), (768, 3072), (3072, 768),
                                 (1000, 50277), (33, 17)])
@pytest.mark.parametrize("layout", ["transposed_view", "contiguous"])
def test_quantize_weight_bit_exact(ops, N, M, layout):
    g = torch.Generator().manual_seed(N * 131 + M)
    src = torch.randn(M, N, generator=g) * 0.02          # nn.Linear layout [out, in]
    logical = src.t()                                     # [N, M] view, as the loader sees it
    dev_in = src.cuda().t() if layout == "transposed_view" else logical.contiguous().cuda()
    for atype in (torch.float16, torch.float32):
        ref = orc.quantize_weight(logical, atype)
        got = ops.quantize_weight(dev_in, atype)
        assert got[0].shape == (N, M) and got[0].stride(0) % 16 == 0
        assert torch.equal(got[0].cpu(), ref[0])
        for a, b, name in zip(got[1:], ref[1:], ("mx", "rx", "my", "ry")):
            assert a.shape == b.shape, name
            assert torch.equal(_bits(a.cpu()), _bits(b)), name


@pytest.mark.parametrize("src_dtype", [torch.float16, torch.bfloat16])
def test_quantize_weight_low_precision_source_and_rescale(ops, src_dtype):
    g = torch.Generator().manual_seed(5)
    src = (torch.randn(256, 96, generator=g) * 0.02).to(src_dtype)
    for k in (0, 1, 3):
        ref = orc.quantize_weight((src / (2 ** k)).t().float(), torch.float16)
        got = ops.quantize_weight(src.cuda().t(), torch.float16, scale=1.0 / (2 ** k))
        assert torch.equal(got[0].cpu(), ref[0])
        for a, b in zip(got[1:], ref[1:]):
            assert torch.equal(_bits(a.cpu()), _bits(b))


def test_quantize_rescale_keeps_codes(ops):
    """Dividing by 2^n before packing leaves codes and ry unchanged and halves mx, my, rx."""
    g = torch.Generator().manual_seed(6)
    src = torch.randn(128, 512, generator=g) * 0.02
    a = ops.quantize_weight(src.cuda().t(), torch.float16, 1.0)
    b = ops.quantize_weight(src.cuda().t(), torch.float16, 0.5)
    assert torch.equal(a[0], b[0]) and torch.equal(a[4], b[4])
    assert torch.equal(a[1].float() * 0.5, b[1].float())


# ------------------------------------------------------------------------------------ mm8_one
MM8_SHAPES = [(4096, 4096), (768, 3072), (3072, 768), (64, 300), (768, 50277), (1000, 48), (40, 1000), (5120, 5120)]


@pytest.mark.parametrize("N,M", MM8_SHAPES)
def test_mm8_one_matches_oracle(ops, N, M):
    from tests.util import packed_case
    cpu, dev = packed_case(N, M, seed=N + 7 * M)
    g = torch.Generator().manual_seed(3000 + N)
    x = torch.randn(N, generator=g).half()
    ref = orc.mm8_kernel(x, *cpu)
    y = torch.zeros(M, dtype=torch.float32, device="cuda")
    torch.ops.rwkv.mm8_one(N, M, x.cuda(), *dev, y)
    err = (y.cpu() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 2e-5 * max(scale, 1.0), (err, scale)
    # deterministic: same bits on a second call; accumulates into y
    y2 = torch.zeros(M, dtype=torch.float32, device="cuda")
    torch.ops.rwkv.mm8_one(N, M, x.cuda(), *dev, y2)
    assert torch.equal(y, y2)
    y3 = torch.full((M,), 3.0, dtype=torch.float32, device="cuda")
    torch.ops.rwkv.mm8_one(N, M, x.cuda(), *dev, y3)
    assert torch.allclose(y3, y + 3.0, rtol=0, atol=1e-5)
    # the rounding the wrapper applies (fp32 -> fp16) agrees with the oracle but for ties
    mism = (y.half().cpu() != ref.half()).float().mean().item()
    assert mism < 0.05, mism


@pytest.mark.parametrize("cluster,width", [(-1, 0), (1, 0), (2, 48), (4, 0), (8, 0), (8, 112), (8, 4096), (0, 16)])
@pytest.mark.parametrize("N,M", [(4096, 4096), (768, 50277), (1000, 48), (16384, 1024), (3072, 768)])
def test_mm8_one_split_reductions_agree(ops, N, M, cluster, width):
    """The cluster kernel (every cluster size, odd panel widths) and the ticket kernel give the
    oracle's result; a forced configuration is bit-reproducible."""
    from chatrwkv_b200._lib import lib
    from tests.util import packed_case
    cpu, dev = packed_case(N, M, seed=N + 7 * M)
    g = torch.Generator().manual_seed(3000 + N)
    x = torch.randn(N, generator=g).half()
    ref = orc.mm8_kernel(x, *cpu)
    lib().rwkv_mm8_one_set_cluster(cluster, width)
    try:
        y = torch.zeros(M, dtype=torch.float32, device="cuda")
        torch.ops.rwkv.mm8_one(N, M, x.cuda(), *dev, y)
        y2 = torch.zeros(M, dtype=torch.float32, device="cuda")
        torch.ops.rwkv.mm8_one(N, M, x.cuda(), *dev, y2)
        torch.cuda.synchronize()
    finally:
        lib().rwkv_mm8_one_set_cluster(0, 0)
    assert (y.cpu() - ref).abs().max().item() <= 2e-5 * max(ref.abs().max().item(), 1.0)
    assert torch.equal(y, y2)


def test_mm8_one_one_signed_input(ops):
    """x >= 0 (the FFN value matmul sees relu(k)^2): centred codes keep the error small."""
    from tests.util import packed_case
    N, M = 3072, 768
    cpu, dev = packed_case(N, M, seed=99)
    g = torch.Generator().manual_seed(1)
    x = (torch.randn(N, generator=g).clamp(min=0) ** 2).half()
    ref = orc.mm8_kernel(x, *cpu)
    y = torch.zeros(M, dtype=torch.float32, device="cuda")
    torch.ops.rwkv.mm8_one(N, M, x.cuda(), *dev, y)
    assert (y.cpu() - ref).abs().max().item() <= 3e-5 * ref.abs().max().item()


def test_mm8_one_unpadded_and_fp32(ops):
    """Contiguous odd-M matrix (byte-load kernel) and the fp32 instantiation."""
    N, M = 96, 301
    g = torch.Generator().manual_seed(4)
    w = torch.randn(N, M, generator=g) * 0.02
    q, mx, rx, my, ry = orc.quantize_weight(w, torch.float32)
    x = torch.randn(N, generator=g)
    ref = orc.mm8_kernel(x, q, mx, rx, my, ry)
    y = torch.zeros(M, dtype=torch.float32, device="cuda")
    torch.ops.rwkv.mm8_one(N, M, x.cuda(), q.cuda(), mx.cuda(), rx.cuda(), my.cuda(), ry.cuda(), y)
    assert (y.cpu() - ref).abs().max().item() <= 2e-5 * max(1.0, ref.abs().max().item())


def test_mm8_rejects_bad_arguments(ops):
    from chatrwkv_b200._lib import RwkvB200Error
    from tests.util import packed_case
    cpu, dev = packed_case(64, 64, seed=1)
    x = torch.randn(64).half().cuda()
    y = torch.zeros(64, dtype=torch.float32, device="cuda")
    with pytest.raises(RwkvB200Error):
        torch.ops.rwkv.mm8_one(64, 64, x.double(), *dev, y)           # unsupported dtype
    with pytest.raises(RwkvB200Error):
        torch.ops.rwkv.mm8_one(64, 64, x, dev[0].t(), *dev[1:], y)    # inner stride != 1


# ------------------------------------------------------------------------------------ mm8_seq
@pytest.mark.parametrize("T", [2, 3, 17, 64, 130])
@pytest.mark.parametrize("N,M", [(768, 768), (768, 3072), (100, 301), (4096, 1024)])
def test_mm8_seq_matches_oracle(ops, T, N, M):
    from tests.util import packed_case
    cpu, dev = packed_case(N, M, seed=N + M + T)
    g = torch.Generator().manual_seed(3000 + T)
    x = torch.randn(T, N, generator=g).half()
    ref = orc.mm8_kernel(x, *cpu)
    y = torch.empty((T, M), dtype=torch.float16, device="cuda")
    torch.ops.rwkv.mm8_seq(T, N, M, x.cuda(), *dev, y)
    # one fp16 rounding of an fp32-accurate sum: within one fp16 ulp of the oracle
    err = (y.float().cpu() - ref).abs()
    tol = ref.abs() * 2 ** -10 + 1e-4
    assert (err <= tol).all(), err.max().item()
    mism = (y.cpu() != ref.half()).float().mean().item()
    assert mism < 0.05, mism


def test_mm8_seq_strided_rows(ops):
    from tests.util import packed_case
    T, N, M = 9, 256, 512
    cpu, dev = packed_case(N, M, seed=77)
    x = torch.randn(T, N + 24).half()
    xs = x.cuda()[:, :N]
    ybig = torch.zeros((T, M + 16), dtype=torch.float16, device="cuda")
    yv = ybig[:, :M]
    torch.ops.rwkv.mm8_seq(T, N, M, xs, *dev, yv)
    ref = orc.mm8_kernel(x[:, :N], *cpu)
    assert ((yv.float().cpu() - ref).abs() <= ref.abs() * 2 ** -10 + 1e-4).all()
    assert (ybig[:, M:] == 0).all()


# ------------------------------------------------------------------------------------ WKV
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("T", [1, 7, 64])
def test_wkv4_forward(ops, dtype, T):
    C = 192
    g = torch.Generator().manual_seed(T)
    w = -torch.exp(torch.empty(C).uniform_(-5, 1, generator=g))
    u = torch.empty(C).uniform_(-1, 1, generator=g)
    aa, bb, pp = torch.zeros(C), torch.zeros(C), torch.zeros(C) - 1e30
    daa, dbb, dpp = aa.cuda(), bb.cuda(), pp.cuda()
    for _ in range(2):      # second pass: carried state
        k = torch.randn(T, C, generator=g).to(dtype)
        v = torch.randn(T, C, generator=g).to(dtype)
        ref = orc.wkv4_forward(T, C, w, u, k, v, aa, bb, pp)
        y = torch.empty((T, C), dtype=dtype, device="cuda")
        torch.ops.rwkv.wkv_forward(1, T, C, w.cuda(), u.cuda(), k.cuda(), v.cuda(), y, daa, dbb, dpp)
        tol = 2e-3 if dtype == torch.float16 else 2e-5
        torch.testing.assert_close(y.cpu().float(), ref.float(), rtol=tol, atol=tol)
        torch.testing.assert_close(daa.cpu(), aa, rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(dbb.cpu(), bb, rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(dpp.cpu(), pp, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("which", [5, 6])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("N,H,T", [(64, 3, 37), (16, 4, 5), (32, 2, 16), (128, 1, 3)])
def test_wkv56_forward(ops, which, dtype, N, H, T):
    C = N * H
    g = torch.Generator().manual_seed(N + T)
    r = torch.randn(T, C, generator=g).to(dtype)
    k = (torch.randn(T, C, generator=g) * 0.5).to(dtype)
    v = torch.randn(T, C, generator=g).to(dtype)
    u = torch.empty(C).uniform_(-1, 1, generator=g).to(dtype)
    state = torch.randn(H, N, N, generator=g) * 0.1
    if which == 6:
        w = torch.exp(-torch.exp(torch.empty(T, C).uniform_(-5, 1, generator=g)))
        fn, ofn = getattr(torch.ops.rwkv6, "forward_" + {torch.float32: "fp32", torch.float16: "fp16", torch.bfloat16: "bf16"}[dtype]), orc.wkv6_forward
    else:
        w = torch.exp(-torch.exp(torch.empty(C).uniform_(-5, 1, generator=g)))
        fn, ofn = getattr(torch.ops.rwkv5, "forward_" + {torch.float32: "fp32", torch.float16: "fp16", torch.bfloat16: "bf16"}[dtype]), orc.wkv5_forward
    ds = state.clone().cuda()
    y = torch.empty((T, C), dtype=dtype, device="cuda")
    fn(1, T, C, H, ds, r.cuda(), k.cuda(), v.cuda(), w.cuda(), u.cuda(), y)
    ref = ofn(1, T, C, H, state, r, k, v, w, u)
    tol = {torch.float32: 1e-4, torch.float16: 4e-3, torch.bfloat16: 3e-2}[dtype]
    torch.testing.assert_close(y.cpu().float(), ref.float(), rtol=tol, atol=tol)
    torch.testing.assert_close(ds.cpu(), state, rtol=1e-4, atol=1e-4)


def test_op_schemas(ops):
    s = str(torch.ops.rwkv.mm8_one.default._schema)
    assert s.startswith("rwkv::mm8_one(int N, int M, Tensor x, Tensor w, Tensor mx, Tensor rx, Tensor my, Tensor ry")
    assert "rwkv::mm8_seq(int B, int N, int M" in str(torch.ops.rwkv.mm8_seq.default._schema)
    assert "rwkv::wkv_forward(int B, int T, int C" in str(torch.ops.rwkv.wkv_forward.default._schema)
    for ns in (torch.ops.rwkv5, torch.ops.rwkv6):
        for f in ("forward_bf16", "forward_fp16", "forward_fp32"):
            assert hasattr(ns, f)


@pytest.mark.parametrize("T,N,M", [(128, 256, 128), (64, 64, 128), (200, 768, 3072), (1024, 4096, 512), (257, 1000, 264)])
def test_mm8_seq_tensor_core_path(ops, T, N, M):
    """Rows >= 64 with an 8-byte-aligned matrix run on tcgen05; same oracle, same tolerance.
    Includes ragged T (not a multiple of 128), N (not a multiple of 64) and M (not of 128)."""
    import ctypes
    from chatrwkv_b200 import _lib
    from tests.util import packed_case
    cpu, dev = packed_case(N, M, seed=N * 3 + M + T)
    g = torch.Generator().manual_seed(T)
    x = torch.randn(T, N, generator=g).half()
    ref = orc.mm8_kernel(x, *cpu)
    y = torch.empty((T, M), dtype=torch.float16, device="cuda")
    torch.ops.rwkv.mm8_seq(T, N, M, x.cuda(), *dev, y)
    torch.cuda.synchronize()
    ws = ops.workspace(torch.device("cuda", torch.cuda.current_device()), 1024, "mm8_seq")
    e = ctypes.c_int(0)
    assert _lib.lib().rwkv_mm8_seq_tc_take_error(ws.data_ptr(), None, ctypes.byref(e)) == 0 and e.value == 0
    err = (y.float().cpu() - ref).abs()
    tol = ref.abs() * 2 ** -10 + 1e-4
    assert (err <= tol).all(), err.max().item()
    assert (y.cpu() != ref.half()).float().mean().item() < 0.05
    # and against the CUDA-core kernel
    _lib.lib().rwkv_mm8_seq_set_path(1)
    try:
        y2 = torch.empty_like(y)
        torch.ops.rwkv.mm8_seq(T, N, M, x.cuda(), *dev, y2)
    finally:
        _lib.lib().rwkv_mm8_seq_set_path(0)
    assert ((y.float() - y2.float()).abs() <= y2.float().abs() * 2 ** -9 + 2e-4).all()
