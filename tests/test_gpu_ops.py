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


# The default kernel feeds the activations to the integer dot-product instructions as 16-bit fixed
# point (exact integer sums, one scale per CTA): per output an error of at most
# 2^-16 max|x*ry| sum|w-128|, in practice ~4e-5 of the output's RMS -- a tenth of the fp16 rounding
# that follows.  `rwkv_mm8_one_set_variant(8)` selects the fp32 form, which is held to fp32 round-off.
MM8_ARITH = [(0, 2.5e-4, 0.15), (8, 2e-5, 0.05)]


@pytest.mark.parametrize("variant,tol,max_mismatch", MM8_ARITH)
@pytest.mark.parametrize("N,M", MM8_SHAPES)
def test_mm8_one_matches_oracle(ops, N, M, variant, tol, max_mismatch):
    from chatrwkv_b200._lib import lib
    from tests.util import packed_case
    cpu, dev = packed_case(N, M, seed=N + 7 * M)
    g = torch.Generator().manual_seed(3000 + N)
    x = torch.randn(N, generator=g).half()
    ref = orc.mm8_kernel(x, *cpu)
    lib().rwkv_mm8_one_set_variant(variant)
    try:
        y = torch.zeros(M, dtype=torch.float32, device="cuda")
        torch.ops.rwkv.mm8_one(N, M, x.cuda(), *dev, y)
        # deterministic: same bits on a second call; accumulates into y
        y2 = torch.zeros(M, dtype=torch.float32, device="cuda")
        torch.ops.rwkv.mm8_one(N, M, x.cuda(), *dev, y2)
        y3 = torch.full((M,), 3.0, dtype=torch.float32, device="cuda")
        torch.ops.rwkv.mm8_one(N, M, x.cuda(), *dev, y3)
        torch.cuda.synchronize()
    finally:
        lib().rwkv_mm8_one_set_variant(0)
    err = (y.cpu() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= tol * max(scale, 1.0), (err, scale)
    assert torch.equal(y, y2)
    assert torch.allclose(y3, y + 3.0, rtol=0, atol=1e-5)
    # the rounding the wrapper applies (fp32 -> fp16) agrees with the oracle but for near-ties
    mism = (y.half().cpu() != ref.half()).float().mean().item()
    assert mism < max_mismatch, mism


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
    assert (y.cpu() - ref).abs().max().item() <= (2e-5 if cluster == -1 else 2.5e-4) * max(ref.abs().max().item(), 1.0)
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
    assert (y.cpu() - ref).abs().max().item() <= 2.5e-4 * ref.abs().max().item()


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


def test_gemm_fp16_cublas_op(ops):
    """The reference's fp16 GEMM operator name (gemm_fp16_cublas.cpp:28-75): 2-D and batched, fp16 and fp32 out."""
    g = torch.Generator().manual_seed(2)
    a = torch.randn(5, 64, generator=g).half().cuda()
    b = torch.randn(64, 48, generator=g).half().cuda()
    for dt in (torch.float16, torch.float32):
        c = torch.empty((5, 48), dtype=dt, device="cuda")
        torch.ops.rwkv.gemm_fp16_cublas(a, b, c)
        ref = a.float() @ b.float()
        # fp16 products accumulated in fp32; |c| reaches ~30 here, so one fp16 rounding of the result is up to 0.016
        assert (c.float() - ref).abs().max().item() <= (4e-2 if dt == torch.float16 else 2e-2)
    a3 = torch.randn(3, 5, 64, generator=g).half().cuda()
    b3 = torch.randn(3, 64, 16, generator=g).half().cuda()
    c3 = torch.empty((3, 5, 16), dtype=torch.float16, device="cuda")
    torch.ops.rwkv.gemm_fp16_cublas(a3, b3, c3)
    assert (c3.float() - torch.bmm(a3.float(), b3.float())).abs().max().item() <= 4e-2


def test_op_schemas(ops):
    s = str(torch.ops.rwkv.mm8_one.default._schema)
    assert s.startswith("rwkv::mm8_one(int N, int M, Tensor x, Tensor w, Tensor mx, Tensor rx, Tensor my, Tensor ry")
    assert "rwkv::mm8_seq(int B, int N, int M" in str(torch.ops.rwkv.mm8_seq.default._schema)
    assert "rwkv::wkv_forward(int B, int T, int C" in str(torch.ops.rwkv.wkv_forward.default._schema)
    for ns in (torch.ops.rwkv5, torch.ops.rwkv6):
        for f in ("forward_bf16", "forward_fp16", "forward_fp32"):
            assert hasattr(ns, f)


@pytest.mark.parametrize("T,N,M", [(128, 256, 128), (64, 64, 128), (200, 768, 3072), (1024, 4096, 512), (257, 1000, 264),
                                   (130, 100, 304), (13, 4104, 512)])
def test_mm8_seq_tensor_core_path(ops, T, N, M):
    """Rows >= 8 with an 8-byte-aligned matrix run on tcgen05; same oracle, same tolerance.
    Includes ragged T (not a multiple of 128 or 8), N (not a multiple of 64 or 8) and M (not of 128)."""
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


@pytest.mark.parametrize("T,N,M", [(256, 320, 9728), (200, 200, 19464), (512, 128, 5000 * 8), (1024, 4096, 4096)])
def test_mm8_seq_cta_pair_form(ops, T, N, M):
    """Launches with an even number of 128-row tiles and no K split (more output tiles than half of the SMs) run as
    clusters of two CTAs that share one 256-row UMMA (tcgen05 cta_group::2), each converting half of the B tile.
    Same sums in the same order: bit-identical to the one-CTA form (set_path bit 3), and both match the oracle.
    Includes a ragged last row tile and ragged N and M."""
    import ctypes
    from chatrwkv_b200 import _lib
    from tests.util import packed_case
    cpu, dev = packed_case(N, M, seed=N + M + T)
    g = torch.Generator().manual_seed(T + 1)
    x = torch.randn(T, N, generator=g).half()
    xd = x.cuda()
    y = torch.empty((T, M), dtype=torch.float16, device="cuda")
    torch.ops.rwkv.mm8_seq(T, N, M, xd, *dev, y)
    _lib.lib().rwkv_mm8_seq_set_path(8)
    try:
        y1 = torch.empty_like(y)
        torch.ops.rwkv.mm8_seq(T, N, M, xd, *dev, y1)
    finally:
        _lib.lib().rwkv_mm8_seq_set_path(0)
    torch.cuda.synchronize()
    ws = ops.workspace(torch.device("cuda", torch.cuda.current_device()), 1024, "mm8_seq")
    e = ctypes.c_int(0)
    assert _lib.lib().rwkv_mm8_seq_tc_take_error(ws.data_ptr(), None, ctypes.byref(e)) == 0 and e.value == 0
    assert torch.equal(y, y1)
    if T * N * M <= 256 * 320 * 9728 * 4:           # the oracle's fp64 product in seconds
        ref = orc.mm8_kernel(x, *cpu)
        err = (y.float().cpu() - ref).abs()
        assert (err <= ref.abs() * 2 ** -10 + 1e-4).all(), err.max().item()


def test_mm8_seq_ignores_stale_scratch_rows(ops):
    """The operand images keep whatever the scratch held in the rows past T of the last 128-row tile
    (here: NaN patterns); no stored output may depend on them."""
    from tests.util import packed_case
    T, N, M = 130, 512, 256
    cpu, dev = packed_case(N, M, seed=5)
    g = torch.Generator().manual_seed(9)
    x = torch.randn(T, N, generator=g).half()
    ref = orc.mm8_kernel(x, *cpu)
    y = torch.empty((T, M), dtype=torch.float16, device="cuda")
    torch.ops.rwkv.mm8_seq(T, N, M, x.cuda(), *dev, y)              # sizes the scratch
    torch.cuda.synchronize()
    ws = ops.workspace(torch.device("cuda", torch.cuda.current_device()), 1024, "mm8_seq")
    ws[256:8 << 20].fill_(0xFF)                                       # fp16 / fp32 NaN everywhere but the error word
    y.zero_()
    torch.ops.rwkv.mm8_seq(T, N, M, x.cuda(), *dev, y)
    torch.cuda.synchronize()
    assert torch.isfinite(y).all()
    assert ((y.float().cpu() - ref).abs() <= ref.abs() * 2 ** -10 + 1e-4).all()
    ws[256:8 << 20].zero_()


# ------------------------------------------------------------------- RWKV-5/6 one-token pieces
def _h(t):
    return t.half()


def _lib_unsupported():
    from chatrwkv_b200 import _lib
    return _lib.ERR_UNSUPPORTED


@pytest.mark.parametrize("D,Lm,Ld", [(4096, 32, 64), (512, 8, 16), (64, 4, 8)])
def test_v6_token_shift_and_decay(ops, D, Lm, Ld):
    """rwkv_v6_token_shift / rwkv_v6_decay against the lines of att_one_v6_0 they replace
    (pkg/model.py:1264-1276, 1286-1287), evaluated on the CPU with fp16 tensors."""
    import ctypes as C
    import torch.nn.functional as F
    from chatrwkv_b200._lib import check, lib
    g = torch.Generator().manual_seed(D + Lm)
    rn = lambda *s, sc=1.0: torch.randn(*s, generator=g) * sc
    x, sx = _h(rn(D)), _h(rn(D))
    ln_w, ln_b = _h(1 + rn(D, sc=0.1)), _h(rn(D, sc=0.1))
    maa_x = _h(torch.rand(D, generator=g))
    maa = [_h(torch.rand(D, generator=g)) for _ in range(5)]
    w1, w2 = _h(rn(D, 5 * Lm, sc=0.05)), _h(rn(5, Lm, D, sc=0.05))
    dw1, dw2 = _h(rn(D, Ld, sc=0.05)), _h(rn(Ld, D, sc=0.05))
    decay = torch.rand(D, generator=g) * 6 - 5
    # reference (fp32 accumulation inside the fp16 matmuls, one rounding per op)
    xx = F.layer_norm(x.float(), (D,), ln_w.float(), ln_b.float()).half()
    dd = sx - xx
    xxx = xx + dd * maa_x
    hid = torch.tanh((xxx.float() @ w1.float()).half()).view(5, 1, Lm)
    m = torch.bmm(hid.float(), w2.float()).half().view(5, D)
    ref5 = [xx + dd * (maa[f] + m[f]) for f in range(5)]
    t1 = torch.tanh((ref5[0].float() @ dw1.float()).half())
    ref_w = torch.exp(-torch.exp(decay + (t1.float() @ dw2.float()).half().float()))

    dev = lambda t: t.cuda().contiguous()
    dx, dsx, dlw, dlb, dmx = dev(x), dev(sx), dev(ln_w), dev(ln_b), dev(maa_x)
    dmaa = [dev(t) for t in maa]
    dw = [dev(w1), dev(w2), dev(dw1), dev(dw2)]
    out5 = [torch.zeros(D, dtype=torch.float16, device="cuda") for _ in range(5)]
    xx_o, dd_o, ns = (torch.zeros(D, dtype=torch.float16, device="cuda") for _ in range(3))
    ws = torch.zeros(lib().rwkv_v6_scratch_bytes(D, max(5 * Lm, Ld)), dtype=torch.uint8, device="cuda")
    arr = lambda ts: (C.c_void_p * len(ts))(*[t.data_ptr() for t in ts])
    st = torch.cuda.current_stream().cuda_stream
    check(lib().rwkv_v6_token_shift(D, Lm, dx.data_ptr(), dsx.data_ptr(), ns.data_ptr(), dlw.data_ptr(), dlb.data_ptr(),
                                    dmx.data_ptr(), arr(dmaa), dw[0].data_ptr(), dw[1].data_ptr(), ws.data_ptr(), ws.numel(),
                                    xx_o.data_ptr(), dd_o.data_ptr(), arr(out5), st), "v6_token_shift")
    w_out = torch.zeros(D, dtype=torch.float32, device="cuda")
    check(lib().rwkv_v6_decay(D, Ld, out5[0].data_ptr(), dw[2].data_ptr(), dw[3].data_ptr(), dev(decay).data_ptr(),
                              ws.data_ptr(), ws.numel(), w_out.data_ptr(), st), "v6_decay")
    torch.cuda.synchronize()
    assert (xx_o.cpu().float() - xx.float()).abs().max() <= 4e-3          # one fp16 ulp at |x| < 4
    assert torch.equal(ns, xx_o)
    assert (dd_o.cpu().float() - dd.float()).abs().max() <= 8e-3
    for f in range(5):
        assert (out5[f].cpu().float() - ref5[f].float()).abs().max() <= 2e-2, f
    assert (w_out.cpu() - ref_w).abs().max() <= 5e-3
    # the single-launch form computes the same values (or declines shapes it does not take)
    out5b = [torch.zeros(D, dtype=torch.float16, device="cuda") for _ in range(5)]
    xx_b, dd_b, ns_b = (torch.zeros(D, dtype=torch.float16, device="cuda") for _ in range(3))
    w_b = torch.zeros(D, dtype=torch.float32, device="cuda")
    rc = lib().rwkv_v6_att_pre(D, Lm, Ld, dx.data_ptr(), dsx.data_ptr(), ns_b.data_ptr(), dlw.data_ptr(), dlb.data_ptr(),
                               dmx.data_ptr(), arr(dmaa), dw[0].data_ptr(), dw[1].data_ptr(), dw[2].data_ptr(),
                               dw[3].data_ptr(), dev(decay).data_ptr(), xx_b.data_ptr(), dd_b.data_ptr(), arr(out5b),
                               w_b.data_ptr(), st)
    torch.cuda.synchronize()
    if (5 * Lm) % 8 == 0 and Ld % 8 == 0:
        assert rc == 0
        # (LayerNorm statistics are summed by 512 instead of 256 threads: fp32 round-off, at most an fp16 ulp)
        assert (xx_b.float() - xx_o.float()).abs().max() <= 4e-3 and (dd_b.float() - dd_o.float()).abs().max() <= 8e-3
        assert torch.equal(ns_b, xx_b)
        for f in range(5):
            assert (out5b[f].cpu().float() - ref5[f].float()).abs().max() <= 2e-2, f
            assert (out5b[f].float() - out5[f].float()).abs().max() <= 8e-3, f
        assert (w_b.cpu() - ref_w).abs().max() <= 5e-3
        # the token shift alone (no decay arguments): the same five vectors bit for bit, nothing written elsewhere
        out5c = [torch.zeros(D, dtype=torch.float16, device="cuda") for _ in range(5)]
        xx_c, dd_c, ns_c = (torch.zeros(D, dtype=torch.float16, device="cuda") for _ in range(3))
        rc = lib().rwkv_v6_att_pre(D, Lm, Ld, dx.data_ptr(), dsx.data_ptr(), ns_c.data_ptr(), dlw.data_ptr(), dlb.data_ptr(),
                                   dmx.data_ptr(), arr(dmaa), dw[0].data_ptr(), dw[1].data_ptr(), None, None, None,
                                   xx_c.data_ptr(), dd_c.data_ptr(), arr(out5c), None, st)
        torch.cuda.synchronize()
        assert rc == 0
        assert torch.equal(xx_c, xx_b) and torch.equal(dd_c, dd_b) and torch.equal(ns_c, ns_b)
        for f in range(5):
            assert torch.equal(out5c[f], out5b[f]), f
        # decay arguments given in part: refused before any launch
        assert lib().rwkv_v6_att_pre(D, Lm, Ld, dx.data_ptr(), dsx.data_ptr(), ns_c.data_ptr(), dlw.data_ptr(), dlb.data_ptr(),
                                     dmx.data_ptr(), arr(dmaa), dw[0].data_ptr(), dw[1].data_ptr(), dw[2].data_ptr(), None, None,
                                     xx_c.data_ptr(), dd_c.data_ptr(), arr(out5c), None, st) == -1
    else:
        assert rc == _lib_unsupported()


@pytest.mark.parametrize("H,N", [(64, 64), (4, 16), (3, 32), (2, 128)])
def test_wkv56_one(ops, H, N):
    """rwkv_wkv56_one against att_one_v6_0's state update, group-norm and gate (pkg/model.py:1289-1296)."""
    import torch.nn.functional as F
    from chatrwkv_b200._lib import check, lib
    g = torch.Generator().manual_seed(H * 1000 + N)
    C_ = H * N
    r, k, v, gate = (_h(torch.randn(C_, generator=g)) for _ in range(4))
    w = torch.exp(-torch.exp(torch.rand(C_, generator=g) * 6 - 5))
    u = torch.rand(C_, generator=g) * 2 - 1
    S = torch.randn(H, N, N, generator=g)
    lw, lb = 1 + torch.randn(C_, generator=g) * 0.1, torch.randn(C_, generator=g) * 0.1
    rr, kk, vv = r.float().view(H, 1, N), k.float().view(H, N, 1), v.float().view(H, 1, N)
    a = kk @ vv
    out = rr @ (u.view(H, N, 1) * a + S)
    S_new = a + w.view(H, N, 1) * S
    out = F.group_norm(out.flatten().unsqueeze(0), num_groups=H, weight=lw, bias=lb, eps=64e-5).squeeze(0)
    ref = out.half() * gate
    d = lambda t: t.cuda().contiguous()
    dS, dS2 = d(S), torch.zeros(H, N, N, device="cuda")
    y = torch.zeros(C_, dtype=torch.float16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    args = [d(r), d(k), d(v), d(w), d(u)]
    dl = [d(lw), d(lb), d(gate)]
    check(lib().rwkv_wkv56_one(H, N, *[t.data_ptr() for t in args], dS.data_ptr(), dS2.data_ptr(), dl[0].data_ptr(),
                               dl[1].data_ptr(), dl[2].data_ptr(), y.data_ptr(), st), "wkv56_one")
    torch.cuda.synchronize()
    torch.testing.assert_close(dS2.cpu(), S_new, rtol=1e-5, atol=1e-5)
    assert (y.cpu().float() - ref.float()).abs().max() <= 2e-2
    # in place (new_state aliases state)
    check(lib().rwkv_wkv56_one(H, N, *[t.data_ptr() for t in args], dS.data_ptr(), dS.data_ptr(), dl[0].data_ptr(),
                               dl[1].data_ptr(), dl[2].data_ptr(), y.data_ptr(), st), "wkv56_one")
    torch.cuda.synchronize()
    assert torch.equal(dS, dS2)


@pytest.mark.parametrize("bad", [float("nan"), float("inf")])
def test_mm8_one_non_finite_activation_gives_nan(ops, bad):
    """A NaN or infinity among the activations must not be lost by the fixed-point arithmetic:
    every output of the rows' K-slice becomes NaN, as it would in fp32 (inf * 0-centred codes)."""
    from tests.util import packed_case
    N, M = 4096, 512
    cpu, dev = packed_case(N, M, seed=3)
    x = torch.randn(N).half()
    x[1234] = bad
    y = torch.zeros(M, dtype=torch.float32, device="cuda")
    torch.ops.rwkv.mm8_one(N, M, x.cuda(), *dev, y)
    assert torch.isnan(y).all() or torch.isinf(y).all() or (torch.isnan(y) | torch.isinf(y)).all()


def test_mm8_seq_single_pass_option(ops):
    """rwkv_mm8_seq_set_path(4): one tensor-core pass with fp16(x*ry); within two fp16 ulps of the oracle."""
    from chatrwkv_b200._lib import lib
    from tests.util import packed_case
    T, N, M = 256, 1024, 768
    cpu, dev = packed_case(N, M, seed=11)
    g = torch.Generator().manual_seed(12)
    x = torch.randn(T, N, generator=g).half()
    ref = orc.mm8_kernel(x, *cpu).half().float()
    y = torch.empty(T, M, dtype=torch.float16, device="cuda")
    lib().rwkv_mm8_seq_set_path(4)
    try:
        torch.ops.rwkv.mm8_seq(T, N, M, x.cuda(), *dev, y)
        torch.cuda.synchronize()
    finally:
        lib().rwkv_mm8_seq_set_path(0)
    err = (y.float().cpu() - ref).abs()
    assert (err <= 2 * 2.0 ** -10 * ref.abs().clamp(min=1.0)).all(), err.max().item()


# ------------------------------------------------------------------- fused seq epilogues, time-parallel WKV-v4
@pytest.mark.parametrize("T", [3, 40, 200])
def test_mm8_seq_fused_epilogues(ops, T):
    """rwkv_mm8_seq_epi against the oracle's matmul followed by the torch ops of ffn_seq / cuda_att_seq
    (pkg/model.py:995-1004, 1346-1360) in fp16, on all three kernels (CUDA cores, tensor cores, split K)."""
    from chatrwkv_b200 import _lib
    from tests.util import packed_case
    N, M = 512, 768
    cpu, dev = packed_case(N, M, seed=T)
    g = torch.Generator().manual_seed(T)
    x = torch.randn(T, N, generator=g).half()
    aux = torch.randn(T, M, generator=g).half()
    aux2 = torch.rand(T, M, generator=g).half()
    base = orc.mm8_kernel(x, *cpu).half()
    want = {
        _lib.EPI_STORE: base,
        _lib.EPI_SIGMOID: torch.sigmoid(base.float()).half(),
        _lib.EPI_RELU_SQ: (torch.relu(base.float()) ** 2).half(),
        _lib.EPI_RESIDUAL: ((aux.float() + base.float()).half().float() * 0.5).half(),
        _lib.EPI_MUL_RESIDUAL: (aux.float() + (aux2.float() * base.float()).half().float()).half(),
        _lib.EPI_SILU: (base.float() * torch.sigmoid(base.float())).half(),
    }
    for epi, ref in want.items():
        a = aux.cuda().clone()
        y = a if epi == _lib.EPI_RESIDUAL else torch.empty((T, M), dtype=torch.float16, device="cuda")   # in place over aux
        ops.mm8_seq_epi(x.cuda(), *dev, y, epi, aux=a if epi in (_lib.EPI_RESIDUAL, _lib.EPI_MUL_RESIDUAL) else None,
                        aux2=aux2.cuda() if epi == _lib.EPI_MUL_RESIDUAL else None,
                        out_scale=0.5 if epi == _lib.EPI_RESIDUAL else 1.0)
        d = (y.float().cpu() - ref.float()).abs()
        assert (d <= ref.float().abs() * 2 ** -9 + 3e-3).all(), (epi, d.max().item())
        assert (y.cpu() != ref).float().mean().item() < 0.06, epi


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("T", [33, 100, 1024, 2500])
def test_wkv4_time_parallel_matches_sequential_oracle(ops, dtype, T):
    """More than 32 steps run as chunks folded through their summaries; the oracle runs the recurrence step by
    step.  Carried state, a second call, and the fused receptance product."""
    C = 320
    g = torch.Generator().manual_seed(T)
    w = -torch.exp(torch.empty(C).uniform_(-5, 1, generator=g))
    u = torch.empty(C).uniform_(-1, 1, generator=g)
    aa, bb, pp = torch.zeros(C), torch.zeros(C), torch.zeros(C) - 1e30
    daa, dbb, dpp = aa.cuda(), bb.cuda(), pp.cuda()
    tol = 3e-3 if dtype == torch.float16 else 5e-5
    for rep in range(2):
        k = torch.randn(T, C, generator=g).to(dtype)
        v = torch.randn(T, C, generator=g).to(dtype)
        ref = orc.wkv4_forward(T, C, w, u, k, v, aa, bb, pp)
        y = torch.empty((T, C), dtype=dtype, device="cuda")
        if rep == 0:
            torch.ops.rwkv.wkv_forward(1, T, C, w.cuda(), u.cuda(), k.cuda(), v.cuda(), y, daa, dbb, dpp)
            torch.testing.assert_close(y.cpu().float(), ref.float(), rtol=tol, atol=tol)
        else:
            r = torch.rand(T, C, generator=g).to(dtype)
            ops.wkv4_seq(w.cuda(), u.cuda(), k.cuda(), v.cuda(), y, daa, dbb, dpp, r=r.cuda())
            want = (r.float() * ref.to(dtype).float()).to(dtype)
            torch.testing.assert_close(y.cpu().float(), want.float(), rtol=tol, atol=tol)
        torch.testing.assert_close(daa.cpu(), aa, rtol=2e-4, atol=2e-5)
        torch.testing.assert_close(dbb.cpu(), bb, rtol=2e-4, atol=2e-5)
        torch.testing.assert_close(dpp.cpu(), pp, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("which", [5, 6])
@pytest.mark.parametrize("T", [65, 200, 2048])
def test_wkv56_time_parallel_matches_sequential_oracle(ops, which, T):
    """More than 64 steps: chunk sums, a scan of the chunk-start states, the chunks again.  Against the step-by-step
    oracle; operator layout through torch.ops, then the model's transposed layout with a separate output state and
    fp16 r, k, v (what RWKV.forward calls)."""
    N, H = 64, 3
    C = N * H
    g = torch.Generator().manual_seed(T + which)
    r = torch.randn(T, C, generator=g)
    k = torch.randn(T, C, generator=g) * 0.5
    v = torch.randn(T, C, generator=g)
    u = torch.empty(C).uniform_(-1, 1, generator=g)
    state = torch.randn(H, N, N, generator=g) * 0.1
    if which == 6:
        w = torch.exp(-torch.exp(torch.empty(T, C).uniform_(-5, 1, generator=g)))
        ofn, fn = orc.wkv6_forward, torch.ops.rwkv6.forward_fp32
    else:
        w = torch.exp(-torch.exp(torch.empty(C).uniform_(-5, 1, generator=g)))
        ofn, fn = orc.wkv5_forward, torch.ops.rwkv5.forward_fp32
    s_ref = state.clone()
    ref = ofn(1, T, C, H, s_ref, r, k, v, w, u)
    ds = state.clone().cuda()
    y = torch.empty((T, C), device="cuda")
    fn(1, T, C, H, ds, r.cuda(), k.cuda(), v.cuda(), w.cuda(), u.cuda(), y)
    scale = max(1.0, ref.abs().max().item())
    assert (y.cpu() - ref).abs().max().item() <= 2e-4 * scale
    torch.testing.assert_close(ds.cpu(), s_ref, rtol=2e-4, atol=2e-4)
    # the model's call: fp16 r, k, v, state [H, key, value], new state in a separate tensor
    rh, kh, vh = r.half(), k.half(), v.half()
    s_ref2 = state.clone()
    ref2 = ofn(1, T, C, H, s_ref2, rh.float(), kh.float(), vh.float(), w, u)
    s_in = state.transpose(-1, -2).contiguous().cuda()
    s_keep = s_in.clone()
    s_out = torch.empty_like(s_in)
    y2 = torch.empty((T, C), device="cuda")
    ops.wkv56_seq(which == 6, H, s_in, rh.cuda(), kh.cuda(), vh.cuda(), w.cuda(), u.cuda(), y2, model_layout=True, state_out=s_out)
    assert (y2.cpu() - ref2).abs().max().item() <= 2e-4 * max(1.0, ref2.abs().max().item())
    torch.testing.assert_close(s_out.transpose(-1, -2).cpu(), s_ref2, rtol=2e-4, atol=2e-4)
    assert torch.equal(s_in, s_keep)


@pytest.mark.parametrize("D,V", [(4096, 1000), (100, 7), (768, 50277)])
def test_embed_row(ops, D, V):
    """rwkv_embed_row copies the row a device-side token id names (pkg/model.py:1475); an id outside the vocabulary
    reads the nearest valid row instead of faulting."""
    from chatrwkv_b200._lib import check, lib
    g = torch.Generator().manual_seed(D + V)
    emb = torch.randn(V, D, generator=g).half().cuda()
    out = torch.zeros(D, dtype=torch.float16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    for tok, row in ((0, 0), (V - 1, V - 1), (V // 2, V // 2), (V + 5, V - 1), (-3, 0)):
        t = torch.tensor([tok], dtype=torch.int64, device="cuda")
        check(lib().rwkv_embed_row(D, V, emb.data_ptr(), emb.stride(0), t.data_ptr(), out.data_ptr(), st), "embed_row")
        torch.cuda.synchronize()
        assert torch.equal(out, emb[row]), tok
