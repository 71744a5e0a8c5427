"""The operator boundary of the reference, re-registered over the sm_100a kernels.

Registers, with the reference's argument lists (rwkv_pip_package/src/rwkv/cuda/wrapper.cpp:
125-141, rwkv5_op.cpp:30-34, rwkv6_op.cpp:30-34):

    torch.ops.rwkv.mm8_one(N, M, x, w, mx, rx, my, ry, y)
    torch.ops.rwkv.mm8_seq(B, N, M, x, w, mx, rx, my, ry, y)
    torch.ops.rwkv.wkv_forward(B, T, C, w, u, k, v, y, aa, bb, pp)
    torch.ops.rwkv.gemm_fp16_cublas(a, b, c)
    torch.ops.rwkv5.forward_{bf16,fp16,fp32}(B, T, C, H, state, r, k, v, w, u, y)
    torch.ops.rwkv6.forward_{bf16,fp16,fp32}(B, T, C, H, state, r, k, v, w, u, y)

Outputs are written in place into caller-allocated tensors, as in the reference.  Where
the reference aborts with a C assert (non-unit inner strides, unsupported dtype) these
raise.  Kernels run on torch's current stream, so calls can be captured into CUDA graphs
(the reference launches on the legacy default stream).

Also exposes `quantize_weight`, the loader's inline packing block (model.py:818-847) as a
function.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import Mm8Problem, check, lib

_DT = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}

# ---------------------------------------------------------------------------------------
# workspace: one zero-initialised buffer per (device, stream); kernels leave it clean.
# ---------------------------------------------------------------------------------------
_workspaces = {}


def workspace(device, nbytes, kind="mm8_one"):
    """Scratch of an operator (split-K partials and tickets of mm8_one; hi/lo activation copies
    of the tensor-core mm8_seq).  Keyed by (kind, device, stream): the kinds lay their buffers
    out differently and mm8_one relies on finding its tickets zero, so they never share one;
    calls that share a buffer are ordered by the stream."""
    if nbytes == 0:
        return None
    key = (kind, device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        if torch.cuda.is_current_stream_capturing():
            raise _lib.RwkvB200Error("workspace must be sized before stream capture (run one eager step first)")
        buf = torch.zeros(max(nbytes, 64 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def _stream(device):
    return torch.cuda.current_stream(device).cuda_stream


def _require(cond, msg):
    if not cond:
        raise _lib.RwkvB200Error(msg)


# ---------------------------------------------------------------------------------------
# packing
# ---------------------------------------------------------------------------------------
def padded_stride(M):
    """Row stride (bytes) of a packed matrix: rows start on 16-byte boundaries so that every
    row can be read with 128-bit loads (and by TMA), e.g. 50277 -> 50288."""
    return (M + 15) // 16 * 16


def quantize_weight(w, atype=torch.float16, scale=1.0):
    """uint8-pack `w[N_in, M_out]` (any strides, e.g. the `.t()` view of an nn.Linear
    weight; fp32, fp16 or bf16) on the GPU.

    Returns `(q, mx, rx, my, ry)`: `q` uint8 of shape [N, M] whose row stride is padded to a
    multiple of 16 bytes; `mx`, `rx` of shape [M] and `my`, `ry` of shape [N, 1] in `atype`,
    bit-identical to the reference loader's values (model.py:822-847).  `scale` (a power of
    two) multiplies the source first: the loader's division of att.output / ffn.value by
    2**(layer // 6) (model.py:785-789).
    """
    _require(w.is_cuda and w.dim() == 2, "quantize_weight needs a 2-D CUDA tensor")
    _require(w.dtype in _DT and atype in (torch.float16, torch.float32), "unsupported dtype")
    N, M = w.shape
    dev = w.device
    with torch.cuda.device(dev):
        q_full = torch.empty((N, padded_stride(M)), dtype=torch.uint8, device=dev)
        if padded_stride(M) != M:
            q_full[:, M:].zero_()
        q = q_full[:, :M]
        mx = torch.empty(M, dtype=atype, device=dev)
        rx = torch.empty(M, dtype=atype, device=dev)
        my = torch.empty((N, 1), dtype=atype, device=dev)
        ry = torch.empty((N, 1), dtype=atype, device=dev)
        nbytes = lib().rwkv_quantize_weight_workspace_bytes(N, M)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        check(lib().rwkv_quantize_weight(
            w.data_ptr(), _DT[w.dtype], w.stride(0), w.stride(1), float(scale), N, M,
            q.data_ptr(), q.stride(0), mx.data_ptr(), rx.data_ptr(), my.data_ptr(), ry.data_ptr(),
            _DT[atype], ws.data_ptr(), nbytes, _stream(dev)), "quantize_weight")
    return q, mx, rx, my, ry


# ---------------------------------------------------------------------------------------
# op implementations (in-place, reference argument order)
# ---------------------------------------------------------------------------------------
def _check_mm8(x, w, mx, rx, my, ry, y):
    _require(w.dtype == torch.uint8 and w.stride(1) == 1, "w must be uint8 with unit inner stride")
    _require(x.stride(-1) == 1 and y.stride(-1) == 1, "x and y need unit inner stride")
    _require(mx.stride(0) == 1 and rx.stride(0) == 1 and my.stride(0) == 1 and ry.stride(0) == 1,
             "scale vectors need unit stride")
    _require(x.dtype in (torch.float16, torch.float32), "Only FP16 and FP32 are currently supported")
    _require(x.dtype == mx.dtype == rx.dtype == my.dtype == ry.dtype, "x and the scale vectors must share a dtype")


def mm8_one_(N, M, x, w, mx, rx, my, ry, y):
    _check_mm8(x, w, mx, rx, my, ry, y)
    _require(y.dtype == torch.float32, "mm8_one accumulates into an fp32 y")
    dev = w.device
    with torch.cuda.device(dev):
        nbytes = lib().rwkv_mm8_one_workspace_bytes(N, M)
        ws = workspace(dev, nbytes)
        check(lib().rwkv_mm8_one(N, M, x.data_ptr(), w.data_ptr(), w.stride(0), mx.data_ptr(), rx.data_ptr(),
                                 my.data_ptr(), ry.data_ptr(), _DT[x.dtype], y.data_ptr(),
                                 ws.data_ptr(), ws.numel(), _stream(dev)), "mm8_one")


def mm8_seq_(B, N, M, x, w, mx, rx, my, ry, y):
    _check_mm8(x, w, mx, rx, my, ry, y)
    _require(y.dtype == x.dtype, "mm8_seq writes y in x.dtype")
    dev = w.device
    with torch.cuda.device(dev):
        nbytes = lib().rwkv_mm8_seq_workspace_bytes(B, N, M)
        ws = workspace(dev, nbytes, "mm8_seq")
        check(lib().rwkv_mm8_seq(B, N, M, x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0),
                                 mx.data_ptr(), rx.data_ptr(), my.data_ptr(), ry.data_ptr(), _DT[x.dtype],
                                 y.data_ptr(), y.stride(0), ws.data_ptr() if ws is not None else None,
                                 ws.numel() if ws is not None else 0, _stream(dev)), "mm8_seq")


def mm8_seq_epi(x, w, mx, rx, my, ry, y, epilogue, aux=None, aux2=None, out_scale=1.0):
    """mm8_seq with a fused epilogue (`_lib.EPI_*`; rwkv_mm8_seq_epi in the header): y[B, M] = epilogue(x[B, N] @ W).
    aux / aux2: [B, M] tensors of y's dtype (row strides honoured); y may alias aux."""
    _check_mm8(x, w, mx, rx, my, ry, y)
    _require(y.dtype == x.dtype, "mm8_seq writes y in x.dtype")
    for t in (aux, aux2):
        _require(t is None or (t.dtype == y.dtype and t.shape == y.shape and t.stride(-1) == 1), "aux must look like y")
    B, N = x.shape
    M = w.shape[1]
    dev = w.device
    with torch.cuda.device(dev):
        nbytes = lib().rwkv_mm8_seq_workspace_bytes(B, N, M)
        ws = workspace(dev, nbytes, "mm8_seq")
        check(lib().rwkv_mm8_seq_epi(B, N, M, x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0),
                                     mx.data_ptr(), rx.data_ptr(), my.data_ptr(), ry.data_ptr(), _DT[x.dtype],
                                     y.data_ptr(), y.stride(0), epilogue,
                                     aux.data_ptr() if aux is not None else None, aux.stride(0) if aux is not None else 0,
                                     aux2.data_ptr() if aux2 is not None else None, aux2.stride(0) if aux2 is not None else 0,
                                     float(out_scale), ws.data_ptr() if ws is not None else None,
                                     ws.numel() if ws is not None else 0, _stream(dev)), "mm8_seq_epi")
    return y


def wkv4_seq(w, u, k, v, y, aa, bb, pp, r=None):
    """WKV-v4 over k, v [T, C] (or [B, T, C]) with the state aa, bb, pp updated in place, parallel in time from 33
    steps on; with `r`, y = r * wkv rounded as cuda_att_seq does (rwkv_wkv4_seq in the header)."""
    _require(k.dtype in (torch.float16, torch.float32) and k.dtype == v.dtype == y.dtype, "Only FP16 and FP32 are currently supported")
    _require(r is None or r.dtype == k.dtype, "r must have k's dtype")
    _require(all(t.dtype == torch.float32 for t in (w, u, aa, bb, pp)), "w, u and the state must be fp32")
    _require(all(t is None or t.is_contiguous() for t in (w, u, k, v, y, aa, bb, pp, r)), "wkv needs contiguous tensors")
    B = k.shape[0] if k.dim() == 3 else 1
    T, C = k.shape[-2], k.shape[-1]
    dev = w.device
    with torch.cuda.device(dev):
        nbytes = lib().rwkv_wkv4_workspace_bytes(B, T, C)
        ws = workspace(dev, nbytes, "wkv4")
        check(lib().rwkv_wkv4_seq(B, T, C, w.data_ptr(), u.data_ptr(), k.data_ptr(), v.data_ptr(),
                                  r.data_ptr() if r is not None else None, y.data_ptr(), _DT[k.dtype],
                                  aa.data_ptr(), bb.data_ptr(), pp.data_ptr(), ws.data_ptr() if ws is not None else None,
                                  ws.numel() if ws is not None else 0, _stream(dev)), "wkv4_seq")
    return y


def wkv_forward_(B, T, C, w, u, k, v, y, aa, bb, pp):
    _require(k.dtype in (torch.float16, torch.float32) and k.dtype == v.dtype == y.dtype,
             "Only FP16 and FP32 are currently supported")
    _require(all(t.dtype == torch.float32 for t in (w, u, aa, bb, pp)), "w, u and the state must be fp32")
    _require(all(t.is_contiguous() for t in (w, u, k, v, y, aa, bb, pp)), "wkv_forward needs contiguous tensors")
    dev = w.device
    with torch.cuda.device(dev):
        nbytes = lib().rwkv_wkv4_workspace_bytes(B, T, C)
        ws = workspace(dev, nbytes, "wkv4")
        check(lib().rwkv_wkv4_seq(B, T, C, w.data_ptr(), u.data_ptr(), k.data_ptr(), v.data_ptr(), None, y.data_ptr(),
                                  _DT[k.dtype], aa.data_ptr(), bb.data_ptr(), pp.data_ptr(),
                                  ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0, _stream(dev)),
              "wkv_forward")


def gemm_fp16_cublas_(a, b, c):
    """c = a @ b for fp16 a, b (2-D, or 3-D batched) with fp32 accumulation, c fp16 or fp32, written in place: the
    plain library GEMM the reference keeps for its un-quantised 'cuda fp16' strategy
    (rwkv_pip_package/src/rwkv/cuda/gemm_fp16_cublas.cpp:28-75, called from model.py:143-162).  It is not on the
    fp16i8 path (every 2-D weight is uint8 there); it is registered so that code written against the reference's
    operator set finds the name, and runs on the same library (cuBLAS through torch.matmul)."""
    _require(a.dtype == torch.float16 and b.dtype == torch.float16, "gemm_fp16_cublas multiplies fp16 tensors")
    _require(c.dtype in (torch.float16, torch.float32), "c must be fp16 or fp32")
    _require(a.dim() == b.dim() and a.dim() in (2, 3), "a and b must both be 2-D or both 3-D")
    _require(a.is_contiguous() and b.is_contiguous() and c.is_contiguous(), "needs contiguous tensors")
    _require(tuple(c.shape) == tuple(a.shape[:-1]) + (b.shape[-1],) and a.shape[-1] == b.shape[-2], "shape mismatch")
    with torch.cuda.device(a.device):
        if c.dtype == torch.float16:
            torch.matmul(a, b, out=c)
        else:
            c.copy_(torch.matmul(a, b))


def _wkv56(which, dtype):
    fn_name = f"rwkv_wkv{which}_forward"

    def impl(B, T, C, H, state, r, k, v, w, u, y):
        _require(state.dtype == torch.float32 and w.dtype == torch.float32, "state and w must be fp32")
        _require(r.dtype == k.dtype == v.dtype == u.dtype == y.dtype == dtype, f"r, k, v, u, y must be {dtype}")
        _require(all(t.is_contiguous() for t in (state, r, k, v, w, u, y)), "needs contiguous tensors")
        _require(B == 1, "B must be 1 (the reference's kernels are wrong for B > 1 as well, rwkv6.cu:17)")
        wkv56_seq(which == 6, H, state, r, k, v, w, u, y, model_layout=False)
    return impl


def wkv56_seq(per_token_w, H, state, r, k, v, w, u, y, model_layout=False, state_out=None):
    """WKV5 (w [H*N]) or WKV6 (w [T, C]) over r, k, v [T, C]; state fp32 [H, N, N] updated in place, in the operators'
    [H, value, key] layout or, with `model_layout`, the [H, key, value] layout of the model's state list.  r, k, v
    may be fp16 with fp32 u, y (the model's sequence path).  `state_out`: where the new state goes (default: in
    place).  Parallel in time from 65 steps on."""
    T, C = r.shape[-2], r.shape[-1]
    dev = state.device
    with torch.cuda.device(dev):
        nbytes = lib().rwkv_wkv56_workspace_bytes(T, C, H)
        ws = workspace(dev, nbytes, "wkv56")
        check(lib().rwkv_wkv56_seq(1 if per_token_w else 0, T, C, H, state.data_ptr(),
                                   (state_out if state_out is not None else state).data_ptr(), 1 if model_layout else 0,
                                   r.data_ptr(), k.data_ptr(), v.data_ptr(), w.data_ptr(), u.data_ptr(), y.data_ptr(),
                                   _DT[r.dtype], _DT[y.dtype], ws.data_ptr() if ws is not None else None,
                                   ws.numel() if ws is not None else 0, _stream(dev)), "wkv56_seq")
    return y


# ---------------------------------------------------------------------------------------
# torch.library registration
# ---------------------------------------------------------------------------------------
_libs = []


def _register():
    T7 = "Tensor x, Tensor w, Tensor mx, Tensor rx, Tensor my, Tensor ry, Tensor(a!) y"
    rw = torch.library.Library("rwkv", "DEF")
    rw.define(f"mm8_one(int N, int M, {T7}) -> ()")
    rw.define(f"mm8_seq(int B, int N, int M, {T7}) -> ()")
    rw.define("wkv_forward(int B, int T, int C, Tensor w, Tensor u, Tensor k, Tensor v, Tensor(a!) y, "
              "Tensor(b!) aa, Tensor(c!) bb, Tensor(d!) pp) -> ()")
    rw.define("gemm_fp16_cublas(Tensor a, Tensor b, Tensor(a!) c) -> ()")
    rw.impl("gemm_fp16_cublas", gemm_fp16_cublas_, "CUDA")
    rw.impl("mm8_one", mm8_one_, "CUDA")
    rw.impl("mm8_seq", mm8_seq_, "CUDA")
    rw.impl("wkv_forward", wkv_forward_, "CUDA")
    _libs.append(rw)
    sig = ("(int B, int T, int C, int H, Tensor(a!) state, Tensor r, Tensor k, Tensor v, Tensor w, Tensor u, "
           "Tensor(b!) y) -> ()")
    for which in (5, 6):
        lb = torch.library.Library(f"rwkv{which}", "DEF")
        for suffix, dt in (("bf16", torch.bfloat16), ("fp16", torch.float16), ("fp32", torch.float32)):
            lb.define(f"forward_{suffix}{sig}")
            lb.impl(f"forward_{suffix}", _wkv56(which, dt), "CUDA")
        _libs.append(lb)


_register()


class _Wkv56Module:
    """Stands in for the `rwkv5` / `rwkv6` extension modules the reference loads
    (model.py:907, 940): same function names, same argument order."""

    def __init__(self, which):
        ns = getattr(torch.ops, f"rwkv{which}")
        self.forward_bf16 = ns.forward_bf16
        self.forward_fp16 = ns.forward_fp16
        self.forward_fp32 = ns.forward_fp32


rwkv5 = _Wkv56Module(5)
rwkv6 = _Wkv56Module(6)


# ---------------------------------------------------------------------------------------
# fused GEMV launches for the decode step
# ---------------------------------------------------------------------------------------
def make_problem(x, w, mx, rx, my, ry, y, epilogue, aux=None, aux2=None, out_scale=1.0):
    p = Mm8Problem()
    p.x, p.w, p.w_stride = x.data_ptr(), w.data_ptr(), w.stride(0)
    p.mx, p.rx, p.my, p.ry = mx.data_ptr(), rx.data_ptr(), my.data_ptr(), ry.data_ptr()
    p.y = y.data_ptr()
    p.aux = aux.data_ptr() if aux is not None else None
    p.aux2 = aux2.data_ptr() if aux2 is not None else None
    p.N, p.M = w.shape
    p.epilogue, p.out_scale = epilogue, out_scale
    p.prologue = _lib.PRO_PLAIN
    return p


def with_ln_mix(p, ln_w, ln_b, mode, sx=None, mix=None, xx_out=None):
    """Turn `p.x` into the residual stream: LayerNorm + token-shift mix happen in the kernel."""
    p.prologue, p.mode = _lib.PRO_LN_MIX, mode
    p.ln_w, p.ln_b = ln_w.data_ptr(), ln_b.data_ptr()
    p.sx = sx.data_ptr() if sx is not None else None
    p.mix = mix.data_ptr() if mix is not None else None
    p.xx_out = xx_out.data_ptr() if xx_out is not None else None
    return p


def with_wkv4(p, k, v, t_decay, t_first, state_in, state_out):
    """`p.x` is r; the kernel runs the RWKV-4 one-step WKV and multiplies r * wkv."""
    p.prologue = _lib.PRO_WKV4
    p.k, p.v = k.data_ptr(), v.data_ptr()
    p.t_decay, p.t_first = t_decay.data_ptr(), t_first.data_ptr()
    p.aa, p.bb, p.pp = (t.data_ptr() for t in state_in)
    p.aa_out, p.bb_out, p.pp_out = (t.data_ptr() for t in state_out)
    return p


def mm8_one_batch(problems, dtype, device, ws=None, exchange=None, flags=0):
    """One launch for 1..4 GEMVs with fused epilogues.  `ws`: zero-initialised uint8 scratch
    owned by the caller (needed under stream capture); default: the per-stream workspace.
    `exchange` (an `_lib.Mm8Exchange`): column-sharded launch that also stores its results into
    the other ranks' buffers (shard.PeerRegion.exchange).  `flags`: _lib.MM8_WIDE_BUILD (see the header)."""
    import ctypes as C
    n = len(problems)
    arr = (Mm8Problem * n)(*problems)
    if ws is None:
        ws = workspace(device, lib().rwkv_mm8_one_batch_workspace_bytes(arr, n))
    check(lib().rwkv_mm8_one_batch_flags(arr, n, C.byref(exchange) if exchange is not None else None, _DT[dtype], flags,
                                         ws.data_ptr(), ws.numel(), _stream(device)), "mm8_one_batch")
