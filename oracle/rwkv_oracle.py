"""CPU restatement of the rwkv pip package's quantized ('fp16i8' / 'fp32i8') inference path.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this module; it is the
checker used by tests/, by the smoke test and by the CPU-baseline legs of bench.py.

Parity status: PINNED against outputs of the reference itself, executed on CPU from the
read-only reference tree (strategy 'cpu fp32i8', RWKV_CUDA_ON=0).  The reference holds no
golden vectors of its own for this path, so tests/golden/make_golden.py ran the reference
and committed its outputs (packed tensors, torch_mm8 results, per-version logits and
states); tests/test_oracle_golden.py checks every function below against them.

Every function cites the reference lines it restates; paths are relative to the reference
project root, `pkg/` = rwkv_pip_package/src/rwkv/.
"""
from __future__ import annotations

import math
import types

import torch
import torch.nn.functional as F

# --------------------------------------------------------------------------------------
# int8 packing  (pkg/model.py:818-847)
# --------------------------------------------------------------------------------------

def quantize_weight(w: torch.Tensor, atype: torch.dtype = torch.float16):
    """Pack fp32 `w[N_in, M_out]` into uint8 codes plus four scale vectors.

    Restates the inline block pkg/model.py:822-847: subtract the row minimum `my` and the
    column minimum `mx` (row first when N_in > M_out, column first otherwise), divide by
    the column maximum `rx`, then by the row maximum `ry`, and code floor(w*256) clipped to
    0..255.  Returns (q uint8 [N,M], mx [M], rx/16 [M], my [N,1], ry/16 [N,1]) with the
    scale vectors cast to `atype`.
    """
    w = w.float().clone()
    if w.shape[0] > w.shape[1]:
        my = torch.amin(w, dim=1).unsqueeze(1)
        w = w - my
        mx = torch.amin(w, dim=0)
        w = w - mx
    else:
        mx = torch.amin(w, dim=0)
        w = w - mx
        my = torch.amin(w, dim=1).unsqueeze(1)
        w = w - my
    rx = torch.amax(w, dim=0)
    w = w / rx
    ry = torch.amax(w, dim=1).unsqueeze(1)
    w = w / ry
    q = torch.clip(torch.floor(w * 256), min=0, max=255).to(dtype=torch.uint8)
    return (q,
            mx.to(dtype=atype).contiguous(),
            (rx / 16).to(dtype=atype).contiguous(),
            my.to(dtype=atype).contiguous(),
            (ry / 16).to(dtype=atype).contiguous())


# --------------------------------------------------------------------------------------
# mm8  (spec: pkg/model.py:91-97; kernel arithmetic: pkg/cuda/operators.cu:116-140, 207-232)
# --------------------------------------------------------------------------------------

def dequant(w, mx, rx, my, ry, dtype=torch.float32):
    """`(w + 0.5) * ry * rx + my + mx` in `dtype` (pkg/model.py:93)."""
    return (w.to(dtype=dtype) + 0.5) * ry.to(dtype) * rx.to(dtype) + my.to(dtype) + mx.to(dtype)


def mm8_spec(x, w, mx, rx, my, ry):
    """The pure-torch specification the reference uses on CPU: dequantise the whole matrix
    in x.dtype, then `x @` (pkg/model.py:91-97)."""
    return x @ ((w.to(dtype=x.dtype) + 0.5) * ry * rx + my + mx)


def mm8_kernel(x, w, mx, rx, my, ry):
    """What the reference CUDA kernels compute for fp16 operands: every operand widened to
    fp32, the sum over the reduction index accumulated wide (operators.cu:130-138,
    224-230).  Accumulation here is float64 so the result is the exactly-rounded fp32 sum,
    independent of summation order.  Returns fp32 `[M]` or `[T, M]`."""
    deq = dequant(w, mx.float(), rx.float(), my.float(), ry.float(), torch.float32)
    return (x.double() @ deq.double()).float()


def mm8_one_fp16(x, w, mx, rx, my, ry):
    """cuda_mm8_one wrapper semantics: fp32 accumulation, then one rounding to x.dtype
    (pkg/model.py:84-86)."""
    return mm8_kernel(x, w, mx, rx, my, ry).to(x.dtype)


mm8_seq_fp16 = mm8_one_fp16  # pkg/model.py:72-74 and operators.cu:138: same rounding point


# --------------------------------------------------------------------------------------
# WKV recurrences
# --------------------------------------------------------------------------------------

def wkv4_forward(T, C, w, u, k, v, aa, bb, pp):
    """RWKV-4 log-space recurrence, one channel per lane, sequential in t
    (operators.cu:30-46 == pkg/model.py:1069-1084).  `w = -exp(time_decay)`, `u =
    time_first`; k, v `[T, C]`; state aa, bb, pp `[C]` fp32 updated IN PLACE.  Returns y
    `[T, C]` in k.dtype."""
    y = torch.empty((T, C), dtype=k.dtype)
    a, b, p = aa.clone().float(), bb.clone().float(), pp.clone().float()
    w = w.float()
    u = u.float()
    for t in range(T):
        kk = k[t].float()
        vv = v[t].float()
        ww = u + kk
        q = torch.maximum(p, ww)
        e1 = torch.exp(p - q)
        e2 = torch.exp(ww - q)
        y[t] = ((e1 * a + e2 * vv) / (e1 * b + e2)).to(k.dtype)
        ww = w + p
        q = torch.maximum(ww, kk)
        e1 = torch.exp(ww - q)
        e2 = torch.exp(kk - q)
        a = e1 * a + e2 * vv
        b = e1 * b + e2
        p = q
    aa.copy_(a)
    bb.copy_(b)
    pp.copy_(p)
    return y


def wkv5_forward(B, T, C, H, state, r, k, v, w, u):
    """RWKV-5 matrix-state recurrence with a static per-head decay (pkg/cuda/rwkv5.cu:32-68
    == pkg/model.py:1245-1251).  `state` fp32 `[H, N, N]` in the KERNEL layout
    `[head, value index i, key index j]`, updated in place; r, k, v `[T, C]`; `w`
    (already exp(-exp(decay))) and `u` hold H*N values.  Returns y `[T, C]` in r.dtype."""
    assert B == 1
    N = C // H
    S = state.view(H, N, N).clone().double()
    wv = w.reshape(H, 1, N).double()
    uv = u.reshape(H, 1, N).double()
    y = torch.empty((T, C), dtype=r.dtype)
    for t in range(T):
        rt = r[t].view(H, 1, N).double()
        kt = k[t].view(H, 1, N).double()
        vt = v[t].view(H, N, 1).double()
        x = vt * kt                      # x[h, i, j] = k[j] * v[i]
        y[t] = ((uv * x + S) * rt).sum(-1).reshape(C).to(r.dtype)
        S = S * wv + x
    state.view(H, N, N).copy_(S.float())
    return y


def wkv6_forward(B, T, C, H, state, r, k, v, w, u):
    """RWKV-6: as wkv5_forward but the decay is per token, `w[T, C]` already
    exp(-exp(.)) (pkg/cuda/rwkv6.cu:30-67 == pkg/model.py:1324-1333)."""
    assert B == 1
    N = C // H
    S = state.view(H, N, N).clone().double()
    uv = u.reshape(H, 1, N).double()
    y = torch.empty((T, C), dtype=r.dtype)
    for t in range(T):
        rt = r[t].view(H, 1, N).double()
        kt = k[t].view(H, 1, N).double()
        vt = v[t].view(H, N, 1).double()
        wt = w[t].view(H, 1, N).double()
        x = vt * kt
        y[t] = ((uv * x + S) * rt).sum(-1).reshape(C).to(r.dtype)
        S = S * wt + x
    state.view(H, N, N).copy_(S.float())
    return y


# --------------------------------------------------------------------------------------
# Model: loader transforms + forward  (pkg/model.py:613-903, 984-1439, 1443-1677)
# --------------------------------------------------------------------------------------

def _ln(x, w, b):
    # F.layer_norm on fp16 computes in fp32 and rounds once; do that explicitly so the
    # result does not depend on the CPU half kernels.
    return F.layer_norm(x.float(), (x.shape[-1],), weight=w.float(), bias=b.float()).to(x.dtype)


class OracleRWKV:
    """Restatement of `RWKV(model, strategy)` for a single-device 'xxx fp16i8' / 'fp32i8'
    strategy.

    `atype=torch.float32` reproduces the reference's 'cpu fp32i8' path (RESCALE_LAYER 0,
    mm8 = dequantise then matmul in fp32).  `atype=torch.float16` reproduces the arithmetic
    of its 'cuda fp16i8' path with RWKV_CUDA_ON=1: fp16 activations with one rounding per
    torch op, mm8 with fp32 accumulation and one rounding (pkg/model.py:63-86), fp32 WKV
    state, RESCALE_LAYER 6 (pkg/model.py:634).
    """

    def __init__(self, ckpt: dict, atype=torch.float16, rescale_layer=None, i8_layers=None):
        """`i8_layers`: how many layers, from the first, hold int8 matrices (the reference's 'xxx fp16i8 *K -> xxx
        fp16', pkg/model.py:684-749: the rest and the head keep plain weights of the activation dtype); None = all
        layers and the head ('xxx fp16i8'), 0 = none ('xxx fp16')."""
        self.atype = atype
        self.i8_layers = i8_layers
        self.RESCALE_LAYER = (6 if atype == torch.float16 else 0) if rescale_layer is None else rescale_layer
        w = {k: v.clone() for k, v in ckpt.items()}
        args = types.SimpleNamespace()
        self.args = args
        args.n_embd = w["emb.weight"].shape[1]
        args.n_att = w["blocks.0.att.key.weight"].shape[0]
        args.n_ffn = w["blocks.0.ffn.key.weight"].shape[0]
        args.n_layer = 0
        self.version = 4
        for x in list(w.keys()):                       # pkg/model.py:662-679
            layer_id = int(x.split(".")[1]) if ("blocks." in x) else 0
            args.n_layer = max(args.n_layer, layer_id + 1)
            if "ln_x" in x:
                self.version = max(5, self.version)
            if "gate.weight" in x:
                self.version = max(5.1, self.version)
            if int(self.version) == 5 and "att.time_decay" in x:
                args.n_head = w[x].shape[0]
                if len(w[x].shape) > 1 and w[x].shape[1] > 1:
                    self.version = max(5.2, self.version)
            if "time_maa" in x:
                self.version = max(6, self.version)
            if int(self.version) == 6 and "time_faaaa" in x:
                args.n_head = w[x].shape[0]
        assert self.version in (4, 5.2, 6), "oracle covers v4, v5.2 and v6"

        # pkg/model.py:754-760
        w["emb.weight"] = F.layer_norm(w["emb.weight"].float(), (args.n_embd,),
                                       weight=w["blocks.0.ln0.weight"].float(),
                                       bias=w["blocks.0.ln0.bias"].float())
        del w["blocks.0.ln0.weight"], w["blocks.0.ln0.bias"]
        real_time_first = any(".time_faaaa" in k for k in w)
        if real_time_first:
            w = {k.replace(".time_faaaa", ".time_first"): v for k, v in w.items()}

        for x in list(w.keys()):                       # pkg/model.py:774-849
            layer_id = int(x.split(".")[1]) if ("blocks." in x) else 0
            if ("ln_out." in x) or ("head." in x):
                layer_id = args.n_layer
            if self.RESCALE_LAYER > 0:
                if "att.output.weight" in x or "ffn.value.weight" in x:
                    w[x] = w[x] / (2 ** int(layer_id // self.RESCALE_LAYER))
            if ".time_" in x:
                w[x] = w[x].squeeze()
            if any(s in x for s in ("key.weight", "value.weight", "receptance.weight",
                                    "gate.weight", "output.weight", "head.weight")):
                w[x] = w[x].t()
            if ".time_decay" in x and "_w" not in x:
                if self.version == 4:
                    w[x] = -torch.exp(w[x].float())
                elif self.version == 5.2:
                    w[x] = torch.exp(-torch.exp(w[x].float())).reshape(args.n_head, -1, 1)
                else:
                    w[x] = w[x].float().reshape(args.n_head, -1, 1)
            elif ".time_first" in x:
                if self.version == 4:
                    w[x] = w[x].float()
                else:
                    if real_time_first:
                        w[x] = w[x].float().reshape(-1, 1, 1)
                    else:
                        w[x] = torch.exp(w[x].float()).reshape(-1, 1, 1)
                    w[x] = w[x].reshape(args.n_head, -1, 1)
            elif ".ln_x" in x:
                w[x] = w[x].float()
            else:
                packed = i8_layers is None or layer_id < i8_layers
                if len(w[x].shape) == 2 and "emb" not in x and "_w1" not in x and "_w2" not in x and packed:
                    q, mx, rx, my, ry = quantize_weight(w[x], atype)
                    w[x] = q
                    w[x + "_mx"], w[x + "_rx"], w[x + "_my"], w[x + "_ry"] = mx, rx, my, ry
                else:
                    w[x] = w[x].to(dtype=atype)
        self.w = w
        self._deq = {}

    # ----- matmul ---------------------------------------------------------------------
    def _mm(self, x, name, out_dtype=None):
        """pkg/model.py:127-138: mm8 in the activation dtype, then `.to(output_dtype)`."""
        w = self.w
        if w[name].dtype != torch.uint8:                 # pkg/model.py:143-167: a plain matmul in the activation dtype
            y = (x.float() @ w[name].float()).to(self.atype)
            return y if out_dtype is None else y.to(out_dtype)
        if name not in self._deq:
            self._deq[name] = dequant(w[name], w[name + "_mx"].float(), w[name + "_rx"].float(),
                                      w[name + "_my"].float(), w[name + "_ry"].float())
        y = (x.float() @ self._deq[name]).to(self.atype)
        return y if out_dtype is None else y.to(out_dtype)

    def zero_state(self):
        """pkg/model.py:1448-1471."""
        a = self.args
        st = []
        for _ in range(a.n_layer):
            if self.version == 4:
                st += [torch.zeros(a.n_embd, dtype=self.atype), torch.zeros(a.n_att), torch.zeros(a.n_att),
                       torch.zeros(a.n_att) - 1e30, torch.zeros(a.n_embd, dtype=self.atype)]
            else:
                N = a.n_att // a.n_head
                st += [torch.zeros(a.n_embd, dtype=self.atype), torch.zeros(a.n_head, N, N),
                       torch.zeros(a.n_embd, dtype=self.atype)]
        return st

    # ----- blocks (sequence form; T=1 is the one-step form) -----------------------------
    def _ffn(self, x, sx, i):
        """ffn_one / ffn_seq / ffn_*_v6 (pkg/model.py:984-1029)."""
        w = self.w
        b, f = f"blocks.{i}.", f"blocks.{i}.ffn."
        xx = _ln(x, w[b + "ln2.weight"], w[b + "ln2.bias"])
        sxx = torch.cat((sx.unsqueeze(0), xx[:-1, :]))
        if self.version == 6:
            d = sxx - xx
            kx = xx + d * w[f + "time_maa_k"]
            rx = xx + d * w[f + "time_maa_r"]
        else:
            kx = xx * w[f + "time_mix_k"] + sxx * (1 - w[f + "time_mix_k"])
            rx = xx * w[f + "time_mix_r"] + sxx * (1 - w[f + "time_mix_r"])
        r = torch.sigmoid(self._mm(rx, f + "receptance.weight"))
        vx = torch.relu(self._mm(kx, f + "key.weight")) ** 2
        out = r * self._mm(vx, f + "value.weight")
        return x + out, xx[-1, :]

    def _att_v4(self, x, st, i):
        """att_one / cuda_att_seq (pkg/model.py:1034-1055, 1346-1360)."""
        w = self.w
        b, a = f"blocks.{i}.", f"blocks.{i}.att."
        T, C = x.shape
        xx = _ln(x, w[b + "ln1.weight"], w[b + "ln1.bias"])
        sxx = torch.cat((st[i * 5 + 0].unsqueeze(0), xx[:-1, :]))
        mk, mv, mr = w[a + "time_mix_k"], w[a + "time_mix_v"], w[a + "time_mix_r"]
        kx = xx * mk + sxx * (1 - mk)
        vx = xx * mv + sxx * (1 - mv)
        rx = xx * mr + sxx * (1 - mr)
        r = torch.sigmoid(self._mm(rx, a + "receptance.weight"))
        k = self._mm(kx, a + "key.weight", torch.float32)
        v = self._mm(vx, a + "value.weight", torch.float32)
        y = wkv4_forward(T, C, w[a + "time_decay"], w[a + "time_first"], k, v,
                         st[i * 5 + 1], st[i * 5 + 2], st[i * 5 + 3])
        out = self._mm(r * y.to(x.dtype), a + "output.weight")
        st[i * 5 + 0] = xx[-1, :]
        return x + out

    def _att_v56(self, x, st, i):
        """att_one_v5_1 / att_seq_v5_2 / att_one_v6_0 / att_seq_v6_0
        (pkg/model.py:1157-1181, 1227-1258, 1263-1340).  State in the model layout
        `[H, key index, value index]`."""
        w = self.w
        b, a = f"blocks.{i}.", f"blocks.{i}.att."
        T, C = x.shape
        H = self.args.n_head
        N = C // H
        xx = _ln(x, w[b + "ln1.weight"], w[b + "ln1.bias"])
        sxx = torch.cat((st[i * 3 + 0].unsqueeze(0), xx[:-1, :]))
        if self.version == 6:
            d = sxx - xx
            xxx = xx + d * w[a + "time_maa_x"]
            xxx = torch.tanh((xxx.float() @ w[a + "time_maa_w1"].float()).to(self.atype)).view(T, 5, -1).transpose(0, 1)
            xxx = torch.bmm(xxx.float(), w[a + "time_maa_w2"].float()).to(self.atype).view(5, T, -1)
            mw, mk, mv, mr, mg = xxx.unbind(dim=0)
            wx = xx + d * (w[a + "time_maa_w"] + mw)
            kx = xx + d * (w[a + "time_maa_k"] + mk)
            vx = xx + d * (w[a + "time_maa_v"] + mv)
            rx = xx + d * (w[a + "time_maa_r"] + mr)
            gx = xx + d * (w[a + "time_maa_g"] + mg)
        else:
            mix = lambda n: xx * w[a + f"time_mix_{n}"] + sxx * (1 - w[a + f"time_mix_{n}"])
            kx, vx, rx, gx = mix("k"), mix("v"), mix("r"), mix("g")
        r = self._mm(rx, a + "receptance.weight", torch.float32)
        k = self._mm(kx, a + "key.weight", torch.float32)
        v = self._mm(vx, a + "value.weight", torch.float32)
        g = F.silu(self._mm(gx, a + "gate.weight"))
        u = w[a + "time_first"].float()
        S = st[i * 3 + 1].transpose(-1, -2).contiguous()        # kernel layout [H, v, k]
        if self.version == 6:
            t1 = torch.tanh((wx.float() @ w[a + "time_decay_w1"].float()).to(self.atype))
            dw = (t1.float() @ w[a + "time_decay_w2"].float()).to(self.atype).float()
            ww = w[a + "time_decay"].reshape(1, C) + dw
            ww = torch.exp(-torch.exp(ww.float()))
            out = wkv6_forward(1, T, C, H, S, r, k, v, ww, u)
        else:
            out = wkv5_forward(1, T, C, H, S, r, k, v, w[a + "time_decay"], u)
        st[i * 3 + 1] = S.transpose(-1, -2)
        out = F.group_norm(out.reshape(T, C), num_groups=H, weight=w[a + "ln_x.weight"],
                           bias=w[a + "ln_x.bias"], eps=64e-5)
        out = out.to(dtype=x.dtype) * g
        out = self._mm(out, a + "output.weight")
        st[i * 3 + 0] = xx[-1, :]
        return x + out

    def forward(self, tokens, state, full_output=False):
        """pkg/model.py:1443-1677."""
        w, args = self.w, self.args
        if state is None:
            state = self.zero_state()
        x = w["emb.weight"][tokens].to(self.atype)
        if x.dim() == 1:
            x = x.unsqueeze(0)
        for i in range(args.n_layer):
            if self.version == 4:
                x = self._att_v4(x, state, i)
                x, state[i * 5 + 4] = self._ffn(x, state[i * 5 + 4], i)
            else:
                x = self._att_v56(x, state, i)
                x, state[i * 3 + 2] = self._ffn(x, state[i * 3 + 2], i)
            if self.RESCALE_LAYER > 0 and (i + 1) % self.RESCALE_LAYER == 0:
                x = x / 2
        if not full_output:
            x = x[-1:, :]
        x = _ln(x, w["ln_out.weight"], w["ln_out.bias"])
        x = self._mm(x, "head.weight")
        if not (full_output and len(tokens) > 1):
            x = x[-1]
        return x.float(), state
