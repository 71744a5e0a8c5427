"""`RWKV(model, strategy).forward(tokens, state)` for the 'cuda fp16i8' strategy (and its mixes with 'cuda fp16'),
on sm_100a kernels.

Mirrors the public surface of the reference runtime class (rwkv_pip_package/src/rwkv/
model.py:612-1677): constructor arguments, `forward(tokens, state, full_output)`, the state
list layout (model.py:1448-1471), `.args`, `.version`, `.strategy[i].{device,atype,wtype}`
and the tensor names in `.w`.  What differs, by design:

  * single-device strategies with fp16 activations are implemented: `cuda[:N] fp16i8`, `cuda[:N] fp16` and splits
    by layer count such as `cuda fp16i8 *20 -> cuda fp16` (anything else the reference's strategy grammar accepts
    raises NotImplementedError).  int8 layers run on this library's kernels; plain fp16 layers are library GEMMs plus
    the reference's pointwise ops, and a model that has any takes the sequence path for one-token calls too;
  * the loader packs on the GPU (ops.quantize_weight) and keeps `emb.weight` on the GPU;
  * packed matrices have a row stride padded to 16 bytes (their shape is unchanged);
  * a one-token `forward` is a single CUDA-graph replay of fused kernels; the state tensors
    it returns are persistent buffers that are updated in place by later calls (pass
    `copy.deepcopy(state)` around to keep a snapshot, as the reference's callers do).  Passing
    back a list whose tensors have been reused in between raises instead of computing on the
    wrong state; RWKV_B200_COPY_STATE=1 returns fresh tensors from every call instead.

`model` may also be a checkpoint dict instead of a file name.
"""
from __future__ import annotations

import gc
import os
import re
import types

import torch
import torch.nn.functional as F

from . import _lib, ops, shard
from ._lib import (EPI_MUL_RESIDUAL, EPI_RELU_SQ, EPI_RESIDUAL, EPI_SIGMOID, EPI_SILU, EPI_STORE, EPI_STORE_F32, check,
                   lib)

STRATEGY_REGEX = r"^(?:(?:^|->) *(?:cuda(?::[\d]+)?|cpu|mps|dml) (?:fp(?:16|32)|bf16)(?:i8|i4|i3)?(?: \*[\d]+\+?)? *)+$"
_MATRIX_KEYS = ("key.weight", "value.weight", "receptance.weight", "gate.weight", "output.weight", "head.weight")


def _ptr_array(tensors):
    import ctypes as C
    arr = (C.c_void_p * max(1, len(tensors)))()
    for i, t in enumerate(tensors):
        arr[i] = t.data_ptr()
    return arr


class _StateList(list):
    """The state list a one-token `forward` returns: the runtime's persistent buffers (see the module
    docstring), stamped with the step that wrote them so that a stale list is recognised."""
    owner = None
    step = -1

    def __deepcopy__(self, memo):
        import copy
        return [copy.deepcopy(t, memo) for t in self]      # a snapshot: plain list, own tensors


class RWKV:
    def __init__(self, model, strategy, verbose=True, convert_and_save_and_exit=None, shard_rank=0, shard_world=1):
        """`shard_world` > 1 (an addition to the reference's signature): this process is rank
        `shard_rank` of a torch.distributed group that runs ONE model with every packed matrix
        split by output columns (shard.py); all ranks must make the same forward calls."""
        prxxx = print if verbose else (lambda *a, **k: None)
        self._rank, self._world = int(shard_rank), int(shard_world)
        if not re.match(STRATEGY_REGEX, strategy):
            raise ValueError("Invalid strategy. Please read https://pypi.org/project/rwkv/")
        strategy = ("->".join([x.strip() for x in strategy.split("->")])).replace("->", " -> ")
        # one device, fp16 activations, int8 or fp16 weights per group of layers: 'cuda fp16i8', 'cuda fp16',
        # 'cuda fp16i8 *20 -> cuda fp16', ... (model.py:684-749 without streaming, other devices or dtypes)
        segments = [re.fullmatch(r"(cuda(?::\d+)?) (fp16i8|fp16)(?: \*(\d+))?", x) for x in strategy.split(" -> ")]
        if any(g is None for g in segments) or len({g.group(1) for g in segments}) != 1:
            raise NotImplementedError(
                f"strategy '{strategy}': this runtime implements single-device 'cuda[:N] fp16i8' / 'cuda[:N] fp16' and "
                "splits between the two by layer count ('cuda fp16i8 *K -> cuda fp16')")
        m = segments[0]
        if shard_world > 1 and not (len(segments) == 1 and m.group(2) == "fp16i8"):
            raise NotImplementedError("column sharding is implemented for 'cuda fp16i8'")
        lib()  # fail loudly now if the CUDA library is not built
        self.device = torch.device(m.group(1) if ":" in m.group(1) else "cuda:%d" % torch.cuda.current_device())
        dev = self.device
        self.args = types.SimpleNamespace()
        args = self.args
        args.strategy_string = strategy
        try:
            self.RESCALE_LAYER = int(os.environ["RWKV_RESCALE_LAYER"])
        except Exception:
            self.RESCALE_LAYER = 6      # 'fp16' in strategy (model.py:634)
        self._use_graph = os.environ.get("RWKV_B200_GRAPH", "1") != "0"
        # RWKV_B200_EXACT=1: decode matmuls in fp32 arithmetic instead of 16-bit fixed-point activations
        # (process-wide; about 20 % slower; see rwkv_mm8_one_set_variant in include/rwkv_b200.h)
        if os.environ.get("RWKV_B200_EXACT", "0") == "1":
            lib().rwkv_mm8_one_set_variant(8)
        # RWKV_B200_SEQ_SINGLE=1: the sequence matmuls multiply fp16(x*ry) in one tensor-core pass instead of the exact
        # hi + lo pair (process-wide; about 1e-4 of the output RMS less accurate, below the fp16 rounding of the result;
        # half the tensor work; see rwkv_mm8_seq_set_path in include/rwkv_b200.h)
        if os.environ.get("RWKV_B200_SEQ_SINGLE", "0") == "1":
            lib().rwkv_mm8_seq_set_path(4)

        if isinstance(model, dict):
            args.MODEL_NAME = "<dict>"
            w = dict(model)
        else:
            args.MODEL_NAME = model.strip()
            if not args.MODEL_NAME.endswith(".pth"):
                args.MODEL_NAME += ".pth"
            prxxx(f"Loading {args.MODEL_NAME} ...")
            w = torch.load(args.MODEL_NAME, map_location="cpu")
        self.w = w

        with torch.no_grad(), torch.cuda.device(dev):
            already = False
            if "_strategy" in w:                                     # model.py:646-656
                already = True
                assert convert_and_save_and_exit is None
                prxxx(f"Converted model: strategy {w['_strategy']}, version {w['_version']}\n")
                assert w["_strategy"] == args.strategy_string
                assert float(w["_version"]) >= 0.7
                assert w["_rescale_layer"] == self.RESCALE_LAYER
                del w["_strategy"], w["_version"], w["_rescale_layer"]

            args.n_embd = w["emb.weight"].shape[1]
            args.n_att = w["blocks.0.att.key.weight"].shape[0]
            args.n_ffn = w["blocks.0.ffn.key.weight"].shape[0]
            if already:   # converted matrices are stored [in, out]
                args.n_att = w["blocks.0.att.key.weight"].shape[1]
                args.n_ffn = w["blocks.0.ffn.key.weight"].shape[1]
            args.n_layer = 0
            self.version = 4
            for x in list(w.keys()):                                 # model.py:662-679
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
            prxxx(f"Model detected: v{self.version:.1f}")
            if self.version not in (4, 5.2, 6):
                raise NotImplementedError(f"RWKV v{self.version}: this runtime implements v4, v5.2 and v6")

            # layers per strategy segment, as the reference deals them (model.py:684-737; n_layer + 1 "layers": the
            # last one holds ln_out and the head)
            plan = [0] * len(segments)
            to_allocate, allocated, free_slots = args.n_layer + 1, 0, 0
            for i, g in enumerate(segments):
                if g.group(3) is not None:
                    plan[i] = int(g.group(3))
                    allocated += plan[i]
                    if allocated >= to_allocate:
                        plan[i] += to_allocate - allocated
                        break
                else:
                    free_slots += 1
            if free_slots > 0 and to_allocate > allocated:
                for i in range(len(segments)):
                    if plan[i] == 0:
                        plan[i] = (to_allocate - allocated) // free_slots
                        allocated += plan[i]
                        free_slots -= 1
            if to_allocate > allocated:
                plan[-1] += to_allocate - allocated
            for i in range(1, len(plan)):
                plan[i] += plan[i - 1]
            self.strategy = []
            for n in range(args.n_layer + 1):
                g = segments[next(i for i in range(len(segments)) if n < plan[i])]
                self.strategy.append(types.SimpleNamespace(
                    device=str(dev) if ":" in m.group(1) else "cuda", atype=torch.float16,
                    wtype=torch.uint8 if g.group(2) == "fp16i8" else torch.float16, stream=False))

            if not already:                                          # model.py:754-760
                emb = w["emb.weight"].to(dev)
                w["emb.weight"] = F.layer_norm(emb.float(), (args.n_embd,),
                                               weight=w["blocks.0.ln0.weight"].to(dev).float(),
                                               bias=w["blocks.0.ln0.bias"].to(dev).float())
                del w["blocks.0.ln0.weight"], w["blocks.0.ln0.bias"], emb

            real_time_first = any(".time_faaaa" in k for k in w)
            args.time_state = any(".time_state" in k for k in w)
            if real_time_first:
                w = {k.replace(".time_faaaa", ".time_first"): v for k, v in w.items()}
                self.w = w

            for x in list(w.keys()):                                 # model.py:774-869
                if x.endswith(("_mx", "_rx", "_my", "_ry")):
                    w[x] = w[x].to(dev).contiguous()
                    continue
                layer_id = int(x.split(".")[1]) if ("blocks." in x) else 0
                if ("ln_out." in x) or ("head." in x):
                    layer_id = args.n_layer
                t = w[x].to(dev)
                t.requires_grad = False
                if already:
                    if t.dtype == torch.uint8:
                        t = self._repad(t)
                    w[x] = t.contiguous() if t.dtype != torch.uint8 else t
                    continue
                scale = 1.0
                if self.RESCALE_LAYER > 0 and ("att.output.weight" in x or "ffn.value.weight" in x):
                    scale = 1.0 / (2 ** int(layer_id // self.RESCALE_LAYER))
                if ".time_" in x:
                    t = t.squeeze()
                is_matrix = any(s in x for s in _MATRIX_KEYS)
                if is_matrix:
                    t = t.t()
                if ".time_decay" in x and "_w" not in x:
                    if self.version == 4:
                        t = -torch.exp(t.float())
                    elif self.version == 5.2:
                        t = torch.exp(-torch.exp(t.float())).reshape(args.n_head, -1, 1)
                    else:
                        t = t.float().reshape(args.n_head, -1, 1)
                elif ".time_first" in x:
                    if self.version == 4:
                        t = t.float()
                    else:
                        t = t.float().reshape(-1, 1, 1) if real_time_first else torch.exp(t.float()).reshape(-1, 1, 1)
                        t = t.reshape(args.n_head, -1, 1)
                elif ".ln_x" in x:
                    t = t.float()
                elif len(t.shape) == 2 and "emb" not in x and "_w1" not in x and "_w2" not in x and \
                        self.strategy[layer_id].wtype == torch.uint8:
                    q, mx, rx, my, ry = ops.quantize_weight(t, torch.float16, scale)
                    t = q
                    w[x + "_mx"], w[x + "_rx"], w[x + "_my"], w[x + "_ry"] = mx, rx, my, ry
                else:
                    if scale != 1.0:
                        t = t * scale
                    t = t.to(dtype=torch.float16)
                w[x] = t if t.dtype == torch.uint8 else t.contiguous()
                if "ffn.value.weight" in x:
                    gc.collect()

            if convert_and_save_and_exit:                             # model.py:894-903
                out = self.export_converted()
                if not convert_and_save_and_exit.endswith(".pth"):
                    convert_and_save_and_exit += ".pth"
                prxxx(f"Saving to {convert_and_save_and_exit}...")
                torch.save(out, convert_and_save_and_exit)
                prxxx("Converted and saved. Now this will exit.")
                raise SystemExit(0)

            if self.version != 4:
                args.n_head = w["blocks.0.att.time_first"].shape[0]
            # the fused one-token path and the batched path are built for int8 matrices throughout; a model with plain
            # fp16 layers runs every call through the sequence path (library GEMMs for those layers)
            self._all_i8 = all(w[k].dtype == torch.uint8 for k in w
                               if torch.is_tensor(w[k]) and any(sk in k for sk in _MATRIX_KEYS) and k.endswith(".weight"))
            self._full_m = {}
            if self._world > 1:
                if self.version != 4:
                    raise NotImplementedError("column sharding is implemented for RWKV-4")
                for x in [k for k, t in w.items() if torch.is_tensor(t) and t.dtype == torch.uint8]:
                    self._full_m[x] = w[x].shape[1]
                    if shard.column_range(w[x].shape[1], self._world, self._world - 1)[0] >= w[x].shape[1]:
                        raise ValueError(f"{x}: {w[x].shape[1]} columns are too few for {self._world} ranks")
                    w[x], w[x + "_mx"], w[x + "_rx"] = shard.column_shard(w[x], w[x + "_mx"], w[x + "_rx"],
                                                                         self._world, self._rank)
                # NCCL all-gathers between the launches: direct launches only (capturing them into a CUDA
                # graph did not return on the B200 pool; it is not attempted).  The peer-store exchange
                # has no collective call and is captured like the single-GPU step.
                self._use_graph = self._use_graph and os.environ.get("RWKV_B200_SHARD_EXCHANGE", "peer") == "peer" \
                    and torch.distributed.get_backend() == "nccl"
                torch.cuda.empty_cache()
            self._init_buffers()
        gc.collect()
        torch.cuda.empty_cache()

    # -----------------------------------------------------------------------------------
    def export_converted(self, strategy_string=None):
        """The loaded weights as the dict the reference's loader saves for
        `convert_and_save_and_exit` (model.py:894-903: every tensor already transposed / packed,
        plus `_strategy`, `_rescale_layer`, `_version`), on the CPU, row padding dropped."""
        if self._world > 1:
            raise NotImplementedError("export_converted: column-sharded models hold only their slices")
        out = {k: (v.contiguous().cpu() if torch.is_tensor(v) else v) for k, v in self.w.items()}
        out["_strategy"] = strategy_string or self.args.strategy_string
        out["_rescale_layer"] = self.RESCALE_LAYER
        out["_version"] = "0.7"
        return out

    @staticmethod
    def _repad(q):
        """Give a contiguous packed matrix the 16-byte row stride the fast kernels want."""
        N, M = q.shape
        P = ops.padded_stride(M)
        if q.stride(0) == P and q.stride(1) == 1:
            return q
        full = torch.zeros((N, P), dtype=torch.uint8, device=q.device)
        full[:, :M].copy_(q)
        return full[:, :M]

    def _init_buffers(self):
        a, dev = self.args, self.device
        D, Fn = a.n_embd, a.n_ffn
        h = lambda n: torch.zeros(n, dtype=torch.float16, device=dev)
        self._b = types.SimpleNamespace(
            x=h(D), m0=h(D), m1=h(D), m2=h(D), m3=h(D), m4=h(D), r=h(a.n_att), k=h(a.n_att), v=h(a.n_att),
            g=h(a.n_att), att=h(a.n_att), fk=h(Fn), fr=h(D), xln=h(D), dd=h(D),
            wdec=torch.zeros(a.n_att, dtype=torch.float32, device=dev),
            logits=torch.zeros(self._full_m.get("head.weight", self.w["head.weight"].shape[1]), dtype=torch.float32,
                               device=dev),
            tok=torch.zeros(1, dtype=torch.int64, device=dev))
        # Column-sharded decode: the gathered activation buffers live in a region that the other
        # ranks have mapped, and the matmul kernels store their column slices into every rank's copy
        # (RWKV_B200_SHARD_EXCHANGE=nccl keeps the all-gather calls between the launches instead).
        self._peer = None
        if self._world > 1 and os.environ.get("RWKV_B200_SHARD_EXCHANGE", "peer") == "peer" and \
                torch.distributed.get_backend() == "nccl":
            bb = self._b
            fields = [("x", torch.float16, D), ("r", torch.float16, a.n_att), ("k", torch.float16, a.n_att),
                      ("v", torch.float16, a.n_att), ("fr", torch.float16, D), ("fk", torch.float16, Fn),
                      ("logits", torch.float32, bb.logits.numel())]
            self._peer = shard.PeerRegion(fields, dev, self._world, self._rank)
            for name, _, _ in fields:
                setattr(bb, name, self._peer.view(name))
        # ring of pinned H2D staging slots for host token ids; a slot is reused only after the copy that read
        # it has completed (callers may enqueue many steps without ever synchronising)
        self._tok_host = torch.zeros(64, dtype=torch.int64).pin_memory()
        self._tok_events = [None] * self._tok_host.numel()
        self._tok_slot = 0
        self._ws = torch.zeros(96 << 20, dtype=torch.uint8, device=dev)
        # Decode state lives in two persistent sets: a step reads set `_cur` and writes the other
        # one (no kernel ever overwrites a vector that another CTA of the same launch still
        # reads), then the roles swap.  One captured graph per direction.
        self._st = None
        self._cur = 0
        self._steps = 0
        # RWKV_B200_COPY_STATE=1: every one-token forward returns fresh state tensors (as the reference does) instead
        # of the persistent buffers; ~160 small copies per token at the 7B shape
        self._copy_state = os.environ.get("RWKV_B200_COPY_STATE", "0") == "1"
        self._graphs = [None, None]
        self._locbuf = {}
        # RWKV_B200_STREAM=1 (or set_decode_path("stream")): RWKV-4 decode as ONE persistent kernel per token over
        # a re-tiled copy of the packed matrices (csrc/mm8_stream.cu) instead of a launch per group of matmuls.
        # Costs a second copy of the codes in HBM (the row-major one still serves prefill); measured slower than
        # the launches at the 7B shape, so it is not the default.
        self._use_stream = (self.version == 4 and self._world == 1 and
                            os.environ.get("RWKV_B200_STREAM", "0") == "1")
        self._stream = None
        self._mm = {}
        self._mm_pad = {}
        self._fork_streams = []
        self._batch_fork = os.environ.get("RWKV_B200_BATCH_FORK", "1") != "0"
        self._v6_decay_fork = os.environ.get("RWKV_B200_V6_DECAY_FORK", "1") != "0"
        self._tile_cache = {}
        self._batch_graphs = {}
        # a matrix with more than 16384 in-features needs the decode kernel's second build: ask for it on every launch
        self._gemv_flags = _lib.MM8_WIDE_BUILD if max(a.n_ffn, a.n_att, a.n_embd) > 16384 else 0

    def _scales(self, name):
        e = self._mm.get(name)
        if e is None:
            w = self.w
            e = (w[name], w[name + "_mx"], w[name + "_rx"], w[name + "_my"], w[name + "_ry"])
            self._mm[name] = e
        return e

    def _problem(self, x, name, y, epi, aux=None, aux2=None, out_scale=1.0):
        wq, mx, rx, my, ry = self._scales(name)
        return ops.make_problem(x, wq, mx, rx, my, ry, y, epi, aux, aux2, out_scale)

    def _gemv(self, problems, exchange=None):
        ops.mm8_one_batch(problems, torch.float16, self.device, self._ws, exchange, self._gemv_flags)

    def _ln_mix(self, T, x, sx, ln_w, ln_b, mode, mixes, outs, xx_out=None, new_state=None, mix_stride=0, rows=False):
        """`rows`: every row of x is a sequence of its own (batched decode) and sx holds their states [T, D]."""
        D = self.args.n_embd
        check(lib().rwkv_ln_mix_rows(T, D, x.data_ptr(), x.stride(0) if x.dim() == 2 else D,
                                sx.data_ptr() if sx is not None else None, (sx.stride(0) if rows and sx is not None else 0),
                                ln_w.data_ptr(), ln_b.data_ptr(),
                                mode, len(mixes), _ptr_array(mixes), mix_stride, _ptr_array(outs),
                                outs[0].stride(0) if (outs and outs[0].dim() == 2) else D,
                                xx_out.data_ptr() if xx_out is not None else None,
                                (xx_out.stride(0) if xx_out.dim() == 2 else D) if xx_out is not None else 0,
                                new_state.data_ptr() if new_state is not None else None,
                                torch.cuda.current_stream(self.device).cuda_stream), "ln_mix")

    # -----------------------------------------------------------------------------------
    def _zero_state(self):
        """model.py:1448-1471.  The entries are rows of two zero-filled allocations (one per dtype, rows padded to 256
        bytes) instead of five tensors per layer: three fill launches for the whole list."""
        a, dev = self.args, self.device
        L = a.n_layer
        pad = lambda n, per: (n + per - 1) // per * per
        h = torch.zeros((L, 2, pad(a.n_embd, 128)), dtype=torch.float16, device=dev)
        st = []
        if self.version == 4:
            f = torch.zeros((L, 3, pad(a.n_att, 64)), dtype=torch.float32, device=dev)
            f[:, 2].fill_(-1e30)
            for i in range(L):
                st += [h[i, 0, :a.n_embd], f[i, 0, :a.n_att], f[i, 1, :a.n_att], f[i, 2, :a.n_att], h[i, 1, :a.n_embd]]
            return st
        N = a.n_att // a.n_head
        S = None if a.time_state else torch.zeros((L, a.n_head, N, N), dtype=torch.float32, device=dev)
        for i in range(L):
            if a.time_state:
                s = self.w[f"blocks.{i}.att.time_state"].transpose(1, 2).to(dtype=torch.float, device=dev).contiguous()
            else:
                s = S[i]
            st += [h[i, 0, :a.n_embd], s, h[i, 1, :a.n_embd]]
        return st

    def forward(self, tokens, state, full_output=False):
        with torch.no_grad(), torch.cuda.device(self.device):
            if state is None:
                state = self._zero_state()
            if torch.is_tensor(tokens):
                if tokens.is_cuda and tokens.numel() == 1 and self._all_i8:
                    return self._forward_one(tokens, state)      # token id stays on the device
                tokens = tokens.tolist()
            if len(tokens) == 1 and self._all_i8:
                return self._forward_one(int(tokens[0]), state)
            return self._forward_seq([int(t) for t in tokens], state, full_output)

    # ----- one token ---------------------------------------------------------------------
    @property
    def _gstate(self):
        return self._st[self._cur]

    def _bind_state(self, state):
        """Make `state` the tensors the next decode step reads."""
        if self._st is None:
            self._st = [[s.contiguous().clone() for s in state], [s.contiguous().clone() for s in state]]
            self._st_ids = [tuple(map(id, lst)) for lst in self._st]      # identity check of a whole list at C speed
            self._cur = 0
            return
        g = self._st[self._cur]
        if tuple(map(id, state)) == self._st_ids[self._cur]:
            if isinstance(state, _StateList) and state.owner is self and state.step != self._steps:
                self._stale(state)
            return
        other = self._st[1 - self._cur]
        if len(other) == len(state) and len(state) > 0 and state[0] is other[0]:
            self._stale(state)
        torch._foreach_copy_(g, [s for s in state])

    def _stale(self, state):
        raise _lib.RwkvB200Error(
            "this state list was returned by an earlier one-token forward() of this model and its tensors have been "
            "reused since (they are the runtime's persistent buffers): keep snapshots with copy.deepcopy(state), or set "
            "RWKV_B200_COPY_STATE=1 to get fresh tensors from every call")

    def _forward_one(self, token, state):
        self._bind_state(state)
        if torch.is_tensor(token):
            self._b.tok.copy_(token.reshape(1))
        else:
            V = self.w["emb.weight"].shape[0]
            if not -V <= token < V:             # as indexing the embedding matrix on the host would (model.py:1475)
                raise IndexError(f"token id {token} is out of range for a vocabulary of {V}")
            token %= V
            slot = self._tok_slot = (self._tok_slot + 1) % self._tok_host.numel()
            if self._tok_events[slot] is not None:
                self._tok_events[slot].synchronize()
            else:
                self._tok_events[slot] = torch.cuda.Event()
            self._tok_host[slot] = token
            self._b.tok.copy_(self._tok_host[slot:slot + 1], non_blocking=True)
            self._tok_events[slot].record(torch.cuda.current_stream(self.device))
        if self.version == 4:
            step = (self._step_one_v4_peer if self._peer is not None else self._step_one_v4_sharded) \
                if self._world > 1 else self._step_one_v4
        else:
            step = self._step_one_v56
        cur = self._cur
        if not self._use_graph:
            step(cur)
        elif self._graphs[cur] is None:
            # one eager step on a copy of the state warms every kernel up before the capture
            saved = [s.clone() for s in self._st[cur]]
            step(cur)
            torch._foreach_copy_(self._st[cur], saved)
            torch.cuda.synchronize(self.device)
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    step(cur)
                self._graphs[cur] = graph
            except Exception as e:       # e.g. a launch kind the capture does not accept
                if os.environ.get("RWKV_B200_VERBOSE"):
                    print(f"[rwkv_b200] CUDA graph capture failed ({e}); decoding with direct launches")
                torch.cuda.synchronize(self.device)
                self._use_graph = False
            torch._foreach_copy_(self._st[cur], saved)
            if self._use_graph:
                graph.replay()
            else:
                step(cur)
        else:
            self._graphs[cur].replay()
        self._cur = 1 - cur
        self._steps += 1
        if self._copy_state:
            return self._b.logits.clone(), [t.clone() for t in self._st[self._cur]]
        out = _StateList(self._st[self._cur])
        out.owner, out.step = self, self._steps
        return self._b.logits.clone(), out

    def _launches_v4(self, cur):
        """The GEMV launches of one RWKV-4 token, in order: four per layer plus the head, with
        everything pointwise fused into their prologues and epilogues (att_one / ffn_one,
        model.py:984-992, 1034-1055).  Reads state set `cur`, writes the other one."""
        b, w, a = self._b, self.w, self.args
        sin, sout = self._st[cur], self._st[1 - cur]
        P, ln, wk = self._problem, ops.with_ln_mix, ops.with_wkv4
        launches = []
        for i in range(a.n_layer):
            bb, att, ffn = f"blocks.{i}.", f"blocks.{i}.att.", f"blocks.{i}.ffn."
            ln1 = (w[bb + "ln1.weight"], w[bb + "ln1.bias"])
            ln2 = (w[bb + "ln2.weight"], w[bb + "ln2.bias"])
            s = i * 5
            launches.append([
                ln(P(b.x, att + "receptance.weight", b.r, EPI_SIGMOID), *ln1, 0, sin[s], w[att + "time_mix_r"], sout[s]),
                ln(P(b.x, att + "key.weight", b.k, EPI_STORE), *ln1, 0, sin[s], w[att + "time_mix_k"]),
                ln(P(b.x, att + "value.weight", b.v, EPI_STORE), *ln1, 0, sin[s], w[att + "time_mix_v"])])
            launches.append([wk(P(b.r, att + "output.weight", b.x, EPI_RESIDUAL, aux=b.x), b.k, b.v,
                                w[att + "time_decay"], w[att + "time_first"], sin[s + 1:s + 4], sout[s + 1:s + 4])])
            launches.append([
                ln(P(b.x, ffn + "receptance.weight", b.fr, EPI_SIGMOID), *ln2, 0, sin[s + 4], w[ffn + "time_mix_r"], sout[s + 4]),
                ln(P(b.x, ffn + "key.weight", b.fk, EPI_RELU_SQ), *ln2, 0, sin[s + 4], w[ffn + "time_mix_k"])])
            scale = 0.5 if (self.RESCALE_LAYER > 0 and (i + 1) % self.RESCALE_LAYER == 0) else 1.0
            launches.append([P(b.fk, ffn + "value.weight", b.x, EPI_MUL_RESIDUAL, aux=b.x, aux2=b.fr, out_scale=scale)])
        launches.append([ln(P(b.x, "head.weight", b.logits, EPI_STORE_F32), w["ln_out.weight"], w["ln_out.bias"], 2)])
        return launches

    def _embed_row(self):
        """x = emb[token] of a decode step, by a kernel of this library (the launch after it starts under it)."""
        e = self.w["emb.weight"]
        check(lib().rwkv_embed_row(e.shape[1], e.shape[0], e.data_ptr(), e.stride(0), self._b.tok.data_ptr(), self._b.x.data_ptr(),
                                   torch.cuda.current_stream(self.device).cuda_stream), "embed_row")

    def _step_one_v4_sharded(self, cur):
        """One RWKV-4 token with every matmul split by output columns over the ranks: the same
        launches as `_launches_v4` on this rank's column slices, an all-gather of the fp16
        slices after each (r, k, v; x; ffn r, k; x; logits) -- four gathers per layer."""
        b, w, a = self._b, self.w, self.args
        G, R = self._world, self._rank
        self._embed_row()
        sin, sout = self._st[cur], self._st[1 - cur]
        P, ln, wk = self._problem, ops.with_ln_mix, ops.with_wkv4
        D, Fn = a.n_embd, a.n_ffn

        def loc(key, M, dtype=torch.float16):
            t = self._locbuf.get(key)
            if t is None:
                t = self._locbuf[key] = torch.zeros(shard.shard_width(M, G), dtype=dtype, device=self.device)
            return t

        def gather(pairs):
            for full, local in pairs:
                if local.numel() * G == full.numel():        # even split: gather straight into place
                    torch.distributed.all_gather_into_tensor(full, local)
                else:
                    full.copy_(shard.gather_columns(local, full.numel(), G))

        def run(problems):
            problems = [p for p in problems if p.M > 0]
            if problems:
                self._gemv(problems)

        lo_d, hi_d = shard.column_range(D, G, R)
        for i in range(a.n_layer):
            bb, att, ffn = f"blocks.{i}.", f"blocks.{i}.att.", f"blocks.{i}.ffn."
            ln1 = (w[bb + "ln1.weight"], w[bb + "ln1.bias"])
            ln2 = (w[bb + "ln2.weight"], w[bb + "ln2.bias"])
            s = i * 5
            lr, lk, lv, lx = loc("r", a.n_att), loc("k", a.n_att), loc("v", a.n_att), loc("x", D)
            run([ln(P(b.x, att + "receptance.weight", lr, EPI_SIGMOID), *ln1, 0, sin[s], w[att + "time_mix_r"], sout[s]),
                 ln(P(b.x, att + "key.weight", lk, EPI_STORE), *ln1, 0, sin[s], w[att + "time_mix_k"]),
                 ln(P(b.x, att + "value.weight", lv, EPI_STORE), *ln1, 0, sin[s], w[att + "time_mix_v"])])
            gather([(b.r, lr), (b.k, lk), (b.v, lv)])
            run([wk(P(b.r, att + "output.weight", lx, EPI_RESIDUAL, aux=b.x[lo_d:]), b.k, b.v,
                    w[att + "time_decay"], w[att + "time_first"], sin[s + 1:s + 4], sout[s + 1:s + 4])])
            gather([(b.x, lx)])
            lfr, lfk = loc("fr", D), loc("fk", Fn)
            run([ln(P(b.x, ffn + "receptance.weight", lfr, EPI_SIGMOID), *ln2, 0, sin[s + 4], w[ffn + "time_mix_r"], sout[s + 4]),
                 ln(P(b.x, ffn + "key.weight", lfk, EPI_RELU_SQ), *ln2, 0, sin[s + 4], w[ffn + "time_mix_k"])])
            gather([(b.fr, lfr), (b.fk, lfk)])
            scale = 0.5 if (self.RESCALE_LAYER > 0 and (i + 1) % self.RESCALE_LAYER == 0) else 1.0
            run([P(b.fk, ffn + "value.weight", lx, EPI_MUL_RESIDUAL, aux=b.x[lo_d:], aux2=b.fr[lo_d:], out_scale=scale)])
            gather([(b.x, lx)])
        ll = loc("logits", b.logits.numel(), torch.float32)
        run([ln(P(b.x, "head.weight", ll, EPI_STORE_F32), w["ln_out.weight"], w["ln_out.bias"], 2)])
        gather([(b.logits, ll)])

    def _step_one_v4_peer(self, cur):
        """One RWKV-4 token with every matmul split by output columns over the ranks and NO
        collective call: each launch stores its column slice into every rank's copy of the
        activation buffer (peer stores over NVLink from the epilogue) and the next launch waits on
        per-rank arrival words (csrc/mm8_cluster.cuh, Exchange).  Same four launches per layer as
        `_launches_v4`; every rank keeps the full recurrent state."""
        b, w, a, pr = self._b, self.w, self.args, self._peer
        G, R = self._world, self._rank
        stream = torch.cuda.current_stream(self.device).cuda_stream
        pr.begin_token(4 * a.n_layer + 1, stream)
        self._embed_row()
        sin, sout = self._st[cur], self._st[1 - cur]
        P, ln, wk = self._problem, ops.with_ln_mix, ops.with_wkv4
        D, Fn = a.n_embd, a.n_ffn
        ld, hd = shard.column_range(D, G, R)
        la, ha = shard.column_range(a.n_att, G, R)
        lf, hf = shard.column_range(Fn, G, R)
        lv, hv = shard.column_range(b.logits.numel(), G, R)
        for i in range(a.n_layer):
            bb, att, ffn = f"blocks.{i}.", f"blocks.{i}.att.", f"blocks.{i}.ffn."
            ln1 = (w[bb + "ln1.weight"], w[bb + "ln1.bias"])
            ln2 = (w[bb + "ln2.weight"], w[bb + "ln2.bias"])
            s = i * 5
            self._gemv([ln(P(b.x, att + "receptance.weight", b.r[la:ha], EPI_SIGMOID), *ln1, 0, sin[s], w[att + "time_mix_r"], sout[s]),
                        ln(P(b.x, att + "key.weight", b.k[la:ha], EPI_STORE), *ln1, 0, sin[s], w[att + "time_mix_k"]),
                        ln(P(b.x, att + "value.weight", b.v[la:ha], EPI_STORE), *ln1, 0, sin[s], w[att + "time_mix_v"])],
                       pr.exchange([("r", la), ("k", la), ("v", la)], wait=i > 0))
            self._gemv([wk(P(b.r, att + "output.weight", b.x[ld:hd], EPI_RESIDUAL, aux=b.x[ld:hd]), b.k, b.v,
                           w[att + "time_decay"], w[att + "time_first"], sin[s + 1:s + 4], sout[s + 1:s + 4])],
                       pr.exchange([("x", ld)], wait=True))
            self._gemv([ln(P(b.x, ffn + "receptance.weight", b.fr[ld:hd], EPI_SIGMOID), *ln2, 0, sin[s + 4], w[ffn + "time_mix_r"], sout[s + 4]),
                        ln(P(b.x, ffn + "key.weight", b.fk[lf:hf], EPI_RELU_SQ), *ln2, 0, sin[s + 4], w[ffn + "time_mix_k"])],
                       pr.exchange([("fr", ld), ("fk", lf)], wait=True))
            scale = 0.5 if (self.RESCALE_LAYER > 0 and (i + 1) % self.RESCALE_LAYER == 0) else 1.0
            self._gemv([P(b.fk, ffn + "value.weight", b.x[ld:hd], EPI_MUL_RESIDUAL, aux=b.x[ld:hd], aux2=b.fr[ld:hd],
                          out_scale=scale)], pr.exchange([("x", ld)], wait=True))
        self._gemv([ln(P(b.x, "head.weight", b.logits[lv:hv], EPI_STORE_F32), w["ln_out.weight"], w["ln_out.bias"], 2)],
                   pr.exchange([("logits", lv)], wait=True))
        pr.end_token(stream)                     # every rank's logits slice is here

    def peer_error(self):
        """1 if a wait on another rank's arrival word gave up since the last call (results were
        then undefined); synchronises the device."""
        return self._peer.take_error() if self._peer is not None else 0

    def _build_stream(self):
        """Re-tile the packed matrices for the persistent decode kernel and lay out its phase tables (one per
        state direction).  Returns False when a matrix does not meet that kernel's limits."""
        import ctypes as C
        L = lib()
        G = L.rwkv_mm8_stream_ctas()
        tables = []
        wstream = None
        for cur in (0, 1):
            launches = self._launches_v4(cur)
            flat = [p for probs in launches for p in probs]
            arr = (_lib.Mm8Problem * len(flat))(*flat)
            counts = (C.c_int32 * len(launches))(*[len(p) for p in launches])
            if wstream is None:
                nbytes = L.rwkv_mm8_stream_weight_bytes(arr, len(flat), G)
                wstream = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
                rc = L.rwkv_mm8_stream_pack(arr, len(flat), G, wstream.data_ptr(), nbytes,
                                            torch.cuda.current_stream(self.device).cuda_stream)
                if rc == _lib.ERR_UNSUPPORTED:
                    return False
                check(rc, "mm8_stream_pack")
            tbytes = L.rwkv_mm8_stream_table_bytes(len(launches))
            host = torch.zeros(tbytes, dtype=torch.uint8)
            rc = L.rwkv_mm8_stream_plan(arr, counts, len(launches), _lib.F16, G, host.data_ptr(), tbytes)
            if rc == _lib.ERR_UNSUPPORTED:
                return False
            check(rc, "mm8_stream_plan")
            tables.append((host, host.to(self.device)))
        sync = torch.zeros(16, dtype=torch.int32, device=self.device)
        self._stream = types.SimpleNamespace(wstream=wstream, tables=tables, sync=sync, trace=None, n_phases=len(launches))
        return True

    def decode_path(self):
        """Which kernels a one-token forward runs: 'stream' (RWKV-4: one persistent kernel) or 'launch' (a launch
        per group of matmuls)."""
        return "stream" if (self.version == 4 and self._world == 1 and self._use_stream) else "launch"

    def set_decode_path(self, path):
        """Switch RWKV-4 decode between 'stream' and 'launch'; captured graphs are dropped."""
        if path not in ("stream", "launch"):
            raise ValueError(path)
        self._use_stream = path == "stream" and self.version == 4 and self._world == 1
        self._graphs = [None, None]

    def launches_per_token(self):
        """Kernel launches of this library per decoded token (the embedding gather is a torch kernel)."""
        L = self.args.n_layer
        if self.version != 4:
            return L * (5 if self.version == 5.2 else 6) + 1
        return 1 if self.decode_path() == "stream" else 4 * L + 1

    def stream_error(self):
        """1 if a wait inside the persistent decode kernel gave up since the last call (the step's results were
        then undefined); synchronises the current stream."""
        import ctypes as C
        if self._stream is None:
            return 0
        e = C.c_int(0)
        check(lib().rwkv_mm8_stream_take_error(self._stream.sync.data_ptr(), torch.cuda.current_stream(self.device).cuda_stream,
                                               C.byref(e)), "mm8_stream_take_error")
        return e.value

    def _step_one_v4(self, cur):
        b, w = self._b, self.w
        if self._use_stream and self._stream is None and not self._build_stream():
            self._use_stream = False
        self._embed_row()
        if self._use_stream:
            st = self._stream
            host, dev = st.tables[cur]
            check(lib().rwkv_mm8_stream_run(dev.data_ptr(), host.data_ptr(), st.wstream.data_ptr(), st.sync.data_ptr(),
                                            st.trace.data_ptr() if st.trace is not None else None,
                                            torch.cuda.current_stream(self.device).cuda_stream), "mm8_stream_run")
        else:
            if not hasattr(self, "_launch_cache"):
                self._launch_cache = [self._launches_v4(0), self._launches_v4(1)]   # fixed buffers: built once
            for probs in self._launch_cache[cur]:
                self._gemv(probs)

    def _plan_v56(self, cur):
        """The launches of one RWKV-5.2 / RWKV-6 token (att_one_v5_1 / att_one_v6_0, ffn_one / ffn_one_v6,
        model.py:984-1016, 1157-1181, 1263-1298) as a list of zero-argument callables over fixed buffers;
        reads state set `cur`, writes the other one.  Nothing in it allocates, so it can be captured."""
        import ctypes as C
        b, w, a, L = self._b, self.w, self.args, lib()
        sin, sout = self._st[cur], self._st[1 - cur]
        P, ln = self._problem, ops.with_ln_mix
        D, H = a.n_embd, a.n_head
        N = a.n_att // H
        v6 = self.version == 6
        dev = self.device
        stream = lambda: torch.cuda.current_stream(dev).cuda_stream
        ptrs = lambda ts: (C.c_void_p * len(ts))(*[t.data_ptr() for t in ts])
        if v6 and not hasattr(self, "_lora_ws"):
            rank = max(w["blocks.0.att.time_maa_w1"].shape[1], w["blocks.0.att.time_decay_w1"].shape[1])
            self._lora_ws = torch.zeros(max(16, L.rwkv_v6_scratch_bytes(D, rank)), dtype=torch.uint8, device=dev)
        plan, keep = [], []
        gemv = lambda probs: plan.append(lambda probs=probs: self._gemv(probs))
        for i in range(a.n_layer):
            bb, att, ffn = f"blocks.{i}.", f"blocks.{i}.att.", f"blocks.{i}.ffn."
            ln1 = (w[bb + "ln1.weight"], w[bb + "ln1.bias"])
            ln2 = (w[bb + "ln2.weight"], w[bb + "ln2.bias"])
            s = i * 3
            u = w[att + "time_first"].reshape(-1)
            if v6:
                Lm = w[att + "time_maa_w1"].shape[1] // 5
                Ld = w[att + "time_decay_w1"].shape[1]
                maa5 = ptrs([w[att + "time_maa_" + n] for n in "wkvrg"])
                out5 = ptrs([b.m0, b.m1, b.m2, b.m3, b.m4])
                keep += [maa5, out5]
                ws = self._lora_ws
                fused = (5 * Lm) % 8 == 0 and Ld % 8 == 0 and D <= 8192
                split = fused and self._v6_decay_fork
                run_decay = lambda att=att, Ld=Ld, ws=ws: check(
                    L.rwkv_v6_decay(D, Ld, b.m0.data_ptr(), w[att + "time_decay_w1"].data_ptr(),
                                    w[att + "time_decay_w2"].data_ptr(), w[att + "time_decay"].data_ptr(), ws.data_ptr(),
                                    ws.numel(), b.wdec.data_ptr(), stream()), "v6_decay")
                if fused:
                    # token shift (and, unless it runs beside the matmuls, the decay) as one single-cluster launch
                    dw = [None] * 3 if split else [w[att + "time_decay_" + n].data_ptr() for n in ("w1", "w2")] + [w[att + "time_decay"].data_ptr()]
                    plan.append(lambda s=s, att=att, ln1=ln1, Lm=Lm, Ld=Ld, maa5=maa5, out5=out5, dw=dw, split=split: check(
                        L.rwkv_v6_att_pre(D, Lm, Ld, b.x.data_ptr(), sin[s].data_ptr(), sout[s].data_ptr(), ln1[0].data_ptr(),
                                          ln1[1].data_ptr(), w[att + "time_maa_x"].data_ptr(), maa5,
                                          w[att + "time_maa_w1"].data_ptr(), w[att + "time_maa_w2"].data_ptr(),
                                          dw[0], dw[1], dw[2], b.xln.data_ptr(), b.dd.data_ptr(), out5,
                                          None if split else b.wdec.data_ptr(), stream()), "v6_att_pre"))
                else:
                    plan.append(lambda s=s, att=att, ln1=ln1, Lm=Lm, maa5=maa5, out5=out5, ws=ws: check(
                        L.rwkv_v6_token_shift(D, Lm, b.x.data_ptr(), sin[s].data_ptr(), sout[s].data_ptr(), ln1[0].data_ptr(),
                                              ln1[1].data_ptr(), w[att + "time_maa_x"].data_ptr(), maa5,
                                              w[att + "time_maa_w1"].data_ptr(), w[att + "time_maa_w2"].data_ptr(),
                                              ws.data_ptr(), ws.numel(), b.xln.data_ptr(), b.dd.data_ptr(), out5, stream()),
                        "v6_token_shift"))
                    plan.append(run_decay)
                if split:
                    # the decay only feeds the recurrence: its two small launches run on a side stream beside the
                    # r / k / v / g matmuls (which leave a fifth of the SM slots free) and join before rwkv_wkv56_one
                    joined = [None]

                    def fork_decay(run_decay=run_decay, joined=joined):
                        main = torch.cuda.current_stream(dev)
                        if not self._fork_streams:
                            self._fork_streams.append(torch.cuda.Stream(dev))
                        side = self._fork_streams[0]
                        start = torch.cuda.Event()
                        start.record(main)
                        side.wait_event(start)
                        with torch.cuda.stream(side):
                            run_decay()
                            joined[0] = torch.cuda.Event()
                            joined[0].record(side)
                    plan.append(fork_decay)
                gemv([P(b.m3, att + "receptance.weight", b.r, EPI_STORE), P(b.m1, att + "key.weight", b.k, EPI_STORE),
                      P(b.m2, att + "value.weight", b.v, EPI_STORE), P(b.m4, att + "gate.weight", b.g, EPI_SILU)])
                if split:
                    plan.append(lambda joined=joined: torch.cuda.current_stream(dev).wait_event(joined[0]))
                decay = b.wdec
            else:
                mix = lambda n: w[att + "time_mix_" + n]
                gemv([ln(P(b.x, att + "receptance.weight", b.r, EPI_STORE), *ln1, 0, sin[s], mix("r"), sout[s]),
                      ln(P(b.x, att + "key.weight", b.k, EPI_STORE), *ln1, 0, sin[s], mix("k")),
                      ln(P(b.x, att + "value.weight", b.v, EPI_STORE), *ln1, 0, sin[s], mix("v")),
                      ln(P(b.x, att + "gate.weight", b.g, EPI_SILU), *ln1, 0, sin[s], mix("g"))])
                decay = w[att + "time_decay"].reshape(-1)
            plan.append(lambda s=s, att=att, decay=decay, u=u: check(
                L.rwkv_wkv56_one(H, N, b.r.data_ptr(), b.k.data_ptr(), b.v.data_ptr(), decay.data_ptr(), u.data_ptr(),
                                 sin[s + 1].data_ptr(), sout[s + 1].data_ptr(), w[att + "ln_x.weight"].data_ptr(),
                                 w[att + "ln_x.bias"].data_ptr(), b.g.data_ptr(), b.att.data_ptr(), stream()), "wkv56_one"))
            gemv([P(b.att, att + "output.weight", b.x, EPI_RESIDUAL, aux=b.x)])
            mode = 1 if v6 else 0
            mk, mr = (w[ffn + "time_maa_k"], w[ffn + "time_maa_r"]) if v6 else (w[ffn + "time_mix_k"], w[ffn + "time_mix_r"])
            gemv([ln(P(b.x, ffn + "receptance.weight", b.fr, EPI_SIGMOID), *ln2, mode, sin[s + 2], mr, sout[s + 2]),
                  ln(P(b.x, ffn + "key.weight", b.fk, EPI_RELU_SQ), *ln2, mode, sin[s + 2], mk)])
            scale = 0.5 if (self.RESCALE_LAYER > 0 and (i + 1) % self.RESCALE_LAYER == 0) else 1.0
            gemv([P(b.fk, ffn + "value.weight", b.x, EPI_MUL_RESIDUAL, aux=b.x, aux2=b.fr, out_scale=scale)])
        gemv([ln(P(b.x, "head.weight", b.logits, EPI_STORE_F32), w["ln_out.weight"], w["ln_out.bias"], 2)])
        self._plan_keep = getattr(self, "_plan_keep", []) + keep
        return plan

    def _step_one_v56(self, cur):
        b, w = self._b, self.w
        self._embed_row()
        if not hasattr(self, "_plans56"):
            self._plans56 = [self._plan_v56(0), self._plan_v56(1)]
        for op in self._plans56[cur]:
            op()

    # ----- sequence ------------------------------------------------------------------------
    def _plain(self, x, name, epilogue=EPI_STORE, aux=None, aux2=None, out_scale=1.0, out=None):
        """A layer kept in fp16 ('cuda fp16', model.py:143-167): a library GEMM with fp32 accumulation, then the
        reference's own pointwise ops on fp16 tensors (one rounding each)."""
        y = x @ self.w[name]
        if epilogue == EPI_SIGMOID:
            y = torch.sigmoid(y)
        elif epilogue == EPI_RELU_SQ:
            y = torch.relu(y) ** 2
        elif epilogue == EPI_RESIDUAL:
            y = aux + y
        elif epilogue == EPI_MUL_RESIDUAL:
            y = aux + aux2 * y
        elif epilogue == EPI_SILU:
            y = F.silu(y)
        if out_scale != 1.0:
            y = y * out_scale
        if out is not None:
            out.copy_(y)
            return out
        return y

    def _mm_seq(self, x, name, out_dtype=None):
        if self.w[name].dtype != torch.uint8:
            y = self._plain(x, name)
            return y if out_dtype is None else y.to(out_dtype)
        wq, mx, rx, my, ry = self._scales(name)
        T = x.shape[0]
        N, M = wq.shape
        if self._world > 1:
            full = self._full_m[name]
            y = torch.zeros((T, shard.shard_width(full, self._world)), dtype=torch.float16, device=x.device)
            if M > 0:
                torch.ops.rwkv.mm8_seq(T, N, M, x, wq, mx, rx, my, ry, y[:, :M])
            y = shard.gather_columns(y, full, self._world).contiguous()
        else:
            y = torch.empty((T, M), dtype=torch.float16, device=x.device)
            torch.ops.rwkv.mm8_seq(T, N, M, x, wq, mx, rx, my, ry, y)
        return y if out_dtype is None else y.to(out_dtype)

    def _mm_epi(self, x, name, epilogue, aux=None, aux2=None, out_scale=1.0, out=None):
        """mm8_seq with the reference's next pointwise op(s) fused into the store (single-GPU path)."""
        if self.w[name].dtype != torch.uint8:
            return self._plain(x, name, epilogue, aux, aux2, out_scale, out)
        wq, mx, rx, my, ry = self._scales(name)
        M = wq.shape[1]
        if M % 8 != 0 and out is None and aux is None and aux2 is None and wq.stride(0) >= (M + 7) // 8 * 8:
            # An out-feature count like 50277 would send the whole matrix to the CUDA-core kernel (the tensor-core one
            # stores columns in groups of 8): run it on the view that includes the row padding (up to 7 more columns,
            # whose results are dropped) with mx, rx padded alike.
            pad = self._mm_pad.get(name)
            if pad is None:
                Mp = (M + 7) // 8 * 8
                pad = self._mm_pad[name] = (torch.as_strided(wq, (wq.shape[0], Mp), (wq.stride(0), 1), wq.storage_offset()),
                                            torch.nn.functional.pad(mx, (0, Mp - M)), torch.nn.functional.pad(rx, (0, Mp - M)))
            y = torch.empty((x.shape[0], pad[0].shape[1]), dtype=torch.float16, device=x.device)
            return ops.mm8_seq_epi(x, pad[0], pad[1], pad[2], my, ry, y, epilogue, None, None, out_scale)[:, :M]
        y = out if out is not None else torch.empty((x.shape[0], M), dtype=torch.float16, device=x.device)
        return ops.mm8_seq_epi(x, wq, mx, rx, my, ry, y, epilogue, aux, aux2, out_scale)

    def _mm_fork(self, jobs, extra=None):
        """Independent matmuls of a batched decode step (r / k / v, or the two of the channel mix) on parallel
        streams: `jobs` = [(x, name, epilogue)]; returns the outputs.  At a handful of rows every matmul is a
        latency-bound chain of three short kernels, and the chains of independent matmuls overlap instead of queueing
        (also inside a captured graph: the side streams fork from and join the capturing stream).  `extra`: one more
        independent piece of work (a callable that launches on the current stream), run on a stream of its own."""
        outs = [torch.empty((x.shape[0], self.w[name].shape[1]), dtype=torch.float16, device=x.device) for x, name, _ in jobs]
        work = [lambda x=x, name=name, epi=epi, y=y: self._mm_epi(x, name, epi, out=y) for (x, name, epi), y in zip(jobs, outs)]
        if extra is not None:
            work.append(extra)
        if not self._batch_fork or len(work) < 2:
            for f in work:
                f()
            return outs
        main = torch.cuda.current_stream(self.device)
        while len(self._fork_streams) < len(work) - 1:
            self._fork_streams.append(torch.cuda.Stream(self.device))
        start = torch.cuda.Event()
        start.record(main)
        joins = []
        for side, f in zip(self._fork_streams, work[1:]):
            side.wait_event(start)
            with torch.cuda.stream(side):
                f()
                ev = torch.cuda.Event()
                ev.record(side)
                joins.append(ev)
        work[0]()
        for ev in joins:
            main.wait_event(ev)
        return outs

    def _att_seq_v4(self, x, st, i, rows=False):
        """cuda_att_seq (model.py:1346-1360): LayerNorm + mixes, r/k/v matmuls (sigmoid in the store), the WKV
        recurrence parallel in time with r * wkv in its store, output matmul with the residual in the store."""
        w, a = self.w, self.args
        T, C = x.shape
        bb, att = f"blocks.{i}.", f"blocks.{i}.att."
        kx, vx, rx = (torch.empty_like(x) for _ in range(3))
        new_sx = torch.empty_like(st[i * 5 + 0])
        self._ln_mix(T, x, st[i * 5 + 0], w[bb + "ln1.weight"], w[bb + "ln1.bias"], 0,
                     [w[att + "time_mix_k"], w[att + "time_mix_v"], w[att + "time_mix_r"]], [kx, vx, rx],
                     new_state=None if rows else new_sx, xx_out=new_sx if rows else None, rows=rows)
        if self._world == 1 and rows:
            r, k, v = self._mm_fork([(rx, att + "receptance.weight", EPI_SIGMOID), (kx, att + "key.weight", EPI_STORE),
                                     (vx, att + "value.weight", EPI_STORE)])
        elif self._world == 1:
            r = self._mm_epi(rx, att + "receptance.weight", EPI_SIGMOID)
            k = self._mm_epi(kx, att + "key.weight", EPI_STORE)             # fp16 k, v: the kernel widens them, as
            v = self._mm_epi(vx, att + "value.weight", EPI_STORE)           # model.py:1355-1356 does before the op
        if self._world == 1:
            if rows:        # T sequences of one step each: the operator's batch dimension, state [T, C]
                ops.wkv4_seq(w[att + "time_decay"], w[att + "time_first"], k.view(T, 1, C), v.view(T, 1, C), k.view(T, 1, C),
                             st[i * 5 + 1], st[i * 5 + 2], st[i * 5 + 3], r=r.view(T, 1, C))
            else:
                ops.wkv4_seq(w[att + "time_decay"], w[att + "time_first"], k, v, k, st[i * 5 + 1], st[i * 5 + 2], st[i * 5 + 3], r=r)
            st[i * 5 + 0] = new_sx
            return self._mm_epi(k, att + "output.weight", EPI_RESIDUAL, aux=x, out=x)
        r = torch.sigmoid(self._mm_seq(rx, att + "receptance.weight"))
        k = self._mm_seq(kx, att + "key.weight", torch.float32)
        v = self._mm_seq(vx, att + "value.weight", torch.float32)
        y = torch.empty((T, C), dtype=torch.float32, device=x.device)
        torch.ops.rwkv.wkv_forward(1, T, C, w[att + "time_decay"], w[att + "time_first"], k, v, y,
                                   st[i * 5 + 1], st[i * 5 + 2], st[i * 5 + 3])
        out = self._mm_seq(r * y.to(x.dtype), att + "output.weight")
        st[i * 5 + 0] = new_sx
        return x + out

    def _att_seq_v56(self, x, st2, i, rows=False):
        """cuda_att_seq_v5_2 / cuda_att_seq_v6_0 (model.py:1363-1439).  `st2` = [att_xx, att_kv]; the first entry is
        replaced, the matrix state is updated in place in the model's [H, key, value] layout.  Kernels of this
        library throughout; the four small low-rank products of RWKV-6 (ranks 32..160) are plain fp16 library GEMMs
        as in the reference (`@`, `bmm`)."""
        import ctypes as C
        w, a, L = self.w, self.args, lib()
        T, D = x.shape
        H = a.n_head
        N = a.n_att // H
        dev = x.device
        bb, att = f"blocks.{i}.", f"blocks.{i}.att."
        stream = torch.cuda.current_stream(dev).cuda_stream
        new_sx = torch.empty_like(st2[0])
        h = lambda *shape: torch.empty(shape, dtype=torch.float16, device=dev)
        if self.version == 6:
            xx, xxx = h(T, D), h(T, D)
            self._ln_mix(T, x, st2[0], w[bb + "ln1.weight"], w[bb + "ln1.bias"], 1, [w[att + "time_maa_x"]], [xxx],
                         xx_out=xx, new_state=None if rows else new_sx, rows=rows)
            if rows:
                new_sx = xx
            # low-rank offsets of the five mixes: tanh(xxx @ w1) as [5, T, Lm], times w2 [5, Lm, D]
            w1, w2 = w[att + "time_maa_w1"], w[att + "time_maa_w2"]
            Lm = w2.shape[1]
            h1, h1t = h(T, 5 * Lm), h(5, T, Lm)
            torch.ops.rwkv.gemm_fp16_cublas(xxx, w1, h1)
            check(L.rwkv_tanh_regroup_f16(T, 5, Lm, h1.data_ptr(), h1t.data_ptr(), stream), "tanh")
            m5 = h(5, T, D)
            torch.ops.rwkv.gemm_fp16_cublas(h1t, w2, m5)
            mixes = h(5, T, D)
            maa5 = (C.c_void_p * 5)(*[w[att + "time_maa_" + n].data_ptr() for n in "wkvrg"])
            out5 = (C.c_void_p * 5)(*[mixes[j].data_ptr() for j in range(5)])
            check(L.rwkv_v6_seq_mix(T, D, xx.data_ptr(), xx.stride(0), st2[0].data_ptr(), st2[0].stride(0) if rows else 0,
                                    m5.data_ptr(), maa5, out5, stream),
                  "v6_seq_mix")
            wx, kx, vx, rx, gx = mixes.unbind(0)
            # per-token decay exp(-exp(time_decay + tanh(wx @ dw1) @ dw2)): only the recurrence needs it, so in a
            # batched decode step its four launches run beside the r / k / v / g matmuls
            dw1, dw2 = w[att + "time_decay_w1"], w[att + "time_decay_w2"]
            h2, d2 = h(T, dw1.shape[1]), h(T, D)
            decay = torch.empty((T, D), dtype=torch.float32, device=dev)

            def decay_chain():
                s_ = torch.cuda.current_stream(dev).cuda_stream
                torch.ops.rwkv.gemm_fp16_cublas(wx, dw1, h2)
                check(L.rwkv_tanh_regroup_f16(T, 1, h2.shape[1], h2.data_ptr(), h2.data_ptr(), s_), "tanh")
                torch.ops.rwkv.gemm_fp16_cublas(h2, dw2, d2)
                check(L.rwkv_v6_seq_decay(T, D, w[att + "time_decay"].data_ptr(), d2.data_ptr(), decay.data_ptr(), s_), "v6_seq_decay")
            if not rows:
                decay_chain()
        else:
            kx, vx, rx, gx = (torch.empty_like(x) for _ in range(4))
            self._ln_mix(T, x, st2[0], w[bb + "ln1.weight"], w[bb + "ln1.bias"], 0,
                         [w[att + f"time_mix_{n}"] for n in "kvrg"], [kx, vx, rx, gx],
                         new_state=None if rows else new_sx, xx_out=new_sx if rows else None, rows=rows)
            decay = w[att + "time_decay"].reshape(-1)
        if rows:    # fp16-rounded r, k, v: the kernel widens them (model.py:1413, 1425-1427)
            r, k, v, g = self._mm_fork([(rx, att + "receptance.weight", EPI_STORE), (kx, att + "key.weight", EPI_STORE),
                                        (vx, att + "value.weight", EPI_STORE), (gx, att + "gate.weight", EPI_SILU)],
                                       extra=decay_chain if self.version == 6 else None)
        else:
            r = self._mm_epi(rx, att + "receptance.weight", EPI_STORE)
            k = self._mm_epi(kx, att + "key.weight", EPI_STORE)
            v = self._mm_epi(vx, att + "value.weight", EPI_STORE)
            g = self._mm_epi(gx, att + "gate.weight", EPI_SILU)
        y = torch.empty((T, D), dtype=torch.float32, device=dev)
        S_in = st2[1] if st2[1].is_contiguous() else st2[1].contiguous()
        S = torch.empty_like(S_in)                  # the caller's state stays as it is, as with the reference's copy
        u = w[att + "time_first"].reshape(-1)
        if rows:
            # T sequences of one step each = T * H independent heads of one step; the per-head vectors repeat per sequence
            u = self._tiled(att + "time_first", u, T)
            if self.version != 6:
                decay = self._tiled(att + "time_decay", decay, T)
            ops.wkv56_seq(self.version == 6, T * H, S_in, r.view(1, T * D), k.view(1, T * D), v.view(1, T * D), decay.view(-1) if
                          self.version != 6 else decay.view(1, T * D), u, y.view(1, T * D), model_layout=True, state_out=S)
        else:
            ops.wkv56_seq(self.version == 6, H, S_in, r, k, v, decay, u, y, model_layout=True, state_out=S)
        out = h(T, D)
        check(L.rwkv_v56_seq_gn_gate(T, H, N, y.data_ptr(), w[att + "ln_x.weight"].data_ptr(), w[att + "ln_x.bias"].data_ptr(),
                                     g.data_ptr(), out.data_ptr(), 64e-5, stream), "gn_gate")
        st2[0] = new_sx
        st2[1] = S
        return self._mm_epi(out, att + "output.weight", EPI_RESIDUAL, aux=x, out=x)

    def _tiled(self, name, t, reps):
        """A per-head / per-channel model vector repeated for `reps` sequences (cached: made once per batch size)."""
        key = (name, reps)
        c = self._tile_cache.get(key)
        if c is None:
            c = self._tile_cache[key] = t.reshape(-1).repeat(reps).contiguous()
        return c

    def _ffn_seq(self, x, sx, i, rows=False):
        """ffn_seq / ffn_seq_v6 (model.py:995-1004, 1019-1029)."""
        w = self.w
        T = x.shape[0]
        bb, ffn = f"blocks.{i}.", f"blocks.{i}.ffn."
        kx, rx = torch.empty_like(x), torch.empty_like(x)
        new_sx = torch.empty_like(sx)
        v6 = self.version == 6
        self._ln_mix(T, x, sx, w[bb + "ln2.weight"], w[bb + "ln2.bias"], 1 if v6 else 0,
                     [w[ffn + ("time_maa_k" if v6 else "time_mix_k")], w[ffn + ("time_maa_r" if v6 else "time_mix_r")]], [kx, rx],
                     new_state=None if rows else new_sx, xx_out=new_sx if rows else None, rows=rows)
        if self._world == 1:
            if rows:
                r, vx = self._mm_fork([(rx, ffn + "receptance.weight", EPI_SIGMOID), (kx, ffn + "key.weight", EPI_RELU_SQ)])
            else:
                r = self._mm_epi(rx, ffn + "receptance.weight", EPI_SIGMOID)
                vx = self._mm_epi(kx, ffn + "key.weight", EPI_RELU_SQ)
            # x + r * (vx @ Wv), and the halving after every RESCALE_LAYER-th layer (model.py:1660-1662), in the store
            half = self.RESCALE_LAYER > 0 and (i + 1) % self.RESCALE_LAYER == 0
            return self._mm_epi(vx, ffn + "value.weight", EPI_MUL_RESIDUAL, aux=x, aux2=r, out_scale=0.5 if half else 1.0,
                                out=x), new_sx
        r = torch.sigmoid(self._mm_seq(rx, ffn + "receptance.weight"))
        vx = torch.relu(self._mm_seq(kx, ffn + "key.weight")) ** 2
        out = r * self._mm_seq(vx, ffn + "value.weight")
        return x + out, new_sx

    # ----- batched decode: B independent sequences, one token each ---------------------------
    def zero_batch_state(self, B):
        """The state of B fresh sequences: the entries of the ordinary state list with a leading batch dimension."""
        return [torch.stack([t] * B).contiguous() for t in self._zero_state()]

    @staticmethod
    def stack_states(states):
        """B ordinary state lists (e.g. after B separate prefills) -> one batch state."""
        return [torch.stack([s[j].contiguous() for s in states]).contiguous() for j in range(len(states[0]))]

    @staticmethod
    def unstack_states(batch_state):
        B = batch_state[0].shape[0]
        return [[t[b] for t in batch_state] for b in range(B)]

    def forward_batch(self, tokens, state):
        """One decode step for B independent sequences at once (an addition to the reference's API, which has no batch
        dimension: its kernels carry a B they cannot use, rwkv6.cu:13-17).  `tokens`: B token ids; `state`: None, a batch
        state returned by an earlier call (or by zero_batch_state / stack_states).  Returns (logits fp32 [B, V],
        batch state).  The B sequences are the rows of the tensor-core mm8_seq kernel, so the packed weights are
        streamed once per step for all of them; every sequence follows the arithmetic of the prefill path with T = 1.
        The RWKV-4 WKV states (aa, bb, pp) are updated in place, everything else is returned in new tensors."""
        if self._world > 1:
            raise NotImplementedError("forward_batch: single-GPU models only")
        with torch.no_grad(), torch.cuda.device(self.device):
            B = len(tokens)
            idx = tokens if torch.is_tensor(tokens) else torch.tensor([int(t) for t in tokens], dtype=torch.int64, device=self.device)
            idx = idx.to(self.device).reshape(B)
            if self._use_graph and os.environ.get("RWKV_B200_BATCH_GRAPH", "1") != "0":
                return self._forward_batch_graph(idx, state)
            return self._forward_batch_eager(idx, state)

    def _forward_batch_graph(self, idx, state):
        """forward_batch as one CUDA-graph replay per batch size.  The graph reads the state from fixed input tensors
        and leaves the new state in fixed output tensors (its first node copies outputs back to inputs), so the list
        it returns is overwritten by the next call with the same batch size: pass copy.deepcopy(state) around to keep
        a snapshot, as with the one-token forward."""
        B = idx.numel()
        g = self._batch_graphs.get(B)
        if g is None:
            g = types.SimpleNamespace(tok=torch.zeros(B, dtype=torch.int64, device=self.device),
                                      inp=self.zero_batch_state(B), out=None, logits=None, graph=None)
            # one eager step on the capture stream warms every kernel up and sizes the per-stream operator workspaces
            side = torch.cuda.Stream(self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):
                self._forward_batch_eager(g.tok, [t.clone() for t in g.inp])
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                g.logits, g.out = self._forward_batch_eager(g.tok, g.inp)
            # the previous step's outputs become the next step's inputs (entries updated in place are their own output)
            moved = [(i, o) for i, o in zip(g.inp, g.out) if i is not o]
            g.graph, g.moved = graph, moved
            self._batch_graphs[B] = g
            state_is_ours = False
        else:
            state_is_ours = state is not None and len(state) == len(g.out) and all(a is b for a, b in zip(state, g.out))
        if state is None:
            state = self.zero_batch_state(B)
            state_is_ours = False
        if state_is_ours:
            if g.moved:
                torch._foreach_copy_([i for i, _ in g.moved], [o for _, o in g.moved])
        else:
            torch._foreach_copy_(g.inp, [t for t in state])
        g.tok.copy_(idx)
        g.graph.replay()
        return g.logits.clone(), list(g.out)

    def _forward_batch_eager(self, idx, state):
        with torch.no_grad():
            w, a = self.w, self.args
            B = idx.numel()
            state = self.zero_batch_state(B) if state is None else list(state)
            x = w["emb.weight"].index_select(0, idx)
            for i in range(a.n_layer):
                if self.version == 4:
                    x = self._att_seq_v4(x, state, i, rows=True)
                    x, state[i * 5 + 4] = self._ffn_seq(x, state[i * 5 + 4], i, rows=True)
                else:
                    st2 = [state[i * 3 + 0], state[i * 3 + 1]]
                    x = self._att_seq_v56(x, st2, i, rows=True)
                    state[i * 3 + 0], state[i * 3 + 1] = st2
                    x, state[i * 3 + 2] = self._ffn_seq(x, state[i * 3 + 2], i, rows=True)
            xln = torch.empty_like(x)
            self._ln_mix(B, x, None, w["ln_out.weight"], w["ln_out.bias"], 0, [], [], xx_out=xln)
            return self._mm_epi(xln, "head.weight", EPI_STORE).float(), state

    def _stage_tokens(self, tokens):
        """Token ids to the device through pinned memory (two slots, reused in turn): a copy from pageable memory would
        make the host wait for everything queued before it, so consecutive chunks of a prompt could not be queued ahead."""
        T = len(tokens)
        if not hasattr(self, "_seq_tok"):
            self._seq_tok = [None, None]
            self._seq_tok_ev = [None, None]
            self._seq_tok_slot = 0
        slot = self._seq_tok_slot = 1 - self._seq_tok_slot
        if self._seq_tok_ev[slot] is not None:
            self._seq_tok_ev[slot].synchronize()
        if self._seq_tok[slot] is None or self._seq_tok[slot].numel() < T:
            self._seq_tok[slot] = torch.empty(max(4096, T), dtype=torch.int64).pin_memory()
            self._seq_tok_ev[slot] = torch.cuda.Event()
        host = self._seq_tok[slot][:T]
        host.copy_(torch.tensor(tokens, dtype=torch.int64))
        idx = torch.empty(T, dtype=torch.int64, device=self.device)
        idx.copy_(host, non_blocking=True)
        self._seq_tok_ev[slot].record(torch.cuda.current_stream(self.device))
        return idx

    def _forward_seq(self, tokens, state, full_output):
        # (Replaying a prompt length that comes back as a CUDA graph was tried: with the copies of the state in and out
        # it was slower than these direct launches at 64, 256 and 1024 tokens.)
        w, a = self.w, self.args
        state = list(state)
        idx = self._stage_tokens(tokens)
        x = w["emb.weight"].index_select(0, idx)
        for i in range(a.n_layer):
            if self.version == 4:
                x = self._att_seq_v4(x, state, i)
                x, state[i * 5 + 4] = self._ffn_seq(x, state[i * 5 + 4], i)
            else:
                st2 = [state[i * 3 + 0], state[i * 3 + 1]]
                x = self._att_seq_v56(x, st2, i)
                state[i * 3 + 0], state[i * 3 + 1] = st2
                x, state[i * 3 + 2] = self._ffn_seq(x, state[i * 3 + 2], i)
            if self._world > 1 and self.RESCALE_LAYER > 0 and (i + 1) % self.RESCALE_LAYER == 0:
                x = x / 2           # (single GPU: fused into the ffn.value store)
        if not full_output:
            x = x[-1:, :]
        xln = torch.empty_like(x)
        self._ln_mix(x.shape[0], x, None, w["ln_out.weight"], w["ln_out.bias"], 0, [], [], xx_out=xln)
        if full_output and self._world == 1:
            out = self._mm_epi(xln, "head.weight", EPI_STORE)
        elif full_output or self._world > 1:
            out = self._mm_seq(xln, "head.weight")
            if not full_output:
                out = out[0]
        elif w["head.weight"].dtype != torch.uint8:
            out = self._plain(xln, "head.weight")[0]
        else:
            wq, mx, rx, my, ry = self._scales("head.weight")
            y = torch.zeros(wq.shape[1], dtype=torch.float32, device=self.device)
            torch.ops.rwkv.mm8_one(wq.shape[0], wq.shape[1], xln[0], wq, mx, rx, my, ry, y)
            out = y.to(torch.float16)
        return out.float(), state
