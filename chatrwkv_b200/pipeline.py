"""Generation loop with the sampler on the GPU: the host-side mirror of `PIPELINE` / `PIPELINE_ARGS`
(rwkv_pip_package/src/rwkv/utils.py:10-135) over `rwkv_sample_logits` (csrc/sample.cu).

Same argument names and meaning as the reference: temperature, top_p, top_k, alpha_frequency, alpha_presence,
alpha_decay, token_ban, token_stop, chunk_len.  What differs: the draw uses this object's seeded stream of uniform
numbers (the reference draws with numpy or torch.multinomial), and tokenizers are the caller's: pass any object with
`encode(str) -> list[int]` and `decode(list[int]) -> str`, or none and work with token ids.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import check, lib


class PIPELINE_ARGS:
    """utils.py:10-21."""

    def __init__(self, temperature=1.0, top_p=0.85, top_k=0, alpha_frequency=0.2, alpha_presence=0.2, alpha_decay=0.996,
                 token_ban=(), token_stop=(), chunk_len=256):
        self.temperature = temperature
        self.top_p = top_p
        self.top_k = top_k
        self.alpha_frequency = alpha_frequency
        self.alpha_presence = alpha_presence
        self.alpha_decay = alpha_decay
        self.token_ban = list(token_ban)
        self.token_stop = list(token_stop)
        self.chunk_len = chunk_len


class Sampler:
    """Device-side state of one generation: occurrence table, ban mask, uniform numbers, the token word."""

    def __init__(self, vocab, device, args=None, seed=0, token_weight=None, n_uniforms=4096):
        a = args or PIPELINE_ARGS()
        self.V, self.device, self.args = int(vocab), torch.device(device), a
        self.occurrence = torch.zeros(self.V, dtype=torch.float32, device=device)
        self.seen = torch.zeros(self.V, dtype=torch.uint8, device=device)
        self.banned = None
        if a.token_ban:
            self.banned = torch.zeros(self.V, dtype=torch.uint8, device=device)
            self.banned[torch.tensor(list(a.token_ban), dtype=torch.long, device=device)] = 1
        self.token_weight = None if token_weight is None else token_weight.to(device=device, dtype=torch.float32).contiguous()
        g = torch.Generator(device="cpu").manual_seed(int(seed))
        self.uniforms = torch.rand(n_uniforms, generator=g, dtype=torch.float32).to(device)
        self.counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.token = torch.zeros(1, dtype=torch.int64, device=device)

    def sample(self, logits, probs_out=None, penalties=True, temperature=None, top_p=None, top_k=None, uniforms=None):
        """One token from fp32 `logits` [V] on the device; returns the device tensor holding its id (int64 [1], reused by
        the next call).  Enqueues one kernel on the current stream; no host synchronisation."""
        a = self.args
        assert logits.is_cuda and logits.dtype == torch.float32 and logits.numel() == self.V and logits.is_contiguous()
        u = self.uniforms if uniforms is None else uniforms
        ptr = lambda t: t.data_ptr() if t is not None else None
        check(lib().rwkv_sample_logits(
            self.V, logits.data_ptr(),
            float(a.temperature if temperature is None else temperature), float(a.top_p if top_p is None else top_p),
            int(a.top_k if top_k is None else top_k),
            ptr(self.occurrence) if penalties else None, ptr(self.seen) if penalties else None, ptr(self.banned),
            ptr(self.token_weight), float(a.alpha_presence), float(a.alpha_frequency), float(a.alpha_decay),
            ptr(u), u.numel() if u is not None else 0, self.counter.data_ptr(), self.token.data_ptr(), ptr(probs_out),
            torch.cuda.current_stream(self.device).cuda_stream), "sample_logits")
        return self.token


class PIPELINE:
    """utils.py:23-135 without the tokenizer loading: `tokenizer` is any object with encode / decode, or None."""

    def __init__(self, model, tokenizer=None, seed=0):
        self.model = model
        self.tokenizer = tokenizer
        self.seed = seed
        self._weights = None

    def encode(self, x):
        ids = self.tokenizer.encode(x)
        return ids.ids if hasattr(ids, "ids") else ids

    def decode(self, x):
        return self.tokenizer.decode(x)

    def _vocab(self):
        return self.model.w["head.weight"].shape[1]

    def _token_weights(self):
        """utils.py:115-118: a token made only of blanks or digits adds 0 to its occurrence, any other 1."""
        if self.tokenizer is None:
            return None
        if self._weights is None:
            w = torch.ones(self._vocab(), dtype=torch.float32)
            for t in range(self._vocab()):
                try:
                    if self.decode([t]) in ' \t0123456789':
                        w[t] = 0.0
                except Exception:
                    pass
            self._weights = w
        return self._weights

    def sample_logits(self, logits, temperature=1.0, top_p=0.85, top_k=0, u=None):
        """utils.py:55-88 on the device; `u` (a number in [0, 1)) fixes the draw, else this object's seeded stream."""
        dev = self.model.device
        lg = logits.to(device=dev, dtype=torch.float32).contiguous()
        if not hasattr(self, "_plain") or self._plain.V != lg.numel():
            self._plain = Sampler(lg.numel(), dev, PIPELINE_ARGS(), self.seed)
        un = None if u is None else torch.tensor([float(u)], dtype=torch.float32, device=dev)
        tok = self._plain.sample(lg, penalties=False, temperature=temperature, top_p=top_p, top_k=top_k, uniforms=un)
        return int(tok.item())

    def _prefill(self, tokens, state, chunk_len):
        out = None
        tokens = list(tokens)
        while len(tokens) > 0:
            out, state = self.model.forward(tokens[:chunk_len], state)
            tokens = tokens[chunk_len:]
        return out, state

    def generate(self, ctx, token_count=100, args=None, callback=None, state=None):
        """utils.py:90-135.  `ctx` is text (needs a tokenizer) or a list of token ids; returns text when there is a
        tokenizer, else the list of generated ids.  The token comes to the host every step (stop list, callback), as in
        the reference; `generate_tokens` is the loop without that round trip."""
        args = args or PIPELINE_ARGS()
        tokens = self.encode(ctx) if isinstance(ctx, str) else list(ctx)
        sampler = Sampler(self._vocab(), self.model.device, args, self.seed, self._token_weights())
        out, state = self._prefill(tokens, state, args.chunk_len)
        all_tokens, out_last, out_str = [], 0, ''
        for i in range(token_count):
            token = int(sampler.sample(out).item())
            if token in args.token_stop:
                break
            all_tokens.append(token)
            if self.tokenizer is not None:
                tmp = self.decode(all_tokens[out_last:])
                if '\ufffd' not in tmp:     # a complete utf-8 string?
                    if callback:
                        callback(tmp)
                    out_str += tmp
                    out_last = i + 1
            elif callback:
                callback(token)
            if i + 1 < token_count:
                out, state = self.model.forward([token], state)
        return out_str if self.tokenizer is not None else all_tokens

    def generate_tokens(self, ctx_tokens, token_count=100, args=None, state=None):
        """The same loop with the token staying on the device between the sampler and the next forward: nothing is
        synchronised until the end, where the ids come back at once and are cut at the first stop token.  Returns
        (ids, state after the last forward)."""
        args = args or PIPELINE_ARGS()
        sampler = Sampler(self._vocab(), self.model.device, args, self.seed, self._token_weights())
        out, state = self._prefill(ctx_tokens, state, args.chunk_len)
        ids = torch.zeros(token_count, dtype=torch.int64, device=self.model.device)
        for i in range(token_count):
            tok = sampler.sample(out)
            ids[i:i + 1].copy_(tok)
            if i + 1 < token_count:
                out, state = self.model.forward(tok, state)
        got = ids.tolist()
        for j, t in enumerate(got):
            if t in args.token_stop:
                return got[:j], state
        return got, state
