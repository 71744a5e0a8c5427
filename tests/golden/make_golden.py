"""Generate the golden fixtures in this directory by EXECUTING THE REFERENCE on CPU.

Run once, in a container that has the read-only reference tree:

    python tests/golden/make_golden.py /path/to/reference

It imports `rwkv.model` from <reference>/rwkv_pip_package/src with RWKV_CUDA_ON=0 and
records, for seeded random-init checkpoints (chatrwkv_b200.synth, regenerated from their
seeds by the tests, so not stored):

  * packing: the uint8 tensors and mx/rx/my/ry the reference loader produces
    (strategies 'cpu fp32i8' and 'cpu fp16i8': the latter gives fp16 scale vectors and the
    RESCALE_LAYER=6 pre-division of att.output / ffn.value);
  * mm8: outputs of the reference's torch_mm8_one / torch_mm8_seq on fp32 operands;
  * models: logits and final states of RWKV-4, RWKV-5.2 and RWKV-6 toy models under
    'cpu fp32i8', for a whole-sequence call, split calls and token-by-token calls.

The fixtures are what pins the CPU oracle (oracle/rwkv_oracle.py) to the reference.
"""
import os
import sys
import tempfile

import numpy as np
import torch

os.environ["RWKV_CUDA_ON"] = "0"
os.environ["RWKV_JIT_ON"] = "0"

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from chatrwkv_b200 import synth  # noqa: E402

# toy model shapes shared with tests/test_oracle_golden.py
TOY = {
    "v4": dict(version=4, n_layer=8, n_embd=64, n_ffn=256, vocab=300, seed=11, head_size=16),
    "v5": dict(version=5.2, n_layer=3, n_embd=64, n_ffn=224, vocab=300, seed=12, head_size=16),
    "v6": dict(version=6, n_layer=3, n_embd=64, n_ffn=224, vocab=300, seed=13, head_size=16,
               maa_rank=8, decay_rank=16),
}
TOKENS = synth.make_tokens(12, 300, 2000)


def main(ref_root):
    sys.path.insert(0, os.path.join(ref_root, "rwkv_pip_package", "src"))
    import rwkv.model as ref

    out = {}
    tmp = tempfile.mkdtemp()

    def load(name, strategy):
        ck = synth.make_checkpoint(**TOY[name])
        path = os.path.join(tmp, f"{name}.pth")
        torch.save(ck, path)
        return ref.RWKV(path, strategy, verbose=False)

    # ---- packing ------------------------------------------------------------------
    for strat, tag in (("cpu fp32i8", "f32"), ("cpu fp16i8", "f16")):
        m = load("v4", strat)
        for key in ("blocks.0.att.key.weight", "blocks.7.att.output.weight",
                    "blocks.0.ffn.key.weight", "blocks.7.ffn.value.weight", "head.weight"):
            for suf in ("", "_mx", "_rx", "_my", "_ry"):
                t = m.w[key + suf]
                arr = t.contiguous().view(torch.int16).numpy() if t.dtype == torch.float16 else t.contiguous().numpy()
                out[f"pack/{tag}/{key}{suf}"] = arr

    # ---- mm8 spec -------------------------------------------------------------------
    m = load("v4", "cpu fp32i8")
    g = torch.Generator().manual_seed(3000)
    for key in ("blocks.0.ffn.key.weight", "blocks.0.ffn.value.weight", "head.weight"):
        w_, mx, rx, my, ry = (m.w[key + s] for s in ("", "_mx", "_rx", "_my", "_ry"))
        x1 = torch.randn(w_.shape[0], generator=g)
        xs = torch.randn(5, w_.shape[0], generator=g)
        out[f"mm8/{key}/x1"] = x1.numpy()
        out[f"mm8/{key}/xs"] = xs.numpy()
        out[f"mm8/{key}/y1"] = ref.torch_mm8_one(x1, w_, mx, rx, my, ry).numpy()
        out[f"mm8/{key}/ys"] = ref.torch_mm8_seq(xs, w_, mx, rx, my, ry).numpy()

    # ---- models -------------------------------------------------------------------
    def st_np(state):
        return [s.detach().float().contiguous().numpy() for s in state]

    for name in ("v4", "v5", "v6"):
        m = load(name, "cpu fp32i8")
        full, st = m.forward(TOKENS, None, full_output=True)
        out[f"model/{name}/full"] = full.numpy()
        for j, s in enumerate(st_np(st)):
            out[f"model/{name}/state_full/{j}"] = s
        # split: 5 + 1 + 6
        o, st = m.forward(TOKENS[:5], None)
        out[f"model/{name}/split_a"] = o.numpy()
        o, st = m.forward(TOKENS[5:6], st)
        out[f"model/{name}/split_b"] = o.numpy()
        o, st = m.forward(TOKENS[6:], st)
        out[f"model/{name}/split_c"] = o.numpy()
        # token by token
        st = None
        ones = []
        for t in TOKENS:
            o, st = m.forward([t], st)
            ones.append(o.numpy())
        out[f"model/{name}/one"] = np.stack(ones)
        for j, s in enumerate(st_np(st)):
            out[f"model/{name}/state_one/{j}"] = s

    np.savez_compressed(os.path.join(HERE, "reference_cpu.npz"), **out)
    print("wrote", os.path.join(HERE, "reference_cpu.npz"), len(out), "arrays")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ["RWKV_REFERENCE_ROOT"])
