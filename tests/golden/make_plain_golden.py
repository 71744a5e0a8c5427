"""Golden vectors for the strategies WITHOUT int8 ('xxx fp32', and the mixed 'xxx fp32i8 *K -> xxx fp32'), made by
EXECUTING THE REFERENCE on CPU (rwkv_pip_package/src/rwkv/model.py, RWKV_CUDA_ON=0) on the toy checkpoints of
make_golden.py:

    RWKV_REFERENCE_ROOT=<path to the ChatRWKV checkout> python tests/golden/make_plain_golden.py

Writes tests/golden/reference_cpu_plain.npz: logits of a whole-sequence call and of token-by-token calls for
RWKV-4 and RWKV-6 under 'cpu fp32' and under 'cpu fp32i8 *2 -> cpu fp32' (the first two layers packed to int8, the
rest and the head plain).  They pin the oracle's unquantised matmul and its per-layer choice of weight type."""
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
from tests.golden.make_golden import TOKENS, TOY  # noqa: E402


def main():
    sys.path.insert(0, os.path.join(os.environ["RWKV_REFERENCE_ROOT"], "rwkv_pip_package", "src"))
    import rwkv.model as ref
    out, tmp = {}, tempfile.mkdtemp()
    for name in ("v4", "v6"):
        ck = synth.make_checkpoint(**TOY[name])
        path = os.path.join(tmp, f"{name}.pth")
        torch.save(ck, path)
        for tag, strategy in (("plain", "cpu fp32"), ("mixed", "cpu fp32i8 *2 -> cpu fp32")):
            m = ref.RWKV(path, strategy, verbose=False)
            full, _ = m.forward(TOKENS, None, full_output=True)
            out[f"{name}/{tag}/full"] = full.numpy()
            st, ones = None, []
            for t in TOKENS:
                o, st = m.forward([t], st)
                ones.append(o.numpy())
            out[f"{name}/{tag}/one"] = np.stack(ones)
    np.savez_compressed(os.path.join(HERE, "reference_cpu_plain.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
