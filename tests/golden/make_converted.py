"""Generate tests/golden/ref_converted_v4.pth: the toy RWKV-4 checkpoint converted for strategy
'cuda fp16i8' BY THE REFERENCE's own loader (`convert_and_save_and_exit`, which needs no GPU:
rwkv_pip_package/src/rwkv/model.py:851, 894-903).  The file pins the packer and the converted-
checkpoint reader end to end: the product must load it and must produce the same packed tensors
from the raw checkpoint.

    python tests/golden/make_converted.py /path/to/reference
"""
import os
import sys
import tempfile

import torch

os.environ["RWKV_CUDA_ON"] = "0"
os.environ["RWKV_JIT_ON"] = "0"
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from chatrwkv_b200 import synth  # noqa: E402
from tests.golden.make_golden import TOY  # noqa: E402

if __name__ == "__main__":
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ["RWKV_REFERENCE_ROOT"]
    sys.path.insert(0, os.path.join(ref_root, "rwkv_pip_package", "src"))
    import rwkv.model as ref
    tmp = tempfile.mkdtemp()
    raw = os.path.join(tmp, "toy_v4.pth")
    torch.save(synth.make_checkpoint(**TOY["v4"]), raw)
    out = os.path.join(HERE, "ref_converted_v4.pth")
    try:
        ref.RWKV(raw, "cuda fp16i8", verbose=False, convert_and_save_and_exit=out)
    except SystemExit:
        pass
    print("wrote", out, os.path.getsize(out))
