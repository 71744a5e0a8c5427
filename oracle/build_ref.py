"""Builds the REFERENCE's own CUDA operators, from the sources where they lie in the
read-only reference tree, into oracle/_ref/ (git-ignored).  Checker and timing baseline only:
the product never loads these files.

    python -m oracle.build_ref /path/to/reference        (or RWKV_REFERENCE_ROOT=/path/to/reference)

Produces oracle/_ref/wkv_cuda_ref.so (wrapper.cpp + operators.cu + gemm_fp16_cublas.cpp:
torch.ops.rwkv.{mm8_one, mm8_seq, wkv_forward, gemm_fp16_cublas}) and rwkv5_ref.so /
rwkv6_ref.so (head size 64), compiled for sm_100 with the reference's own flags
(rwkv_pip_package/src/rwkv/model.py:32-38, 907-908, 940-941).  They register the same
operator names as the product, so tests load them in a separate process
(tests/ref_cuda_runner.py).

It also stages the reference's Python runtime (rwkv_pip_package/src/rwkv/{__init__,model}.py) as
oracle/_ref/pkg/rwkv/ so that tests/ref_model_runner.py can run the reference's own
`RWKV(model, 'cuda fp16i8').forward` beside the product on a GPU machine that has no reference
tree; like the .so files the staged package is git-ignored and never imported by the product.
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def default_reference_root():
    """RWKV_REFERENCE_ROOT, else a directory `reference` beside the repository."""
    env = os.environ.get("RWKV_REFERENCE_ROOT")
    if env:
        return env
    return os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def stage_package(ref_root):
    """Stage the reference's Python runtime under oracle/_ref/pkg/ (checker only)."""
    src = os.path.join(ref_root, "rwkv_pip_package", "src", "rwkv")
    dst = os.path.join(OUT, "pkg", "rwkv")
    os.makedirs(dst, exist_ok=True)
    for name in ("__init__.py", "model.py"):
        shutil.copyfile(os.path.join(src, name), os.path.join(dst, name))
    return dst


def build(ref_root=None, force=False):
    ref_root = ref_root or default_reference_root()
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    from torch.utils.cpp_extension import load
    cu = os.path.join(ref_root, "rwkv_pip_package", "src", "rwkv", "cuda")
    os.makedirs(OUT, exist_ok=True)
    jobs = [
        ("wkv_cuda_ref", ["wrapper.cpp", "operators.cu", "gemm_fp16_cublas.cpp"],
         ["--use_fast_math", "-O3", "--extra-device-vectorization"], ["-lcublas"]),
        ("rwkv5_ref", ["rwkv5_op.cpp", "rwkv5.cu"],
         ["-res-usage", "--use_fast_math", "-O3", "-Xptxas -O3", "--extra-device-vectorization", "-D_N_=64"], []),
        ("rwkv6_ref", ["rwkv6_op.cpp", "rwkv6.cu"],
         ["-res-usage", "--use_fast_math", "-O3", "-Xptxas -O3", "--extra-device-vectorization", "-D_N_=64", "-D_T_=4096"], []),
    ]
    built = []
    for name, srcs, cuflags, ld in jobs:
        so = os.path.join(OUT, name + ".so")
        if os.path.exists(so) and not force:
            built.append(so)
            continue
        bdir = os.path.join(OUT, "build_" + name)
        os.makedirs(bdir, exist_ok=True)
        load(name=name, sources=[os.path.join(cu, s) for s in srcs], extra_cuda_cflags=cuflags,
             extra_ldflags=ld, build_directory=bdir, is_python_module=False, verbose=False)
        os.replace(os.path.join(bdir, name + ".so"), so)
        shutil.rmtree(bdir, ignore_errors=True)
        built.append(so)
    built.append(stage_package(ref_root))
    return built


def build_if_reference_present(ref_root=None):
    ref_root = ref_root or default_reference_root()
    if os.path.isdir(os.path.join(ref_root, "rwkv_pip_package")):
        return build(ref_root)
    return []


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    print(build(args[0] if args else None, force="--force" in sys.argv))
