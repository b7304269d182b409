"""Builds the reference's own NVIDIA kernel rungs for sm_100 as two torch-extension libraries,
from the sources where they lie in the reference checkout (nothing is copied into this repo):

    python oracle/build_ref_ladder.py /path/to/reference

Outputs only under oracle/_ref/ (git-ignored): ref_gemm_unified.so (finegemm_0..11) and
ref_fmha_unified.so (finefmha_0..4).  finegemm_12 (CUTLASS) and finefmha_5 (ThunderKittens) are
left out: their submodule directories are empty in the checkout.  Flags follow the reference's
setup.py (kernels/gemm/pkg/setup.py:171-189, kernels/fmha/pkg/setup.py:169-187) with the
architecture replaced by sm_100.  TEST / COMPARISON INFRASTRUCTURE ONLY: the product never loads
these; oracle/run_ref_ladder.py times them on a GPU next to the library (separate process, since
they register the same torch op namespaces).
"""
import glob
import os
import shutil
import sys

from torch.utils.cpp_extension import load

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

NVCC = ["-O3", "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__",
        "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "--expt-relaxed-constexpr", "--expt-extended-lambda", "--use_fast_math",
        "-gencode", "arch=compute_100,code=sm_100"]


def build(ref_root: str, which: str) -> str:
    pkg = os.path.join(ref_root, "kernels", which, "pkg", f"{which}_unified", "csrc")
    sources = [os.path.join(pkg, f"{which}_kernel.cu")]
    sources += sorted(glob.glob(os.path.join(pkg, "auto", "*.cu")))
    sources += sorted(glob.glob(os.path.join(pkg, "semi", "*_nv.cu")))
    name = f"ref_{which}_unified"
    build_dir = os.path.join(OUT, name + "_build")
    os.makedirs(build_dir, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    load(name=name, sources=sources, extra_cuda_cflags=NVCC + ["-std=c++20" if which == "fmha" else "-std=c++17"],
         extra_cflags=["-O3"], build_directory=build_dir, is_python_module=False, verbose=True)
    so = os.path.join(build_dir, name + ".so")
    final = os.path.join(OUT, name + ".so")
    os.replace(so, final)
    shutil.rmtree(build_dir, ignore_errors=True)  # objects and ninja files are not needed afterwards
    return final


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("REFERENCE_ROOT", "")
    if not os.path.isdir(os.path.join(root, "kernels")):
        sys.exit("usage: build_ref_ladder.py /path/to/reference [gemm] [fmha]  (or set REFERENCE_ROOT)")
    for which in (sys.argv[2:] or ["gemm", "fmha"]):
        print(build(root, which))
