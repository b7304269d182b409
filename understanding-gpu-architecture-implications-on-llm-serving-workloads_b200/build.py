"""Builds libb200k.so (the C-ABI library of sm_100a kernels) in-tree with nvcc.

The reference builds its kernels with torch's CUDAExtension for sm_80/sm_90
(kernels/gemm/pkg/setup.py:148-203, kernels/fmha/pkg/setup.py:161-203); here
the kernels have no torch dependency, so a plain nvcc command per translation
unit is enough and a rebuild takes seconds.

    python build.py            # build if sources are newer than the library
    python build.py --force    # rebuild everything
    python build.py --verbose  # also print ptxas resource usage (-Xptxas -v)
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OBJ_DIR = PKG_DIR / "build"
LIB_PATH = PKG_DIR / "lib" / "libb200k.so"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compiles every csrc/*.cu for sm_100a and links lib/libb200k.so."""
    nvcc = _nvcc()
    OBJ_DIR.mkdir(exist_ok=True)
    LIB_PATH.parent.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [PKG_DIR.parent / "include" / "b200k.h"]
    srcs = sources()
    jobs = []
    for src in srcs:
        obj = OBJ_DIR / (src.stem + ".o")
        if force or verbose or _stale(obj, [src] + headers):
            cmd = [nvcc, *ARCH_FLAGS, *COMMON, "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append((src, cmd))

    def run(job):
        src, cmd = job
        p = subprocess.run(cmd, capture_output=True, text=True)
        return src, p

    with ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 1))) as ex:
        for src, p in ex.map(run, jobs):
            if verbose or p.returncode != 0:
                sys.stderr.write(f"--- {src.name}\n{p.stdout}{p.stderr}")
            if p.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src.name}")
    objs = [OBJ_DIR / (s.stem + ".o") for s in srcs]
    if force or jobs or _stale(LIB_PATH, objs):
        cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(LIB_PATH), *map(str, objs)]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            sys.stderr.write(p.stdout + p.stderr)
            raise RuntimeError("link of libb200k.so failed")
    return LIB_PATH


SHIM_SRC = PKG_DIR / "torch_shim" / "ops_shim.cpp"
SHIM_PATH = PKG_DIR / "lib" / "libb200k_torch_ops.so"


def build_shim(force: bool = False) -> Path:
    """Compiles the torch-op binding (torch_shim/ops_shim.cpp: the reference's TORCH_LIBRARY schema
    blocks with CUDA implementations that forward to the C ABI) against the installed torch headers and
    links it to lib/libb200k.so.  Host C++ only (g++); about a minute because of the torch headers."""
    import torch
    from torch.utils import cpp_extension as ce
    deps = [SHIM_SRC, PKG_DIR.parent / "include" / "b200k.h", LIB_PATH]
    if not force and not _stale(SHIM_PATH, deps):
        return SHIM_PATH
    cuda_home = Path(_nvcc()).resolve().parent.parent
    torch_lib = Path(torch.__file__).resolve().parent / "lib"
    flags = ["-O2", "-std=c++17", "-fPIC", "-shared", "-w",
             f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    flags += [f"-I{p}" for p in ce.include_paths()] + [f"-I{cuda_home / 'include'}"]
    flags += [str(SHIM_SRC), "-o", str(SHIM_PATH)]
    flags += [f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
              f"-L{LIB_PATH.parent}", "-lb200k", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
    # The binding throws c10::Error through torch's frames, so it must share torch's C++ runtime
    # (libstdc++.so.6): a compiler set up to link libstdc++ statically gives a library that loads and
    # runs until the first exception crosses into torch, and then crashes.  The system g++ is tried
    # first, $CXX last, and a result without a dynamic libstdc++ is rejected.
    tried = []
    for cxx in dict.fromkeys(c for c in (os.environ.get("B200K_CXX"), "/usr/bin/g++", shutil.which("g++"),
                                          os.environ.get("CXX")) if c and Path(c).exists()):
        p = subprocess.run([cxx, *flags], capture_output=True, text=True)
        if p.returncode != 0:
            tried.append(f"{cxx}: {(p.stdout + p.stderr)[-400:]}")
            continue
        with open(SHIM_PATH, "rb") as f:
            if b"libstdc++.so.6" in f.read():
                return SHIM_PATH
        tried.append(f"{cxx}: links libstdc++ statically")
        SHIM_PATH.unlink()
    sys.stderr.write("\n".join(tried) + "\n")
    raise RuntimeError("build of libb200k_torch_ops.so failed")


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
    if "--no-shim" not in sys.argv:
        print(build_shim(force="--force" in sys.argv))
