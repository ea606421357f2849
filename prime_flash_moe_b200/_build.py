"""In-tree build of the native libraries (no JIT cache, no pip install).

* ``_lib/libpmoe_b200.so``  - CUDA kernels + C ABI (``include/pmoe_b200.h``), built with nvcc for
  ``sm_100a`` only. No torch dependency.
* ``_C.so``                  - the TORCH_LIBRARY binding (``csrc/torch_binding.cpp``), linked against
  ``libpmoe_b200.so`` and libtorch.

``python prime_flash_moe_b200/_build.py`` builds both (run as a script: importing the package needs the
libraries to exist already); targets newer than their sources are kept.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "_lib"
OBJ_DIR = PKG / "_lib" / "obj"
NATIVE_LIB = LIB_DIR / "libpmoe_b200.so"
TORCH_EXT = PKG / "_C.so"

CUDA_SOURCES = ["host_common.cu", "moe_align.cu", "moe_bf16.cu", "moe_mxfp8.cu", "moe_ep.cu", "moe_pre.cu",
                "moe_bwd_bf16.cu"]
NVCC_FLAGS = [
    "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; the native library cannot be built")
    return cand


def _newer(target: Path, deps) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(Path(d).stat().st_mtime <= t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print("+", " ".join(str(c) for c in cmd), flush=True)
    r = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(str(c) for c in cmd)}\n{r.stdout}\n{r.stderr}")
    if verbose and (r.stdout or r.stderr):
        print(r.stdout, r.stderr, flush=True)


def build_native(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [ROOT / "include" / "pmoe_b200.h"]
    sources = [CSRC / s for s in CUDA_SOURCES]
    if not force and _newer(NATIVE_LIB, sources + headers):
        return NATIVE_LIB
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    nvcc = _nvcc()
    extra = ["-Xptxas", "-v"] if ptxas_info else []

    def compile_one(src: Path) -> Path:
        obj = OBJ_DIR / (src.stem + ".o")
        if force or not _newer(obj, [src] + headers):
            _run([nvcc, *NVCC_FLAGS, *extra, "-c", src, "-o", obj], verbose or ptxas_info)
        return obj

    with ThreadPoolExecutor(max_workers=4) as ex:
        objs = list(ex.map(compile_one, sources))
    _run([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", NATIVE_LIB, *objs], verbose)
    return NATIVE_LIB


def build_torch_binding(force: bool = False, verbose: bool = False) -> Path:
    build_native(force=False, verbose=verbose)
    src = CSRC / "torch_binding.cpp"
    deps = [src, ROOT / "include" / "pmoe_b200.h", NATIVE_LIB]
    if not force and _newer(TORCH_EXT, deps):
        return TORCH_EXT
    import torch
    from torch.utils import cpp_extension as ce

    inc = [f"-I{p}" for p in ce.include_paths()]
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    inc.append(f"-I{cuda_home}/include")
    torch_lib = Path(torch.__file__).parent / "lib"
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = [
        os.environ.get("CXX", "g++"), "-std=c++17", "-O2", "-fPIC", "-shared", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
        *inc, src, "-o", TORCH_EXT,
        f"-L{LIB_DIR}", "-lpmoe_b200", f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda",
        "-lc10_cuda", "-Wl,-rpath,$ORIGIN/_lib", f"-Wl,-rpath,{torch_lib}", "-Wl,--no-as-needed",
    ]
    _run(cmd, verbose)
    return TORCH_EXT


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_native(force=force, verbose=verbose)
    build_torch_binding(force=force, verbose=verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
