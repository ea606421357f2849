"""Build the test-side native pieces under ``oracle/``. TEST INFRASTRUCTURE ONLY.

* ``oracle/_build/liboracle_c.so`` - the plain-C restatement ``oracle/moe_oracle_c.c`` (gcc).
* ``oracle/_ref/libprime_moe_ref.so`` - the REFERENCE's own sm_100a kernels, compiled by nvcc from
  the two ``.cu`` files where they lie in the reference checkout (nothing is copied), plus
  ``oracle/ref_shim.cu``. Only built when the reference checkout is present; the output directory is
  git-ignored and travels to a GPU machine as a prebuilt file.

    python oracle/build_ref.py /path/to/prime-flash-moe      (or PMOE_REFERENCE_ROOT=/path/to/prime-flash-moe)

Without a path (argument or environment variable) only the C restatement is built and a prebuilt
``oracle/_ref`` library, if present, is used as it is.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_OUT = HERE / "_ref" / "libprime_moe_ref.so"
C_OUT = HERE / "_build" / "liboracle_c.so"
def _default_ref():
    """The reference checkout named by PMOE_REFERENCE_ROOT, else a checkout called ``reference`` beside this
    repository if there is one, else None (a prebuilt library is then used as it is)."""
    env = os.environ.get("PMOE_REFERENCE_ROOT")
    if env:
        return Path(env)
    beside = HERE.parent.parent / "reference"
    return beside if (beside / "prime_moe" / "csrc" / "kernels").exists() else None


def _run(cmd):
    r = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"{' '.join(str(c) for c in cmd)}\n{r.stdout}\n{r.stderr}")


def _stale(target: Path, deps) -> bool:
    return not target.exists() or any(Path(d).stat().st_mtime > target.stat().st_mtime for d in deps)


def build_c_oracle() -> Path:
    src = HERE / "moe_oracle_c.c"
    if _stale(C_OUT, [src]):
        C_OUT.parent.mkdir(exist_ok=True)
        _run([os.environ.get("CC", "gcc"), "-O2", "-std=c11", "-shared", "-fPIC", src, "-o", C_OUT, "-lm"])
    return C_OUT


def build_reference(ref_root=None):
    """Returns the library path, or None when neither the reference checkout nor a prebuilt library is available."""
    ref_root = Path(ref_root) if ref_root else _default_ref()
    if ref_root is None:
        return REF_OUT if REF_OUT.exists() else None
    kdir = ref_root / "prime_moe" / "csrc" / "kernels"
    srcs = [kdir / "fused_moe_bf16_kernel.cu", kdir / "fused_moe_mxfp8_kernel.cu"]
    if not all(s.exists() for s in srcs):
        return REF_OUT if REF_OUT.exists() else None
    shim = HERE / "ref_shim.cu"
    if _stale(REF_OUT, srcs + [shim, kdir / "tcgen05_prelude.cuh"]):
        REF_OUT.parent.mkdir(exist_ok=True)
        nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
        _run([nvcc, "-std=c++20", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-shared",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", *srcs, shim, "-o", REF_OUT])
    return REF_OUT


if __name__ == "__main__":
    print(build_c_oracle())
    print(build_reference(sys.argv[1] if len(sys.argv) > 1 else None))
