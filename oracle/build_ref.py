"""Build recipe for the reference's own Blackwell kernel (test/bench infrastructure, not product).

Compiles `kernels/fa4_blackwell.cu` of the reference checkout, from where it lies (read-only), into
`oracle/_ref/fa4_ref.so` registering the torch-op namespace `fa4_ref`.  Flags follow the reference's
own build (bench/eval.py:122-128 nvcc flags, :225 `-DFA3_LIB_NAME`, :186-200 `-lcuda`) plus the
defines `torch.utils.cpp_extension.load` adds.  No reference source is copied into this repository;
only the built `.so` lands under `oracle/_ref/` (git-ignored).

The `.so` needs a GPU to run.  It is used by `bench.py --impl reference-kernel` (optional A/B timing of the
reference's kernel against ours on the same tensors) and by nothing else.

The reference checkout is found through `--ref`, the environment variable FA_REFERENCE_ROOT, or a directory named
`reference` beside this repository.

Usage:  python oracle/build_ref.py [--ref /path/to/reference] [--force]
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT_SO = os.path.join(OUT_DIR, "fa4_ref.so")
NAMESPACE = "fa4_ref"


def default_ref_root() -> str:
    env = os.environ.get("FA_REFERENCE_ROOT")
    return env if env else os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(ref_root: str | None = None, force: bool = False, verbose: bool = True) -> str | None:
    """Returns the path of the built library, or None when the reference checkout is absent."""
    ref_root = ref_root or default_ref_root()
    src = os.path.join(ref_root, "kernels", "fa4_blackwell.cu")
    if not os.path.isfile(src):
        return OUT_SO if os.path.isfile(OUT_SO) else None
    if os.path.isfile(OUT_SO) and not force and os.path.getmtime(OUT_SO) >= os.path.getmtime(src):
        return OUT_SO
    import torch
    from torch.utils.cpp_extension import include_paths

    os.makedirs(OUT_DIR, exist_ok=True)
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = [
        os.path.join(cuda_home, "bin", "nvcc"),
        "-O3", "-std=c++17", "--use_fast_math", "--expt-relaxed-constexpr", "--expt-extended-lambda",
        "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
        f"-DFA3_LIB_NAME={NAMESPACE}",
        "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=1",
        "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__",
        "-D__CUDA_NO_BFLOAT16_CONVERSIONS__", "-D__CUDA_NO_HALF2_OPERATORS__",
        "-shared", "-Xcompiler", "-fPIC",
    ]
    for inc in include_paths() + [sysconfig.get_paths()["include"]]:
        cmd += ["-isystem", inc]
    cmd += [src, "-o", OUT_SO, f"-L{tlib}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
            f"-L{cuda_home}/lib64/stubs", "-lcuda", f"-Xlinker", f"-rpath={tlib}"]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    return OUT_SO


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=None, help="reference checkout (default: $FA_REFERENCE_ROOT or ../reference)")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    p = build(a.ref, a.force)
    print(p if p else "reference checkout absent and no prebuilt library", file=sys.stderr)
