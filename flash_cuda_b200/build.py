"""In-tree build of the two shared libraries (no JIT cache, so the built files travel with the tree):

  flash_cuda_b200/lib/libfa_b200.so     the C-ABI library (include/fa_b200.h): CUDA kernels + planner
  flash_cuda_b200/lib/fa_b200_torch.so  the torch-op boundary (`fwd`, `get_scheduler_metadata`), links the first

nvcc cross-compiles for sm_100a without a GPU.  `python -m flash_cuda_b200.build [--force] [-v]`.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB = os.environ.get("FA_B200_LIB_DIR") or os.path.join(PKG, "lib")   # FA_B200_LIB_DIR: use (or build into) another directory
OBJ = os.path.join(LIB, "obj")
INCLUDE = os.path.join(os.path.dirname(PKG), "include")
CAPI_SO = os.path.join(LIB, "libfa_b200.so")
TORCH_SO = os.path.join(LIB, "fa_b200_torch.so")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")

CU_SOURCES = ["fa_capi.cu", "fa_general.cu", "fa_combine.cu", "fa_decode.cu", "fa_prefill_tc.cu", "fa_append.cu"]
HEADERS = ["fa_internal.h", "fa_sched.h", "ptx.cuh"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def _digest(paths, extra=""):
    h = hashlib.sha256(extra.encode())
    for p in paths:
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _stale(target, stamp_value):
    stamp = target + ".stamp"
    if not os.path.isfile(target) or not os.path.isfile(stamp):
        return True
    with open(stamp) as f:
        return f.read().strip() != stamp_value


def _write_stamp(target, stamp_value):
    with open(target + ".stamp", "w") as f:
        f.write(stamp_value)


def _run(cmd, verbose, log=None):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log is not None:
        with open(log, "w") as f:
            f.write(r.stdout)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("build step failed: " + " ".join(cmd[:3]) + " ...")
    if verbose:
        print(r.stdout)
    return r.stdout


def build_capi(force=False, verbose=False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    hdrs = [os.path.join(CSRC, h) for h in HEADERS] + [os.path.join(INCLUDE, "fa_b200.h")]
    objs, jobs = [], []
    for src in CU_SOURCES:
        sp = os.path.join(CSRC, src)
        op = os.path.join(OBJ, src.replace(".cu", ".o"))
        objs.append(op)
        stamp = _digest([sp] + hdrs, " ".join(NVCC_FLAGS))
        if force or _stale(op, stamp):
            jobs.append((sp, op, stamp))
    if jobs:
        def one(job):
            sp, op, stamp = job
            _run([NVCC] + NVCC_FLAGS + ["-c", sp, "-o", op], verbose, log=op + ".log")
            _write_stamp(op, stamp)
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 1)) as ex:
            list(ex.map(one, jobs))
    if jobs or not os.path.isfile(CAPI_SO):
        _run([NVCC, "-shared", "-o", CAPI_SO] + objs + ["-lcudart"], verbose)
        _write_build_info(len(jobs))
    return CAPI_SO


BUILD_INFO = os.path.join(LIB, "build_info.json")


def sources_digest() -> str:
    """Digest of every source the C-ABI library is compiled from (kernels, headers, flags)."""
    paths = [os.path.join(CSRC, f) for f in CU_SOURCES + HEADERS] + [os.path.join(INCLUDE, "fa_b200.h")]
    return _digest(paths, " ".join(NVCC_FLAGS))


def _write_build_info(compiled: int) -> None:
    import json
    import time
    try:
        ver = subprocess.run([NVCC, "--version"], stdout=subprocess.PIPE, text=True).stdout.strip().splitlines()[-1]
    except Exception:
        ver = "unknown"
    with open(BUILD_INFO, "w") as f:
        json.dump({"sources_sha256": sources_digest(), "nvcc": ver, "built_at": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()),
                   "objects_compiled": compiled, "flags": NVCC_FLAGS}, f)


def build_record() -> dict:
    """What the loaded library was built from, and whether that still matches the sources in the tree: lets a
    benchmark line say which binary produced it."""
    import json
    rec = {"lib": os.path.relpath(CAPI_SO, os.path.dirname(PKG)), "present": os.path.isfile(CAPI_SO)}
    if os.path.isfile(BUILD_INFO):
        with open(BUILD_INFO) as f:
            info = json.load(f)
        rec.update(sources_sha16=info.get("sources_sha256", "")[:16], built_at=info.get("built_at"), nvcc=info.get("nvcc"),
                   matches_tree=info.get("sources_sha256") == sources_digest())
    return rec


def build_torch_op(force=False, verbose=False, namespace="_vllm_fa3_C") -> str:
    import torch
    from torch.utils.cpp_extension import include_paths

    src = os.path.join(CSRC, "torch_op.cpp")
    stamp = _digest([src, os.path.join(INCLUDE, "fa_b200.h")], namespace + torch.__version__)
    if not force and not _stale(TORCH_SO, stamp):
        return TORCH_SO
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", f"-DFA3_LIB_NAME={namespace}",
           "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=1"]
    for inc in include_paths() + [sysconfig.get_paths()["include"], os.path.join(CUDA_HOME, "include")]:
        cmd += ["-isystem", inc]
    cmd += [src, "-o", TORCH_SO, f"-L{LIB}", "-lfa_b200", f"-L{tlib}", "-lc10", "-lc10_cuda", "-ltorch_cpu",
            "-ltorch_cuda", "-ltorch", f"-L{CUDA_HOME}/lib64", "-lcudart",
            "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{tlib}"]
    _run(cmd, verbose)
    _write_stamp(TORCH_SO, stamp)
    return TORCH_SO


def build_all(force=False, verbose=False):
    return build_capi(force, verbose), build_torch_op(force, verbose)


def ptxas_report() -> str:
    """Registers / spills / shared memory per kernel, from the logs of the last compile."""
    out = []
    for src in CU_SOURCES:
        log = os.path.join(OBJ, src.replace(".cu", ".o.log"))
        if os.path.isfile(log):
            out.append("== " + src)
            with open(log) as f:
                out.append(f.read())
    return "\n".join(out)


if __name__ == "__main__":
    force = "--force" in sys.argv
    verbose = "-v" in sys.argv
    print(*build_all(force, verbose), sep="\n")
    if "--ptxas" in sys.argv:
        print(ptxas_report())
