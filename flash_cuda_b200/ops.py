"""The torch-op boundary from Python: loads `fa_b200_torch.so`, which registers `fwd` and
`get_scheduler_metadata` with the reference's schemas (kernels/fa4_blackwell.cu:10187-10205), and mirrors
the reference harness' caller `call_fwd` (bench/scenarios.py:932-940).

There is no eager/PyTorch implementation behind these functions: if the extension cannot be loaded they raise.
"""
from __future__ import annotations

import os

import torch

from . import build as _build

NAMESPACE = "_vllm_fa3_C"
_loaded = False


def load(build_if_missing: bool = True):
    """Loads the op library (idempotent) and returns `torch.ops.<NAMESPACE>`."""
    global _loaded
    if not _loaded:
        if not (os.path.isfile(_build.TORCH_SO) and os.path.isfile(_build.CAPI_SO)):
            if not build_if_missing:
                raise RuntimeError("flash_cuda_b200 extension is not built; run `python -m flash_cuda_b200.build`")
            _build.build_all()
        torch.ops.load_library(_build.TORCH_SO)
        _loaded = True
    ns = getattr(torch.ops, NAMESPACE)
    if getattr(ns, "fwd", None) is None:
        raise RuntimeError(f"torch.ops.{NAMESPACE}.fwd is not registered")
    return ns


def fwd(*args):
    """`torch.ops._vllm_fa3_C.fwd(*args)` with the 37 positional arguments of the schema.
    Returns [out, softmax_lse, empty, empty]."""
    return load().fwd(*args)


def get_scheduler_metadata(*args):
    return load().get_scheduler_metadata(*args)


def call_fwd(q, k, v, *, cu_seqlens_q, max_seqlen_q, max_seqlen_k, softmax_scale, causal, cu_seqlens_k=None,
             seqused_k=None, page_table=None, leftpad_k=None, q_descale=None, k_descale=None, v_descale=None,
             window_left=-1, window_right=-1, softcap=0.0, s_aux=None, num_splits=0, scheduler_metadata=None,
             out=None, sm_margin=0):
    """Keyword front end that places everything in the schema's positional order; returns (out, lse)."""
    res = fwd(q, k, v, None, None, None, out, cu_seqlens_q, cu_seqlens_k, None, None, seqused_k,
              int(max_seqlen_q), int(max_seqlen_k), page_table, None, leftpad_k, None, None, None,
              q_descale, k_descale, v_descale, float(softmax_scale), bool(causal), int(window_left),
              int(window_right), float(softcap), True, scheduler_metadata, int(num_splits), None, int(sm_margin),
              s_aux, 1, 0, None)
    return res[0], res[1]
