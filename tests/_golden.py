"""Loader for the fixtures under tests/golden/ (made by tests/golden/make_golden.py)."""
from __future__ import annotations

import json
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

with open(os.path.join(GOLDEN_DIR, "INDEX.json")) as _f:
    NAMES = json.load(_f)

_T = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float8_e4m3fn": torch.float8_e4m3fn}
_TENSORS = ("q", "k", "v", "cu_seqlens_q", "cu_seqlens_k", "seqused_k", "page_table",
            "q_descale", "k_descale", "v_descale", "s_aux", "leftpad_k")


def load(name: str) -> dict:
    """Returns {'cfg': dict, 'ref_out': fp32 tensor, 'softmax_scale', 'max_seqlen_q/k', <input tensors or None>}."""
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    meta = json.loads(bytes(z["meta"]).decode())
    d = {"cfg": meta["cfg"], "softmax_scale": meta["softmax_scale"],
         "max_seqlen_q": meta["max_seqlen_q"], "max_seqlen_k": meta["max_seqlen_k"],
         "ref_out": torch.from_numpy(z["ref_out"].copy())}
    for n in _TENSORS:
        if n not in z.files:
            d[n] = None
            continue
        t = torch.from_numpy(z[n].copy())
        dt = meta["dtypes"][n]
        if dt in _T:
            t = t.view(_T[dt])
        d[n] = t
    return d


def oracle_kwargs(d: dict) -> dict:
    """Keyword arguments of oracle.ref_attention.ref_attention for a loaded fixture."""
    cfg = d["cfg"]
    return dict(
        cu_seqlens_q=d["cu_seqlens_q"], cu_seqlens_k=d["cu_seqlens_k"], seqused_k=d["seqused_k"],
        page_table=d["page_table"], leftpad_k=d["leftpad_k"],
        q_descale=d["q_descale"], k_descale=d["k_descale"], v_descale=d["v_descale"],
        softmax_scale=d["softmax_scale"], causal=bool(cfg["causal"]),
        window_left=int(cfg["window_left"]), window_right=int(cfg["window_right"]),
        softcap=float(cfg["softcap"]), s_aux=d["s_aux"] if cfg["sink"] else None,
    )


def fwd_args(d: dict, device, out=None, num_splits=None, scheduler_metadata=None) -> tuple:
    """The 37 positional arguments of the `fwd` op, in the order the reference's harness passes them
    (bench/scenarios.py:910-929)."""
    cfg = d["cfg"]

    def dev(t):
        return None if t is None else t.to(device)

    return (
        dev(d["q"]), dev(d["k"]), dev(d["v"]),
        None, None, None,
        out,
        dev(d["cu_seqlens_q"]), dev(d["cu_seqlens_k"]), None,
        None, dev(d["seqused_k"]),
        d["max_seqlen_q"], d["max_seqlen_k"],
        dev(d["page_table"]), None, dev(d["leftpad_k"]),
        None, None, None,
        dev(d["q_descale"]), dev(d["k_descale"]), dev(d["v_descale"]),
        d["softmax_scale"], bool(cfg["causal"]),
        int(cfg["window_left"]), int(cfg["window_right"]),
        float(cfg["softcap"]), True,
        scheduler_metadata, int(cfg["num_splits"] if num_splits is None else num_splits), None,
        0,
        dev(d["s_aux"]) if cfg["sink"] else None, 1, 0, None,
    )
