"""CPU restatement (TEST INFRASTRUCTURE ONLY) of the step in front of attention when the op is given `k_new` / `v_new`
and a rotary table: append to the paged cache in place, rotate the new keys and the queries.

Parity unpinned against the reference: it pins these arguments of the op to None (bench/scenarios.py:915-921) and holds
no kernel, test or vector for them.  What is restated is the op's documented behaviour: new key i of sequence b goes to
key index seqused_k[b] + i and is rotated at position r_b + i (r_b = seqlens_rotary[b] if given, else seqused_k[b]);
query i is rotated at r_b + i under causal / windowed attention and at r_b otherwise; interleaved pairs dimensions
(2j, 2j+1), otherwise (j, j + rotary_dim/2); dimensions >= rotary_dim pass through.  Arithmetic in fp32 with each
product and sum rounded on its own (torch elementwise ops), result rounded to the element type: the CUDA kernel is
written to give the same bits.
"""
from __future__ import annotations

from typing import Optional

import torch


def rotate_rows(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pos: torch.Tensor, interleaved: bool) -> torch.Tensor:
    """x (n, heads, hd) of a 16-bit type, cos/sin (seqlen_ro, rd/2) of the same type, pos (n) int64 -> rotated x."""
    rd = 2 * cos.shape[1]
    xf = x.to(torch.float32)
    c = cos.to(torch.float32)[pos].unsqueeze(1)   # (n, 1, rd/2)
    s = sin.to(torch.float32)[pos].unsqueeze(1)
    out = xf.clone()
    if interleaved:
        x1, x2 = xf[..., 0:rd:2], xf[..., 1:rd:2]
        out[..., 0:rd:2] = x1 * c - x2 * s
        out[..., 1:rd:2] = x1 * s + x2 * c
    else:
        x1, x2 = xf[..., :rd // 2], xf[..., rd // 2:rd]
        out[..., :rd // 2] = x1 * c - x2 * s
        out[..., rd // 2:rd] = x1 * s + x2 * c
    return out.to(x.dtype)


def append_kv_reference(k_new, v_new, k_cache, v_cache, *, page_table, seqused_k, cu_seqlens_k_new, q=None,
                        cu_seqlens_q=None, rotary_cos=None, rotary_sin=None, seqlens_rotary=None,
                        rotary_interleaved: bool = True, q_positions_advance: bool = True):
    """Returns (q_rotated or q, k_cache', v_cache', seqused_k') — fresh tensors, the inputs are not modified."""
    k_cache, v_cache = k_cache.clone(), v_cache.clone()
    page = k_cache.shape[1]
    B = seqused_k.numel()
    cu_n = [int(x) for x in cu_seqlens_k_new.tolist()]
    used = [int(x) for x in seqused_k.tolist()]
    base = used if seqlens_rotary is None else [int(x) for x in seqlens_rotary.tolist()]
    rot = rotary_cos is not None
    q_out = q
    if rot:
        q_out = q.clone()
        cu_q = [int(x) for x in cu_seqlens_q.tolist()]
    for b in range(B):
        n0, n1 = cu_n[b], cu_n[b + 1]
        if n1 > n0:
            kb, vb = k_new[n0:n1], v_new[n0:n1]
            if rot:
                kb = rotate_rows(kb, rotary_cos, rotary_sin, base[b] + torch.arange(n1 - n0), rotary_interleaved)
            for i in range(n1 - n0):
                kidx = used[b] + i
                pg = int(page_table[b, kidx // page])
                k_cache[pg, kidx % page] = kb[i]
                v_cache[pg, kidx % page] = vb[i]
        if rot and cu_q[b + 1] > cu_q[b]:
            ql = cu_q[b + 1] - cu_q[b]
            pos = base[b] + (torch.arange(ql) if q_positions_advance else torch.zeros(ql, dtype=torch.long))
            q_out[cu_q[b]:cu_q[b + 1]] = rotate_rows(q[cu_q[b]:cu_q[b + 1]], rotary_cos, rotary_sin, pos, rotary_interleaved)
    seq_out = torch.tensor([used[b] + cu_n[b + 1] - cu_n[b] for b in range(B)], dtype=torch.int32)
    return q_out, k_cache, v_cache, seq_out
