"""Multi-GPU driver: one process per GPU (torch.distributed), two sharding modes.

1. `fwd_head_sharded` — (batch, kv-head) work items are independent, so each rank runs the single-GPU op on
   its contiguous block of kv heads (and the q heads that share them).  No collective on the data path; the
   output slices are disjoint.  The reference has no counterpart (its `cp_world_size` is pinned to 1,
   bench/scenarios.py:59); the independence is the one its grid already uses
   (kernels/fa4_blackwell.cu:6947: one tile per (batch, head)).

2. `fwd_kv_sharded` — long context: the key range is split evenly, rank r holds keys
   [r*K/N, (r+1)*K/N) of every sequence as its own paged pool; the queries are replicated.  Each rank
   computes a normalised partial O_r and LSE_r with the single-GPU op, ONE all-gather brings all partials
   into local memory, and the split-KV merge kernel (the maths of kernels/fa4_blackwell.cu:5964-5985)
   produces the result on every rank.  Causal masking is bottom-right aligned on the GLOBAL key count: every
   rank but the last sees only keys in the past of all queries (requires q_len <= K/N), the last rank is
   causal on its local length.

The compute callables are injectable so that the host logic (partitioning, gather order, merge) can be tested
with gloo on CPU ranks; by default they are the CUDA ops and nothing else is ever substituted.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def head_slice(hq: int, hkv: int, rank: int, world: int) -> Tuple[slice, slice]:
    """Contiguous block of kv heads for `rank` and the q heads that share them."""
    if hkv % world != 0:
        raise ValueError(f"hkv={hkv} is not divisible by world={world}; shard the batch instead")
    per = hkv // world
    rep = hq // hkv
    return slice(rank * per * rep, (rank + 1) * per * rep), slice(rank * per, (rank + 1) * per)


def _default_attn():
    from . import ops
    return ops.call_fwd


def _default_combine():
    from . import capi
    return capi.combine


def fwd_head_sharded(q, k, v, *, rank: int, world: int, attn_fn: Optional[Callable] = None, s_aux=None,
                     q_descale=None, k_descale=None, v_descale=None, **kw):
    """Runs this rank's share of the heads.  q (total_q, hq, hd); k/v contiguous (total_k, hkv, d) or paged
    (pages, page, hkv, d).  Returns (out_slice (total_q, hq/world, hdv), lse_slice (hq/world, total_q), q-head slice).
    The slices are views: no copy is made, the op reads them through their strides."""
    attn_fn = attn_fn or _default_attn()
    hq = q.shape[1]
    hkv = k.shape[-2]
    qs, ks = head_slice(hq, hkv, rank, world)
    qv = q[:, qs, :]
    kv_ = k[..., ks, :]
    vv = v[..., ks, :]

    def cut(d):   # (batch, hkv) descale tables follow the kv heads; scalars pass through
        return d if d is None or d.numel() == 1 else d[:, ks].contiguous()

    out, lse = attn_fn(qv, kv_, vv, s_aux=None if s_aux is None else s_aux[qs], q_descale=cut(q_descale),
                       k_descale=cut(k_descale), v_descale=cut(v_descale), **kw)
    return out, lse, qs


def fwd_kv_sharded(q, k_local, v_local, *, page_table_local, seqused_k_local, cu_seqlens_q, max_seqlen_q: int,
                   max_seqlen_k_local: int, softmax_scale: float, causal: bool, rank: int, world: int,
                   group=None, attn_fn: Optional[Callable] = None, combine_fn: Optional[Callable] = None,
                   s_aux=None, **kw):
    """Long-context attention with the key range sharded over `world` ranks (see module docstring).
    Returns (out (total_q, hq, hdv), lse (hq, total_q)) on every rank."""
    attn_fn = attn_fn or _default_attn()
    combine_fn = combine_fn or _default_combine()
    if causal and world > 1 and max_seqlen_q > max_seqlen_k_local:
        raise ValueError("kv sharding needs q_len <= keys per rank so that only the last rank is causal")
    local_causal = causal and rank == world - 1
    # the sink joins exactly once, in the merge
    out_r, lse_r = attn_fn(q, k_local, v_local, cu_seqlens_q=cu_seqlens_q, seqused_k=seqused_k_local,
                           page_table=page_table_local, max_seqlen_q=max_seqlen_q,
                           max_seqlen_k=max_seqlen_k_local, softmax_scale=softmax_scale, causal=local_causal,
                           s_aux=s_aux if world == 1 else None, **kw)
    if world == 1:
        return out_r, lse_r
    total_q, hq, hdv = out_r.shape
    # one packed buffer per rank: [O_r as fp32 | LSE_r], gathered with a single collective
    packed = torch.empty(total_q * hq * hdv + hq * total_q, device=out_r.device, dtype=torch.float32)
    packed[:total_q * hq * hdv].view(total_q, hq, hdv).copy_(out_r)
    packed[total_q * hq * hdv:].view(hq, total_q).copy_(lse_r)
    gathered = torch.empty(world * packed.numel(), device=out_r.device, dtype=torch.float32)
    dist.all_gather_into_tensor(gathered, packed, group=group)
    g = gathered.view(world, packed.numel())
    # the merge kernel wants (S, total_q, hq, hdv) and (S, hq, total_q), each contiguous
    o_part = g[:, :total_q * hq * hdv].reshape(world, total_q, hq, hdv).contiguous()
    lse_part = g[:, total_q * hq * hdv:].reshape(world, hq, total_q).contiguous()
    return combine_fn(o_part, lse_part, s_aux, out_r.dtype)
