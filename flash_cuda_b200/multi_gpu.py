"""Multi-GPU driver: one process per GPU (torch.distributed), two sharding modes.

1. `fwd_head_sharded` — (batch, kv-head) work items are independent, so each rank runs the single-GPU op on
   its contiguous block of kv heads (and the q heads that share them).  No collective on the data path; the
   output slices are disjoint.  The reference has no counterpart (its `cp_world_size` is pinned to 1,
   bench/scenarios.py:59); the independence is the one its grid already uses
   (kernels/fa4_blackwell.cu:6947: one tile per (batch, head)).

2. `fwd_kv_sharded` — long context: the key range is split evenly, rank r holds keys
   [r*K/N, (r+1)*K/N) of every sequence as its own paged pool; the queries are replicated.  Each rank's
   attention kernel writes its normalised partial O_r (fp32) and LSE_r straight into one packed send buffer
   [O_r | LSE_r]; ONE all-gather brings all partials into local memory, and the split-KV merge kernel (the maths
   of kernels/fa4_blackwell.cu:5964-5985) reads the gathered buffer in place and produces the result on every
   rank.  No staging copy sits between kernel, collective and merge.
   `merge="all_to_all"` is the variant for large rank counts: the partials are exchanged so that rank j receives
   only query rows [j*T/N, (j+1)*T/N) of every partial (1/N of the all-gather's bytes), merges that slice, and an
   all-gather of the 16-bit result rows (and of the LSE) completes the output.  `merge="auto"` (the default) takes
   the all-gather form up to 2 ranks and the all-to-all form from 4 ranks on.
   Causal masking is bottom-right aligned on the GLOBAL key count: every rank but the last sees only keys in the
   past of all queries (requires q_len <= K/N), the last rank is causal on its local length.

The compute callables are injectable so that the host logic (partitioning, buffer layout, collectives, merge) can
be tested with gloo on CPU ranks; by default they are the CUDA library's entry points and nothing else is ever
substituted.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

from . import capi


def head_slice(hq: int, hkv: int, rank: int, world: int) -> Tuple[slice, slice]:
    """Contiguous block of kv heads for `rank` and the q heads that share them."""
    if hkv % world != 0:
        raise ValueError(f"hkv={hkv} is not divisible by world={world}; shard the batch instead")
    per = hkv // world
    rep = hq // hkv
    return slice(rank * per * rep, (rank + 1) * per * rep), slice(rank * per, (rank + 1) * per)


def resolve_merge(merge: str, world: int, total_q: int) -> str:
    """"auto": one in-place all-gather up to 2 ranks; from 4 ranks on the all-to-all form, whose bytes per rank do
    not grow with the rank count (measured at 4 GPUs on the long-context shape: 0.93 ms against 1.72 ms exposed)."""
    if merge != "auto":
        return merge
    return "all_to_all" if world >= 4 and total_q % world == 0 else "all_gather"


def _default_attn():
    from . import ops
    return ops.call_fwd


def _default_partial(q, k, v, *, out, lse, **kw):
    """The attention kernel writing an fp32 partial: `out` (total_q, hq, hdv) fp32 and `lse` (hq, total_q) are views
    into the caller's send buffer."""
    capi.fwd(q, k, v, out=out, lse=lse, **kw)


def _default_combine(o_part, lse_part, s_aux, out_dtype):
    return capi.combine(o_part, lse_part, s_aux, out_dtype)


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
                   group=None, partial_fn: Optional[Callable] = None, combine_fn: Optional[Callable] = None,
                   attn_fn: Optional[Callable] = None, s_aux=None, merge: str = "auto",
                   out_dtype: Optional[torch.dtype] = None, marks: Optional[list] = None, **kw):
    """Long-context attention with the key range sharded over `world` ranks (see module docstring).
    Returns (out (total_q, hq, hdv), lse (hq, total_q)) on every rank.

    `marks`, when given, is a list that receives two CUDA events recorded on the current stream: one after the
    attention kernel, one after the merge (what lies between them is the collective plus the merge kernel)."""
    partial_fn = partial_fn or _default_partial
    combine_fn = combine_fn or _default_combine
    if causal and world > 1 and max_seqlen_q > max_seqlen_k_local:
        raise ValueError("kv sharding needs q_len <= keys per rank so that only the last rank is causal")
    local_causal = causal and rank == world - 1
    out_dtype = out_dtype or (torch.bfloat16 if q.dtype == torch.float8_e4m3fn else q.dtype)

    def mark():
        if marks is not None and q.is_cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            marks.append(ev)

    common = dict(cu_seqlens_q=cu_seqlens_q, seqused_k=seqused_k_local, page_table=page_table_local,
                  max_seqlen_q=max_seqlen_q, max_seqlen_k=max_seqlen_k_local, softmax_scale=softmax_scale,
                  causal=local_causal, **kw)
    if world == 1:
        attn_fn = attn_fn or _default_attn()
        res = attn_fn(q, k_local, v_local, s_aux=s_aux, **common)
        mark()
        mark()
        return res

    total_q, hq = q.shape[0], q.shape[1]
    hdv = v_local.shape[-1]
    merge = resolve_merge(merge, world, total_q)
    n_o, per = capi.partial_layout(total_q, hq, hdv)
    if merge == "all_gather":
        # every rank's slot of the gather buffer is its own send buffer: the kernel writes there, the collective
        # runs in place, the merge kernel reads all slots where they lie.  The sink joins exactly once, in the merge.
        gathered = torch.empty(world, per, device=q.device, dtype=torch.float32)
        o_part = gathered[:, :n_o].view(world, total_q, hq, hdv)
        lse_part = gathered[:, n_o:n_o + hq * total_q].view(world, hq, total_q)
        partial_fn(q, k_local, v_local, out=o_part[rank], lse=lse_part[rank], s_aux=None, **common)
        mark()
        dist.all_gather_into_tensor(gathered.view(-1), gathered[rank], group=group)
        res = combine_fn(o_part, lse_part, s_aux, out_dtype)
        mark()
        return res
    if merge != "all_to_all":
        raise ValueError(f"unknown merge mode {merge!r}")
    if total_q % world != 0:
        raise ValueError("merge='all_to_all' needs total_q divisible by the number of ranks")
    rows = total_q // world
    # O leaves the kernel as (total_q, hq, hdv): the rows of destination j are one contiguous block, so the
    # exchange sends straight from the kernel's output.  The LSE is (hq, total_q); its (small) per-destination
    # blocks are gathered into send order first.
    o_r = torch.empty(total_q, hq, hdv, device=q.device, dtype=torch.float32)
    lse_r = torch.empty(hq, total_q, device=q.device, dtype=torch.float32)
    partial_fn(q, k_local, v_local, out=o_r, lse=lse_r, s_aux=None, **common)
    mark()
    o_recv = torch.empty(world, rows, hq, hdv, device=q.device, dtype=torch.float32)
    dist.all_to_all_single(o_recv.view(-1), o_r.view(-1), group=group)
    lse_send = lse_r.view(hq, world, rows).permute(1, 0, 2).contiguous()
    lse_recv = torch.empty(world, hq, rows, device=q.device, dtype=torch.float32)
    dist.all_to_all_single(lse_recv.view(-1), lse_send.view(-1), group=group)
    out_j, lse_j = combine_fn(o_recv, lse_recv, s_aux, out_dtype)       # this rank's query rows
    out = torch.empty(total_q, hq, hdv, device=q.device, dtype=out_dtype)
    dist.all_gather_into_tensor(out.view(-1), out_j.contiguous().view(-1), group=group)
    lse_all = torch.empty(world, hq, rows, device=q.device, dtype=torch.float32)
    dist.all_gather_into_tensor(lse_all.view(-1), lse_j.contiguous().view(-1), group=group)
    lse = lse_all.permute(1, 0, 2).reshape(hq, total_q)
    mark()
    return out, lse
