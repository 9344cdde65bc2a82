"""Host logic of the multi-GPU driver on two gloo CPU ranks: partitioning, the single all-gather, the merge.
The per-rank compute and the merge are the CPU oracle here (injected); on GPUs they are the CUDA ops."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flash_cuda_b200 import multi_gpu as MG
from flash_cuda_b200 import workloads as W
from oracle.ref_attention import combine_partials, ref_attention


def _oracle_attn(q, k, v, *, max_seqlen_q=None, max_seqlen_k=None, **kw):
    out, lse = ref_attention(q, k, v, **kw)
    return out.to(torch.bfloat16), lse


def _oracle_partial(q, k, v, *, out, lse, max_seqlen_q=None, max_seqlen_k=None, **kw):
    """Stands in for the CUDA kernel in its partial form: normalised O in fp32 and the LSE, written into the
    caller's views of the send buffer."""
    o, l = ref_attention(q, k, v, **kw)
    out.copy_(o)
    lse.copy_(l)


def _oracle_combine(o_part, lse_part, s_aux, out_dtype):
    out, lse = combine_partials(o_part, lse_part, s_aux)
    return out.to(out_dtype), lse


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mode, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        if mode == "heads":
            p = W.make_problem("mg_heads", [(40, 40), (9, 70)], hq=8, hkv=4, hd=64, causal=True, sink=True, seed=5)
            out, lse, qs = MG.fwd_head_sharded(p.q, p.k, p.v, rank=rank, world=world, attn_fn=_oracle_attn,
                                               **p.capi_kw())
            outs = [torch.empty_like(out) for _ in range(world)]
            lses = [torch.empty_like(lse) for _ in range(world)]
            dist.all_gather(outs, out.contiguous())
            dist.all_gather(lses, lse.contiguous())
            full_out, full_lse = torch.cat(outs, dim=1), torch.cat(lses, dim=0)
            ref_out, ref_lse = ref_attention(p.q, p.k, p.v, **p.oracle_kw())
            ok = (full_out.float() - ref_out).abs().max().item() < 2e-2 and torch.allclose(full_lse, ref_lse, atol=1e-5)
        else:
            # one sequence, q_len 48 against 256 keys in pages of 16; rank r owns keys [128 r, 128 r + 128)
            page, K, ql = 16, 256, 48
            p = W.make_problem("mg_kv", [(ql, K)], hq=4, hkv=2, hd=64, causal=True, page_size=page,
                               permute_pages=False, spare_pages=0, sink=(mode != "kv"), seed=9)
            per = K // world
            pages = slice(rank * per // page, (rank + 1) * per // page)
            k_loc, v_loc = p.k[pages].contiguous(), p.v[pages].contiguous()
            pt = torch.arange(per // page, dtype=torch.int32).view(1, -1)
            out, lse = MG.fwd_kv_sharded(
                p.q, k_loc, v_loc, page_table_local=pt, seqused_k_local=torch.tensor([per], dtype=torch.int32),
                cu_seqlens_q=p.cu_seqlens_q, max_seqlen_q=ql, max_seqlen_k_local=per,
                softmax_scale=p.softmax_scale, causal=True, rank=rank, world=world, partial_fn=_oracle_partial,
                combine_fn=_oracle_combine, s_aux=p.s_aux,
                merge={"kv_a2a": "all_to_all", "kv_auto": "auto"}.get(mode, "all_gather"))
            ref_out, ref_lse = ref_attention(p.q, p.k, p.v, **p.oracle_kw())
            ok = (out.float() - ref_out).abs().max().item() < 2e-2 and torch.allclose(lse, ref_lse, atol=1e-2)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_merge_form_follows_the_rank_count():
    assert MG.resolve_merge("auto", 2, 4096) == "all_gather"
    assert MG.resolve_merge("auto", 4, 4096) == "all_to_all" and MG.resolve_merge("auto", 8, 4096) == "all_to_all"
    assert MG.resolve_merge("auto", 4, 4097) == "all_gather"          # rows do not divide: one all-gather
    assert MG.resolve_merge("all_gather", 8, 4096) == "all_gather"


def test_four_rank_kv_sharding_with_the_automatic_merge():
    world = 4
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), "kv_auto", ret), nprocs=world, join=True)
    assert dict(ret) == {r: True for r in range(world)}


@pytest.mark.parametrize("mode", ["heads", "kv", "kv_sink", "kv_a2a"])
def test_two_rank_sharding_matches_single_rank(mode):
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), mode, ret), nprocs=world, join=True)
    assert dict(ret) == {0: True, 1: True}


def test_head_slice_partition():
    seen = []
    for r in range(4):
        qs, ks = MG.head_slice(32, 8, r, 4)
        assert (qs.stop - qs.start) == 8 and (ks.stop - ks.start) == 2 and qs.start == ks.start * 4
        seen += list(range(ks.start, ks.stop))
    assert seen == list(range(8))
    with pytest.raises(ValueError):
        MG.head_slice(32, 8, 0, 3)
