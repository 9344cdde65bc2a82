"""Two, four and eight real GPUs (skipped when fewer are visible): the sharded drivers give the single-GPU result.
Ranks are child processes over NCCL with NVLS off; a rank only leaves between steps."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    import torch.distributed as dist
    from flash_cuda_b200 import multi_gpu as MG, ops, workloads as W
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        ops.load(build_if_missing=False)
        # --- KV-range sharding: q 256 x k 8192, 8 heads, hd192/hdv128, causal
        q_len, k_len, heads, page = 256, 8192, 8, 64
        full = W.long_context(dev, seed=5, q_len=q_len, k_len=k_len, heads=heads)
        ref_out, ref_lse = ops.call_fwd(full.q, full.k, full.v, **full.capi_kw())
        per = k_len // world
        pages = slice(rank * per // page, (rank + 1) * per // page)
        k_loc, v_loc = full.k[pages].contiguous(), full.v[pages].contiguous()
        pt = torch.arange(per // page, device=dev, dtype=torch.int32).view(1, -1)
        ok_kv = True
        for merge in ("all_gather", "all_to_all"):
            out, lse = MG.fwd_kv_sharded(full.q, k_loc, v_loc, page_table_local=pt,
                                         seqused_k_local=torch.tensor([per], device=dev, dtype=torch.int32),
                                         cu_seqlens_q=full.cu_seqlens_q, max_seqlen_q=q_len, max_seqlen_k_local=per,
                                         softmax_scale=full.softmax_scale, causal=True, rank=rank, world=world,
                                         merge=merge)
            ok_kv = ok_kv and (out.float() - ref_out.float()).abs().max().item() <= 1e-2 and \
                (lse - ref_lse).abs().max().item() <= 2e-3
        # --- head sharding: each rank its block of kv heads, outputs are the matching slices
        p = W.make_problem("mg", [(300, 300), (40, 700)], hq=16, hkv=8, hd=128, causal=True, seed=6).to(dev)
        ref2, lse2 = ops.call_fwd(p.q, p.k, p.v, **p.capi_kw())
        o_s, l_s, qs = MG.fwd_head_sharded(p.q, p.k, p.v, rank=rank, world=world, **p.capi_kw())
        ok_h = torch.equal(o_s, ref2[:, qs, :]) and torch.allclose(l_s, lse2[qs], atol=1e-6)
        torch.cuda.synchronize()
        dist.barrier()
        ret[rank] = (bool(ok_kv), bool(ok_h))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharding_matches_single_gpu(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert dict(ret) == {r: (True, True) for r in range(world)}
