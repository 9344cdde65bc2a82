"""Seeded random sweep over the argument space of `fwd` against the CPU oracle: head dims, dtypes (16-bit, all-e4m3,
16-bit queries over an e4m3 cache), GQA ratios, prefill / decode / chunked / mixed batches, causal and windows,
soft cap, sink, page sizes from 1 to 256 keys, leftpad, explicit split counts.  The router decides the kernel, as
it does for a caller.  (A sweep of this kind found a stage of the e4m3 decode path that started inside a page.)"""
import random

import pytest
import torch

from flash_cuda_b200 import capi, workloads as W
from oracle.ref_attention import ref_attention

pytestmark = pytest.mark.gpu


def _draw(rng, n):
    hd, hdv = rng.choice([(64, 64), (96, 96), (128, 128), (128, 128), (192, 128), (192, 192), (256, 256)])
    dtype, kv_dtype = rng.choice(["bf16", "fp16", "bf16"]), None
    if hd == 128 and rng.random() < 0.3:
        if rng.random() < 0.5:
            dtype = "fp8"
        else:
            kv_dtype = "fp8"
    hkv = rng.choice([1, 2, 4])
    hq = hkv * rng.choice([1, 2, 4, 8])
    kind = rng.choice(["prefill", "decode", "mixed", "chunk"])
    reqs = []
    for _ in range(rng.randint(1, 4)):
        if kind == "prefill":
            q = rng.randint(1, 600)
            k = q + rng.choice([0, 0, rng.randint(0, 300)])
        elif kind == "decode":
            q = rng.randint(1, 3)
            k = rng.randint(q, 1500)
        elif kind == "chunk":
            q = rng.randint(1, 300)
            k = q + rng.randint(0, 1200)
        elif rng.random() < 0.5:
            q = rng.randint(1, 3)
            k = rng.randint(q, 900)
        else:
            q = rng.randint(100, 500)
            k = q + rng.randint(0, 200)
        reqs.append((q, k))
    causal = rng.random() < 0.8
    wl = rng.choice([-1, -1, rng.randint(0, 400)])
    wr = -1 if causal or wl < 0 else rng.choice([-1, 0, rng.randint(0, 100)])
    if causal and wl >= 0:
        wr = 0
    page = rng.choice([0, 0, 1, 2, 4, 8, 16, 32, 64, 128, 256])
    leftpad = None
    if page > 0 and rng.random() < 0.3:
        leftpad = [rng.randint(0, k - q - 1) if k > q + 1 else 0 for q, k in reqs]
    kw = dict(hq=hq, hkv=hkv, hd=hd, hdv=hdv, dtype=dtype, kv_dtype=kv_dtype, causal=causal, window_left=wl,
              window_right=wr, softcap=rng.choice([0.0, 0.0, 30.0, 5.0]), sink=rng.random() < 0.3, page_size=page,
              leftpad=leftpad, seed=1000 + n)
    extra = {"num_splits": rng.choice([2, 3])} if rng.random() < 0.3 else {}
    return reqs, kw, extra


@pytest.mark.parametrize("seed", [3, 17])
def test_random_configurations_match_the_oracle(seed, cuda_device):
    rng = random.Random(seed)
    failures = []
    for n in range(250):
        reqs, kw, extra = _draw(rng, n)
        p = W.make_problem(f"sweep{seed}_{n}", reqs, **kw)
        ref_out, ref_lse = ref_attention(p.q, p.k, p.v, **p.oracle_kw())
        pd = p.to(cuda_device)
        out, lse, _ = capi.fwd(pd.q, pd.k, pd.v, check=True, **dict(pd.capi_kw(), **extra))
        out, lse = out.float().cpu(), lse.cpu()
        tol = 6e-2 if "fp8" in (kw["dtype"], kw["kv_dtype"]) else 2e-2     # same tolerances as the fixtures
        if kw["softcap"] > 0:
            tol *= 1.5
        fin = torch.isfinite(ref_lse)
        err = (out - ref_out).abs().max().item()
        lse_err = (lse[fin] - ref_lse[fin]).abs().max().item() if fin.any() else 0.0
        if not (err <= tol and lse_err <= 2e-2 and torch.equal(torch.isfinite(lse), fin) and torch.isfinite(out).all()):
            failures.append((n, reqs, kw, extra, err, lse_err))
    assert not failures, failures[:3]


def test_random_scheduler_metadata_is_bit_exact(cuda_device):
    """Integer output: every word of the work list equals the CPU restatement, over random batches of every kind."""
    from oracle import sched_oracle as SO
    rng = random.Random(29)
    sms = torch.cuda.get_device_properties(cuda_device).multi_processor_count
    code = {torch.bfloat16: SO.DT_BF16, torch.float16: SO.DT_FP16, torch.float8_e4m3fn: SO.DT_FP8}
    for n in range(250):
        hd, hdv = rng.choice([(64, 64), (96, 96), (128, 128), (192, 128), (192, 192), (256, 256)])
        hkv = rng.choice([1, 2, 4, 8])
        hq = hkv * rng.choice([1, 2, 4, 8])
        kind = rng.choice(["prefill", "decode", "mixed"])
        q_lens, k_lens = [], []
        for _ in range(rng.randint(1, 40)):
            if kind == "prefill":
                q = rng.randint(0, 3000)
                k = q + rng.randint(0, 2000)
            elif kind == "decode":
                q, k = rng.randint(0, 4), rng.randint(0, 40000)
            elif rng.random() < 0.6:
                q, k = rng.randint(1, 3), rng.randint(1, 9000)
            else:
                q = rng.randint(100, 2000)
                k = q + rng.randint(0, 500)
            q_lens.append(q)
            k_lens.append(k)
        if max(q_lens) == 0:
            continue
        page = rng.choice([0, 1, 4, 8, 16, 64, 128, 256])
        leftpad = [rng.randint(0, max(0, k - 1)) for k in k_lens] if (page and rng.random() < 0.3) else None
        causal = rng.random() < 0.8
        wl = rng.choice([-1, -1, rng.randint(0, 3000)])
        wr = -1 if (causal or wl < 0) else rng.choice([-1, rng.randint(0, 100)])
        if causal and wl >= 0:
            wr = 0
        ns = rng.choice([0, 0, 1, 3, 8])
        dtype = rng.choice([torch.bfloat16, torch.float16] + ([torch.float8_e4m3fn] if hd == 128 else []))
        shape = dict(batch=len(q_lens), max_seqlen_q=max(q_lens), max_seqlen_k=max(max(k_lens), 1), hq=hq, hkv=hkv, hd=hd,
                     hdv=hdv, page_size=page)
        cu_q = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=cuda_device)
        md = capi.get_scheduler_metadata(
            cuda_device, dtype=dtype, seqused_k=torch.tensor(k_lens, dtype=torch.int32, device=cuda_device), cu_seqlens_q=cu_q,
            leftpad_k=None if leftpad is None else torch.tensor(leftpad, dtype=torch.int32, device=cuda_device),
            causal=causal, window_left=wl, window_right=wr, num_splits=ns, **shape)
        plan = SO.make_plan(num_sms_device=sms, q_dtype=code[dtype], num_splits=ns, **shape)
        want = SO.scheduler_metadata(plan, batch=len(q_lens), max_seqlen_q=shape["max_seqlen_q"],
                                     max_seqlen_k=shape["max_seqlen_k"], q_lens=q_lens, k_lens=k_lens, leftpad=leftpad,
                                     causal=causal, window_left=wl, window_right=wr)
        assert md.cpu().tolist() == want, (n, shape, causal, wl, wr, ns, dtype)
