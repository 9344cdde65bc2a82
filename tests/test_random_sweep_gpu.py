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
