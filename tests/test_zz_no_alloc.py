"""The allocation-free decode entry point `fa_b200_decode_fwd_static`, through the C ABI.

Some callers cannot obtain device memory when they call: a serving worker whose KV-cache pool already owns all
free HBM, or a host in another language with no device allocator.  For them the library keeps the decode scratch
in an 8 MiB array of its own.  The result must match the ordinary entry point (`fa_b200_fwd`, caller workspace) on
the same inputs, call after call, because the array still holds the previous call's contents; and, so that the
comparison is not the library against itself only, it must match the CPU oracle too.

This file sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import pytest
import torch

from flash_cuda_b200 import capi, workloads as W
from oracle.ref_attention import ref_attention

pytestmark = pytest.mark.gpu


def _problems():
    # 1: split-KV (partials + work list live in the scratch); 2: a different, smaller batch right afterwards;
    # 3: fp8 cache with sink and per-batch leftpad
    return [
        (W.make_problem("na_split", [(1, 3000), (1, 700), (2, 5000)], hq=8, hkv=2, hd=128, page_size=64,
                        leftpad=[5, 0, 63], seed=21), 4),
        (W.make_problem("na_small", [(1, 200), (1, 64)], hq=8, hkv=2, hd=128, page_size=64, seed=22), 0),
        (W.make_problem("na_fp8", [(1, 900), (1, 4100)], hq=16, hkv=4, hd=128, page_size=32, kv_dtype="fp8",
                        sink=True, leftpad=[0, 31], seed=23), 2),
    ]


def test_static_scratch_decode_matches_workspace_decode(cuda_device):
    oracle = {}
    for rounds in range(2):                       # two passes: every call finds the previous call's leftovers
        for p, nsplit in _problems():
            if p.name not in oracle:
                oracle[p.name] = ref_attention(p.q, p.k, p.v, **p.oracle_kw())
            pd = p.to(cuda_device)
            kw = dict(pd.capi_kw(), num_splits=nsplit)
            ref_out, ref_lse, _ = capi.fwd(pd.q, pd.k, pd.v, route=capi.FA_ROUTE_DECODE, check=True, **kw)
            out, lse = capi.decode_fwd_static(pd.q, pd.k, pd.v, **kw)
            torch.cuda.synchronize()
            assert torch.isfinite(out.float()).all()
            assert (out.float() - ref_out.float()).abs().max().item() <= 2e-2, p.name
            fin = torch.isfinite(ref_lse)
            assert torch.equal(torch.isfinite(lse), fin)
            torch.testing.assert_close(lse[fin], ref_lse[fin], atol=5e-3, rtol=1e-2)
            # ... and against the fp32 oracle, with the tolerance of the cache type
            o_out, o_lse = oracle[p.name]
            tol = 6e-2 if p.k.dtype == torch.float8_e4m3fn else 2e-2
            assert (out.float().cpu() - o_out).abs().max().item() <= tol, p.name
            ofin = torch.isfinite(o_lse)
            torch.testing.assert_close(lse.cpu()[ofin], o_lse[ofin], atol=5e-3, rtol=1e-2)


def test_static_scratch_rejects_what_does_not_fit(cuda_device):
    # 64 splits x 64 rows x 32 heads x 128 columns of fp32 partials = 64 MiB > 8 MiB
    big = W.make_problem("na_big", [(2, 4200)] * 32, hq=32, hkv=8, hd=128, page_size=64, seed=24).to(cuda_device)
    with pytest.raises(capi.FaError) as ei:
        capi.decode_fwd_static(big.q, big.k, big.v, **dict(big.capi_kw(), num_splits=64))
    assert ei.value.code == capi.FA_ERR_STATIC_LIMIT and "8 MiB" in str(ei.value)
    # a shape the decode route does not take (head_dim 256) is refused, not rerouted
    dense = W.make_problem("na_dense", [(4, 64)], hq=4, hkv=4, hd=256, page_size=64, seed=25).to(cuda_device)
    with pytest.raises(capi.FaError) as ei:
        capi.decode_fwd_static(dense.q, dense.k, dense.v, **dense.capi_kw())
    assert ei.value.code == capi.FA_ERR_UNSUPPORTED
