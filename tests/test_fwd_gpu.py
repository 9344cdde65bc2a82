"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle and the reference's
own numbers (fixtures).  Tolerances are the ones the benchmark definition states: bf16/fp16 outputs within
max-abs 2e-2 of the fp32 reference, fp8 within 6e-2; LSE within the reference harness' LSE tolerance
(atol 5e-3, rtol 1e-2, bench/scenarios.py:695); integer outputs bit-exact."""
import pytest
import torch

import _golden
from flash_cuda_b200 import capi, workloads as W
from oracle.ref_attention import ref_attention

pytestmark = pytest.mark.gpu

TOL = {torch.bfloat16: 2e-2, torch.float16: 2e-2, torch.float8_e4m3fn: 6e-2}
ROUTES = {"auto": capi.FA_ROUTE_AUTO, "general": capi.FA_ROUTE_GENERAL, "tc": capi.FA_ROUTE_PREFILL_TC,
          "decode": capi.FA_ROUTE_DECODE}


def _tol(q, k):
    return max(TOL[q.dtype], TOL[k.dtype])


def _check(out, lse, ref_out, ref_lse, tol, what):
    out = out.float().cpu()
    assert torch.isfinite(out).all(), f"{what}: non-finite output"
    err = (out - ref_out).abs().max().item()
    assert err <= tol, f"{what}: max-abs error {err:.4g} > {tol}"
    lse = lse.cpu()
    fin = torch.isfinite(ref_lse)
    assert torch.equal(torch.isfinite(lse), fin), f"{what}: LSE finiteness pattern differs"
    assert torch.all(lse[~fin] == ref_lse[~fin]), f"{what}: LSE of empty rows must be -inf"
    torch.testing.assert_close(lse[fin], ref_lse[fin], atol=5e-3, rtol=1e-2)
    return err


def _fwd(route, *args, **kw):
    """capi.fwd; a forced route that does not take the shape skips the test (AUTO never skips)."""
    try:
        return capi.fwd(*args, route=route, **kw)
    except capi.FaError as e:
        if route != capi.FA_ROUTE_AUTO and e.code == capi.FA_ERR_UNSUPPORTED:
            pytest.skip("forced route does not take this shape")
        raise


def _run_fixture(d, dev, route, num_splits=None):
    cfg = d["cfg"]
    kw = dict(
        cu_seqlens_q=d["cu_seqlens_q"], cu_seqlens_k=d["cu_seqlens_k"], seqused_k=d["seqused_k"],
        page_table=d["page_table"], leftpad_k=d["leftpad_k"], q_descale=d["q_descale"], k_descale=d["k_descale"],
        v_descale=d["v_descale"], s_aux=d["s_aux"] if cfg["sink"] else None)
    kw = {n: (None if t is None else t.to(dev)) for n, t in kw.items()}
    out, lse, ws = _fwd(
        route, d["q"].to(dev), d["k"].to(dev), d["v"].to(dev), check=True, max_seqlen_q=d["max_seqlen_q"],
        max_seqlen_k=d["max_seqlen_k"], softmax_scale=d["softmax_scale"], causal=bool(cfg["causal"]),
        window_left=int(cfg["window_left"]), window_right=int(cfg["window_right"]), softcap=float(cfg["softcap"]),
        num_splits=int(cfg["num_splits"]) if num_splits is None else num_splits, **kw)
    return out, lse


@pytest.mark.parametrize("route", list(ROUTES))
@pytest.mark.parametrize("name", _golden.NAMES)
def test_golden_fixture(name, route, cuda_device):
    """Output against the reference's `ref_fp32` numbers; LSE against the oracle."""
    d = _golden.load(name)
    out, lse = _run_fixture(d, cuda_device, ROUTES[route])
    _, ref_lse = ref_attention(d["q"], d["k"], d["v"], **_golden.oracle_kwargs(d))
    _check(out, lse, d["ref_out"], ref_lse, _tol(d["q"], d["k"]), f"{name}/{route}")


@pytest.mark.parametrize("nsplits", [2, 3, 7])
@pytest.mark.parametrize("name", ["g_paged_decode_leftpad", "g_paged_decode_p64_sink", "g_causal_gqa_mix",
                                  "g_fp8kv_paged_decode", "g_win_cap_sink"])
def test_split_kv_matches_unsplit(name, nsplits, cuda_device):
    d = _golden.load(name)
    out, lse = _run_fixture(d, cuda_device, capi.FA_ROUTE_GENERAL, num_splits=nsplits)
    _, ref_lse = ref_attention(d["q"], d["k"], d["v"], **_golden.oracle_kwargs(d))
    _check(out, lse, d["ref_out"], ref_lse, _tol(d["q"], d["k"]), f"{name}/splits{nsplits}")


# boundary / off-by-one / tail (seqlen_q, seqlen_k) pairs the reference's edge grid lists
# (bench/scenarios.py:492-494)
EDGE_PAIRS = [(1, 1), (3, 3), (64, 1), (64, 32), (64, 128), (128, 192), (255, 256), (108, 256), (113, 128),
              (113, 211), (128, 217), (799, 3), (384, 256), (640, 128), (512, 256), (1023, 1024), (1024, 1023)]


@pytest.mark.parametrize("route", list(ROUTES))
@pytest.mark.parametrize("mode", ["causal", "noncausal", "local", "gqa"])
def test_edge_pairs(mode, route, cuda_device):
    worst = 0.0
    for i, (ql, kl) in enumerate(EDGE_PAIRS):
        kw = dict(hq=4, hkv=4, hd=128, causal=True, seed=1000 + i)
        if mode == "noncausal":
            kw["causal"] = False
        elif mode == "local":
            kw.update(hkv=1, window_left=max(1, min(ql, kl) // 3), window_right=0)
        elif mode == "gqa":
            kw.update(hkv=1)
        p = W.make_problem(f"edge_{mode}_{ql}_{kl}", [(ql, kl), (ql, kl)], **kw)
        ref_out, ref_lse = ref_attention(p.q, p.k, p.v, **p.oracle_kw())
        pd = p.to(cuda_device)
        out, lse, _ = _fwd(ROUTES[route], pd.q, pd.k, pd.v, check=True, **pd.capi_kw())
        worst = max(worst, _check(out, lse, ref_out, ref_lse, 2e-2, p.name + "/" + route))
    assert worst <= 2e-2


@pytest.mark.parametrize("route", list(ROUTES))
def test_per_batch_leftpad_and_ragged_pages(route, cuda_device):
    p = W.make_problem("leftpad_vec", [(1, 700), (1, 64), (2, 65), (1, 1), (3, 1000)], hq=8, hkv=2, hd=128,
                       page_size=64, leftpad=[63, 0, 17, 0, 640], sink=True, seed=7)
    ref_out, ref_lse = ref_attention(p.q, p.k, p.v, **p.oracle_kw())
    pd = p.to(cuda_device)
    out, lse, _ = _fwd(ROUTES[route], pd.q, pd.k, pd.v, check=True, **pd.capi_kw())
    _check(out, lse, ref_out, ref_lse, 2e-2, "leftpad_vec/" + route)


@pytest.mark.parametrize("route", list(ROUTES))
def test_empty_and_degenerate_sequences(route, cuda_device):
    """A sequence with no query rows, one with no keys, and one fully behind the leftpad."""
    p = W.make_problem("degenerate", [(0, 50), (20, 0), (4, 30), (16, 16)], hq=4, hkv=2, hd=128, causal=True,
                       page_size=16, leftpad=[0, 0, 30, 0], seed=11)
    ref_out, ref_lse = ref_attention(p.q, p.k, p.v, **p.oracle_kw())
    pd = p.to(cuda_device)
    out, lse, _ = _fwd(ROUTES[route], pd.q, pd.k, pd.v, check=True, **pd.capi_kw())
    _check(out, lse, ref_out, ref_lse, 2e-2, "degenerate/" + route)
    assert torch.all(out[:24] == 0)


@pytest.mark.parametrize("kv_dtype", [None, "fp8"])
@pytest.mark.parametrize("hq,hkv,q_lens", [
    (32, 1, [1, 1, 1]),        # MQA: 32 rows per kv head = 2 row tiles
    (16, 2, [5, 3, 1]),        # speculative decode: up to 40 rows, ragged (the last sequence has 1 tile only)
    (32, 8, [16, 7, 2]),       # 64 rows = 4 tiles, the most the route takes
])
def test_decode_route_with_several_row_tiles(hq, hkv, q_lens, kv_dtype, cuda_device):
    """rep * q_len above 16: the decode route runs one work item per 16-row tile; splits included."""
    ctx = [700, 129, 64]
    p = W.make_problem("decode_tiles", list(zip(q_lens, ctx)), hq=hq, hkv=hkv, hd=128, causal=True, page_size=64,
                       leftpad=[5, 0, 40], kv_dtype=kv_dtype, sink=True, seed=21)
    ref_out, ref_lse = ref_attention(p.q, p.k, p.v, **p.oracle_kw())
    pd = p.to(cuda_device)
    for nsplits in (1, 3):
        kw = dict(pd.capi_kw())
        kw["num_splits"] = nsplits
        out, lse, _ = capi.fwd(pd.q, pd.k, pd.v, route=capi.FA_ROUTE_DECODE, check=True, **kw)
        _check(out, lse, ref_out, ref_lse, _tol(p.q, p.k), f"decode_tiles/{hq}/{hkv}/{kv_dtype}/s{nsplits}")
    out, lse, _ = capi.fwd(pd.q, pd.k, pd.v, check=True, **pd.capi_kw())   # AUTO takes the same route
    _check(out, lse, ref_out, ref_lse, _tol(p.q, p.k), "decode_tiles/auto")


@pytest.mark.parametrize("kv_dtype", [None, "fp8"])
@pytest.mark.parametrize("page_size", [16, 32, 128, 192, 256, 320])
def test_decode_route_page_sizes(page_size, kv_dtype, cuda_device):
    p = W.make_problem("decode_pages", [(1, 1000), (2, 257), (1, 64), (1, 3)], hq=8, hkv=2, hd=128, causal=True,
                       page_size=page_size, leftpad=[9, 0, 0, 1], kv_dtype=kv_dtype, seed=31)
    ref_out, ref_lse = ref_attention(p.q, p.k, p.v, **p.oracle_kw())
    pd = p.to(cuda_device)
    out, lse, _ = capi.fwd(pd.q, pd.k, pd.v, route=capi.FA_ROUTE_DECODE, check=True, **pd.capi_kw())
    _check(out, lse, ref_out, ref_lse, _tol(p.q, p.k), f"decode_pages/{page_size}/{kv_dtype}")


def test_small_shapes_of_benchmark_configs(cuda_device):
    """Each benchmark configuration at a size the oracle finishes in seconds."""
    probs = [
        W.dense_noncausal(B=2, H=4, S=200),
        W.causal_gqa_prefill(B=2, S=300),
        W.causal_gqa_prefill(B=1, S=260, dtype="fp8"),
        W.varlen_window_softcap_sink(n=5, lo=20, hi=400, window=100),
        W.paged_decode(B=6, ctx_lo=30, ctx_hi=1500),
        W.paged_decode(B=6, ctx_lo=30, ctx_hi=1500, kv_dtype="fp8"),
    ]
    for p in probs:
        ref_out, ref_lse = ref_attention(p.q, p.k, p.v, **p.oracle_kw())
        pd = p.to(cuda_device)
        out, lse, _ = capi.fwd(pd.q, pd.k, pd.v, check=True, **pd.capi_kw())
        _check(out, lse, ref_out, ref_lse, _tol(p.q, p.k), p.name)


def test_unsupported_is_an_error_not_a_fallback(cuda_device):
    p = W.make_problem("odd_hd", [(8, 8)], hq=2, hkv=2, hd=100, seed=3).to(cuda_device)   # head_dim % 8 != 0
    with pytest.raises(capi.FaError) as ei:
        capi.fwd(p.q, p.k, p.v, **p.capi_kw())
    assert ei.value.code == capi.FA_ERR_UNSUPPORTED and "unsupported" in str(ei.value)


@pytest.mark.parametrize("case", [
    dict(reqs=[(1, 700), (1, 64), (1, 6500), (1, 1), (1, 1000), (1, 6400)], hq=8, hkv=2, page_size=64,
         leftpad=[63, 0, 17, 0, 640, 128], causal=True, wl=-1, wr=-1),
    dict(reqs=[(300, 300), (17, 900), (128, 128), (64, 64)], hq=4, hkv=4, page_size=0, leftpad=None, causal=True,
         wl=100, wr=0),
    dict(reqs=[(5, 40), (70, 333)], hq=4, hkv=1, page_size=0, leftpad=None, causal=False, wl=20, wr=11),
])
def test_scheduler_metadata_is_bit_exact(case, cuda_device):
    """Integer output: every word equals the CPU restatement."""
    from oracle import sched_oracle as SO
    reqs = case["reqs"]
    q_lens, k_lens = [a for a, _ in reqs], [b for _, b in reqs]
    B = len(reqs)
    cu_q = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=cuda_device)
    seqused = torch.tensor(k_lens, dtype=torch.int32, device=cuda_device)
    lp = None if case["leftpad"] is None else torch.tensor(case["leftpad"], dtype=torch.int32, device=cuda_device)
    shape = dict(batch=B, max_seqlen_q=max(q_lens), max_seqlen_k=max(k_lens), hq=case["hq"], hkv=case["hkv"],
                 hd=128, hdv=128, page_size=case["page_size"])
    md = capi.get_scheduler_metadata(cuda_device, dtype=torch.bfloat16, seqused_k=seqused, cu_seqlens_q=cu_q,
                                     leftpad_k=lp, causal=case["causal"], window_left=case["wl"],
                                     window_right=case["wr"], **shape)
    sms = torch.cuda.get_device_properties(cuda_device).multi_processor_count
    plan = SO.make_plan(num_sms_device=sms, **shape)
    want = SO.scheduler_metadata(plan, batch=B, max_seqlen_q=max(q_lens), max_seqlen_k=max(k_lens), q_lens=q_lens,
                                 k_lens=k_lens, leftpad=case["leftpad"], causal=case["causal"],
                                 window_left=case["wl"], window_right=case["wr"])
    assert md.cpu().tolist() == want
