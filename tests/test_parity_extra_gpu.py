"""More GPU parity cases, through the C ABI, against the CPU oracle:

  * the reference harness' RELATIVE error criterion (bench/scenarios.py:681-687, bench/eval.py:1269-1273):
    max|out - ref| <= mult * max|baseline - ref| + fwd_atol, mult = 2 (3 with softcap),
    fwd_atol = 2 * max|(ref + 0.3 - 0.3) - ref|, where the baseline is the plain attention evaluated in the input
    dtype (the form of the criterion that needs no second kernel);
  * shapes the router accepts that the fixtures do not reach: page sizes 1 / 2 / 4 / 8, the tensor-core prefill
    kernel over pages of 16 .. 256 keys, head_dim 192 with 192 value columns, fp16 queries over an e4m3 cache,
    decode at head_dim 64 and 192/128, a q_descale that is not 1 with 16-bit queries;
  * e4m3 prefill: full-tensor error of the tensor-core route against the oracle, with the margin asserted;
  * scheduler metadata: consumed by the prefill route, refused when it belongs to another problem;
  * the bounded-wait path: a wait that nobody satisfies ends by itself with an error code.
"""
import pytest
import torch

import _golden
from flash_cuda_b200 import capi, workloads as W
from oracle.ref_attention import ref_attention

pytestmark = pytest.mark.gpu

TC, DEC, GEN, AUTO = capi.FA_ROUTE_PREFILL_TC, capi.FA_ROUTE_DECODE, capi.FA_ROUTE_GENERAL, capi.FA_ROUTE_AUTO


def _check(p, dev, route, tol, lse_atol=5e-3, **extra):
    ref_out, ref_lse = ref_attention(p.q, p.k, p.v, **p.oracle_kw())
    pd = p.to(dev)
    out, lse, _ = capi.fwd(pd.q, pd.k, pd.v, route=route, check=True, **dict(pd.capi_kw(), **extra))
    out, lse = out.float().cpu(), lse.cpu()
    assert torch.isfinite(out).all(), p.name
    err = (out - ref_out).abs().max().item()
    assert err <= tol, f"{p.name}: max-abs error {err:.4g} > {tol}"
    fin = torch.isfinite(ref_lse)
    assert torch.equal(torch.isfinite(lse), fin), p.name
    torch.testing.assert_close(lse[fin], ref_lse[fin], atol=lse_atol, rtol=1e-2)
    return err


# ---------------------------------------------------------------------------------------------------------
# relative criterion
# ---------------------------------------------------------------------------------------------------------
SIXTEEN_BIT = [n for n in _golden.NAMES if "fp8" not in n]


@pytest.mark.parametrize("name", SIXTEEN_BIT)
def test_error_at_most_twice_the_in_dtype_baseline(name, cuda_device):
    d = _golden.load(name)
    assert d["q"].dtype in (torch.bfloat16, torch.float16) and d["k"].dtype == d["q"].dtype
    cfg = d["cfg"]
    ref = d["ref_out"]
    base, _ = ref_attention(d["q"], d["k"], d["v"], round_to=d["q"].dtype, **_golden.oracle_kwargs(d))
    kw = dict(cu_seqlens_q=d["cu_seqlens_q"], cu_seqlens_k=d["cu_seqlens_k"], seqused_k=d["seqused_k"],
              page_table=d["page_table"], leftpad_k=d["leftpad_k"], s_aux=d["s_aux"] if cfg["sink"] else None)
    kw = {n: (None if t is None else t.to(cuda_device)) for n, t in kw.items()}
    out, _, _ = capi.fwd(d["q"].to(cuda_device), d["k"].to(cuda_device), d["v"].to(cuda_device), check=True,
                         max_seqlen_q=d["max_seqlen_q"], max_seqlen_k=d["max_seqlen_k"],
                         softmax_scale=d["softmax_scale"], causal=bool(cfg["causal"]),
                         window_left=int(cfg["window_left"]), window_right=int(cfg["window_right"]),
                         softcap=float(cfg["softcap"]), num_splits=int(cfg["num_splits"]), **kw)
    mult = 3.0 if float(cfg["softcap"]) > 0 else 2.0
    fwd_atol = 2.0 * (ref + 0.3 - 0.3 - ref).abs().max().item()
    err = (out.float().cpu() - ref).abs().max().item()
    base_err = (base - ref).abs().max().item()
    assert err <= mult * base_err + fwd_atol, f"{name}: err {err:.3e} > {mult} x baseline {base_err:.3e} + {fwd_atol:.1e}"


@pytest.mark.parametrize("route", [AUTO, GEN])
def test_relative_criterion_on_benchmark_shapes(route, cuda_device):
    probs = [W.causal_gqa_prefill(B=1, S=1024), W.dense_noncausal(B=1, H=4, S=512),
             W.varlen_window_softcap_sink(n=3, lo=100, hi=700, window=256), W.paged_decode(B=8, ctx_lo=200, ctx_hi=3000)]
    for p in probs:
        ref, _ = ref_attention(p.q, p.k, p.v, **p.oracle_kw())
        base, _ = ref_attention(p.q, p.k, p.v, round_to=p.q.dtype, **p.oracle_kw())
        pd = p.to(cuda_device)
        out, _, _ = capi.fwd(pd.q, pd.k, pd.v, route=route, check=True, **pd.capi_kw())
        mult = 3.0 if p.softcap > 0 else 2.0
        err = (out.float().cpu() - ref).abs().max().item()
        base_err = (base - ref).abs().max().item()
        assert err <= mult * base_err + 2.0 * (ref + 0.3 - 0.3 - ref).abs().max().item(), (p.name, err, base_err)


# ---------------------------------------------------------------------------------------------------------
# shapes outside the fixtures
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("page_size", [1, 2, 4, 8])
def test_small_pages(page_size, cuda_device):
    """Pages smaller than a TMA box: decode-shaped and prefill-shaped batches (AUTO picks the route)."""
    dec = W.make_problem(f"small_pages_dec{page_size}", [(1, 333), (1, 64), (2, 129), (1, 1)], hq=8, hkv=2, hd=128,
                         causal=True, page_size=page_size, leftpad=[7, 0, 0, 0], sink=True, seed=41)
    pre = W.make_problem(f"small_pages_pre{page_size}", [(200, 200), (40, 300)], hq=4, hkv=2, hd=128, causal=True,
                         page_size=page_size, seed=42)
    for p in (dec, pre):
        _check(p, cuda_device, AUTO, 2e-2)


@pytest.mark.parametrize("kv_dtype", [None, "fp8"])
@pytest.mark.parametrize("page_size", [1, 2, 4, 8])
def test_decode_route_gathers_small_pages(page_size, kv_dtype, cuda_device):
    """The streaming decode kernel over pages of 1, 2 and 4 keys (rows fetched 16 bytes per lane with cp.async) and
    of 8 keys (TMA boxes), with a permuted page table, leftpad, ragged ends, several query tokens and split-KV."""
    p = W.make_problem(f"dec_gather_p{page_size}_{kv_dtype}", [(1, 1000), (2, 257), (1, 64), (1, 3), (4, 130)], hq=8,
                       hkv=2, hd=128, causal=True, page_size=page_size, leftpad=[9, 0, 0, 1, 66], kv_dtype=kv_dtype,
                       sink=True, seed=55)
    tol = 6e-2 if kv_dtype else 2e-2
    _check(p, cuda_device, DEC, tol)
    _check(p, cuda_device, DEC, tol, num_splits=3)
    _check(p, cuda_device, AUTO, tol)


@pytest.mark.parametrize("page_size", [128, 256])
def test_e4m3_cache_decode_stage_starting_inside_a_page(page_size, cuda_device):
    """An e4m3 cache is streamed in 128-key stages, but split and window boundaries fall on 64-key blocks: a stage
    may start in the middle of a page of 128 or 256 keys, and its rows must still come from the right pages."""
    p = W.make_problem(f"e4m3_midpage_{page_size}", [(2, 946), (1, 863), (3, 1210)], hq=8, hkv=2, hd=128, dtype="bf16",
                       kv_dtype="fp8", causal=True, window_left=319, window_right=0, page_size=page_size, seed=58)
    _check(p, cuda_device, AUTO, 6e-2)
    _check(p, cuda_device, DEC, 6e-2, num_splits=3)
    q = W.make_problem(f"e4m3_midpage_split_{page_size}", [(2, 584), (3, 1210)], hq=4, hkv=4, hd=128, dtype="bf16",
                       kv_dtype="fp8", causal=True, page_size=page_size, seed=59)
    _check(q, cuda_device, AUTO, 6e-2)
    _check(q, cuda_device, DEC, 6e-2, num_splits=5)


@pytest.mark.parametrize("dtype", ["bf16", "fp8"])
@pytest.mark.parametrize("page_size", [1, 4, 16])
def test_prefill_over_small_pages_read_many_times_is_de_paged(page_size, dtype, cuda_device):
    """Long query chunks over pages of 1 .. 16 keys: every key block is read by many query tiles, so the call copies
    the sequences' keys out of the pages once and runs over contiguous K/V.  Ragged lengths (the slabs' tails are
    zero-filled up to the next 128 keys), leftpad, a permuted page table, sink; with and without metadata."""
    p = W.make_problem(f"depage_{page_size}_{dtype}", [(700, 700), (300, 901), (513, 640)], hq=8, hkv=2, hd=128,
                       dtype=dtype, causal=True, page_size=page_size, leftpad=[0, 77, 0], sink=True, seed=62,
                       fp8_scales="tensor" if dtype == "fp8" else "per_head")
    tol = 6e-2 if dtype == "fp8" else 2e-2
    _check(p, cuda_device, AUTO, tol)
    _check(p, cuda_device, TC, tol, scheduler_metadata=_metadata_for(p, cuda_device))
    w = W.make_problem(f"depage_win_{page_size}_{dtype}", [(1100, 1500)], hq=4, hkv=1, hd=128, dtype=dtype, causal=True,
                       window_left=300, window_right=0, page_size=page_size, seed=63,
                       fp8_scales="tensor" if dtype == "fp8" else "per_head")
    _check(w, cuda_device, TC, tol)


@pytest.mark.parametrize("hd,hdv", [(64, 64), (192, 128)])
@pytest.mark.parametrize("page_size", [1, 4])
def test_decode_route_small_pages_other_head_dims(page_size, hd, hdv, cuda_device):
    """The cp.async producer's other row widths: 128-byte rows (head_dim 64: four rows per instruction) and 384-byte
    rows (head_dim 192: a row's chunks straddle instructions)."""
    p = W.make_problem(f"dec_small_hd{hd}_p{page_size}", [(1, 700), (2, 257), (1, 65), (1, 2)], hq=8, hkv=2, hd=hd,
                       hdv=hdv, causal=True, page_size=page_size, leftpad=[5, 0, 0, 0], seed=57)
    _check(p, cuda_device, DEC, 2e-2)
    _check(p, cuda_device, DEC, 2e-2, num_splits=2)


@pytest.mark.parametrize("page_size", [1, 2, 4, 8, 16, 32, 64, 128, 256])
@pytest.mark.parametrize("dtype", ["bf16", "fp8"])
def test_tensor_core_prefill_over_pages(page_size, dtype, cuda_device):
    """The tcgen05 prefill kernel forced onto paged KV: pages of 1, 2, 4 keys (rows gathered four at a time), pages
    that divide a 128-key tile and pages that hold one or two whole tiles; ragged lengths, a chunk (q_len < k_len)
    and leftpad."""
    p = W.make_problem(f"tc_pages_{dtype}_{page_size}", [(300, 300), (130, 700), (256, 257), (5, 1000)], hq=4, hkv=2,
                       hd=128, dtype=dtype, causal=True, page_size=page_size, leftpad=[0, 70, 0, 129], seed=43)
    _check(p, cuda_device, TC, 6e-2 if dtype == "fp8" else 2e-2)


def test_head_dim_192_with_192_value_columns(cuda_device):
    p = W.make_problem("hd192_192", [(150, 150), (33, 400)], hq=4, hkv=2, hd=192, hdv=192, causal=True, seed=44)
    _check(p, cuda_device, AUTO, 2e-2)
    pp = W.make_problem("hd192_192_paged", [(1, 500), (3, 260)], hq=4, hkv=2, hd=192, hdv=192, causal=True,
                        page_size=64, seed=45)
    _check(pp, cuda_device, AUTO, 2e-2)


@pytest.mark.parametrize("route", [AUTO, DEC, GEN])
def test_fp16_queries_over_e4m3_cache(route, cuda_device):
    p = W.make_problem("fp16q_fp8kv", [(1, 900), (2, 2100), (1, 64)], hq=16, hkv=4, hd=128, dtype="fp16",
                       kv_dtype="fp8", causal=True, page_size=64, leftpad=[3, 0, 63], sink=True, seed=46)
    _check(p, cuda_device, route, 6e-2)


@pytest.mark.parametrize("hd,hdv", [(64, 64), (192, 128)])
@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
def test_decode_route_head_dims(hd, hdv, dtype, cuda_device):
    """The streaming decode kernel at the other head dims of the reference's paged kernel
    (kernels/fa4_blackwell.cu:9958-9983), pages of 16 and 64 keys, contiguous K/V, splits."""
    for page_size in (64, 16, 0):
        p = W.make_problem(f"dec_hd{hd}_{dtype}_p{page_size}", [(1, 1000), (2, 130), (1, 64), (1, 3)], hq=8, hkv=2,
                           hd=hd, hdv=hdv, dtype=dtype, causal=True, page_size=page_size,
                           leftpad=[9, 0, 0, 1] if page_size else None, sink=True, seed=47)
        _check(p, cuda_device, DEC, 2e-2)
        _check(p, cuda_device, DEC, 2e-2, num_splits=3)
    pa = W.make_problem(f"dec_hd{hd}_auto", [(1, 3000)] * 3, hq=8, hkv=2, hd=hd, hdv=hdv, dtype=dtype, page_size=64, seed=48)
    _check(pa, cuda_device, AUTO, 2e-2)


@pytest.mark.parametrize("route", [DEC, GEN, AUTO])
def test_q_descale_with_16_bit_queries(route, cuda_device):
    """q_descale multiplies the logits whatever the type of Q (kernels/fa3_hopper.cu:101-108): every route must
    apply it, also the decode route, where Q is never e4m3."""
    p = W.make_problem("qdescale", [(1, 700), (2, 300)], hq=8, hkv=2, hd=128, kv_dtype="fp8", causal=True,
                       page_size=64, seed=49)
    qd = torch.tensor([[0.5, 1.7], [2.0, 0.25]], dtype=torch.float32)
    p.q_descale = qd
    _check(p, cuda_device, route, 6e-2)


def test_e4m3_prefill_full_tensor_error_has_margin(cuda_device):
    """All-e4m3 causal prefill on the tensor-core route (P is rounded to e4m3 for the PV product): the error over
    the WHOLE output against the fp32 oracle, not a sample.  The limit of the benchmark definition is 6e-2; the
    kernel has to stay below 4.5e-2 here so that another seed does not tip it over."""
    worst = 0.0
    for seed in (0, 1, 2):
        p = W.causal_gqa_prefill(B=1, S=1536, dtype="fp8", seed=seed)
        worst = max(worst, _check(p, cuda_device, TC, 6e-2))
    print(f"e4m3 prefill full-tensor max error over 3 seeds: {worst:.4g}")
    assert worst <= 4.5e-2


@pytest.mark.parametrize("page_size", [0, 64])
def test_mixed_decode_and_prefill_batch(page_size, cuda_device):
    """Decode-shaped sequences (1-2 new tokens) and prefill-shaped ones in one call: the library splits the batch
    between the decode kernel and the tensor-core prefill kernel (two work lists, one call); the result must not
    depend on which kernel took which sequence."""
    reqs = [(1, 900), (1, 300), (700, 700), (1, 64), (2, 1500), (300, 1200), (1, 1), (0, 40)]
    p = W.make_problem(f"mixed_p{page_size}", reqs, hq=8, hkv=2, hd=128, causal=True, page_size=page_size,
                       leftpad=[3, 0, 0, 10, 0, 100, 0, 0] if page_size else None, sink=True, seed=56)
    assert p.q.shape[0] * 4 < len(reqs) * p.max_seqlen_q        # ragged enough for the split to be chosen
    _check(p, cuda_device, AUTO, 2e-2)
    _check(p, cuda_device, TC, 2e-2)                            # forced: the prefill kernel alone gives the same


# ---------------------------------------------------------------------------------------------------------
# scheduler metadata
# ---------------------------------------------------------------------------------------------------------
def _metadata_for(p, dev, **over):
    hq, hd = p.q.shape[1], p.q.shape[2]
    paged = p.page_table is not None
    kw = dict(batch=len(p.q_lens), max_seqlen_q=p.max_seqlen_q, max_seqlen_k=p.max_seqlen_k, hq=hq,
              hkv=p.k.shape[-2], hd=hd, hdv=p.v.shape[-1], dtype=p.q.dtype,
              seqused_k=None if p.seqused_k is None else p.seqused_k.to(dev),
              cu_seqlens_q=p.cu_seqlens_q.to(dev), cu_seqlens_k=None if p.cu_seqlens_k is None else p.cu_seqlens_k.to(dev),
              leftpad_k=None if p.leftpad_k is None else p.leftpad_k.to(dev), page_size=p.k.shape[1] if paged else 0,
              causal=p.causal, window_left=p.window_left, window_right=p.window_right, has_softcap=p.softcap > 0)
    kw.update(over)
    return capi.get_scheduler_metadata(dev, **kw)


def test_prefill_route_consumes_scheduler_metadata(cuda_device):
    """Ragged batch on the tensor-core route: with the metadata the kernel walks the sorted (batch, tile) list,
    without it the arithmetic order; both give the oracle's numbers."""
    p = W.make_problem("md_prefill", [(700, 700), (30, 30), (257, 900), (0, 10), (1300, 1300)], hq=4, hkv=2, hd=128,
                       causal=True, window_left=500, window_right=0, seed=51)
    md = _metadata_for(p, cuda_device)
    assert int(md[9]) == TC and int(md[4]) == 256
    _check(p, cuda_device, TC, 2e-2)
    _check(p, cuda_device, TC, 2e-2, scheduler_metadata=md)
    _check(p, cuda_device, AUTO, 2e-2, scheduler_metadata=md)


@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
@pytest.mark.parametrize("growth", [3.0, 12.0])
def test_row_maximum_that_grows_late(growth, dtype, cuda_device):
    """Keys whose scores grow along the sequence: every 128-key block raises the row maxima, by a few log2 units
    (the lazy reference point stays) or by tens (the block's row sum exposes the stale reference point and the
    block is redone with a new one).  Non-causal, so that every block takes the prefill kernel's fast form."""
    p = W.make_problem("late_max", [(300, 1024), (128, 640)], hq=4, hkv=2, hd=128, causal=False, dtype=dtype, seed=56)
    # block j of the keys is scaled so that its largest logits sit about j * growth (natural-log units) higher
    q_rms = p.q.float().pow(2).mean().sqrt().item()
    for (k0, k1) in zip(p.cu_seqlens_k[:-1].tolist(), p.cu_seqlens_k[1:].tolist()):
        for j, b0 in enumerate(range(k0, k1, 128)):
            blk = p.k[b0:min(b0 + 128, k1)].float()
            bump = j * growth / (p.softmax_scale * q_rms * 128 ** 0.5 * 3.0)
            p.k[b0:min(b0 + 128, k1)] = (blk * (1.0 + bump)).to(p.k.dtype)
    for route in (TC, AUTO):
        _check(p, cuda_device, route, 3e-2)


def test_work_order_by_kv_head(cuda_device):
    """A K/V footprint above the L2 size switches the prefill kernel's work order to kv-head-major (arithmetic
    order and metadata list alike).  The footprint is judged from max_seqlen_k, which may be an upper bound: a large
    bound selects that order on a small problem.  The order changes which CTA computes what, not the result."""
    p = W.make_problem("kvmajor", [(700, 700), (30, 30), (257, 900), (1300, 1300)], hq=8, hkv=2, hd=128,
                       causal=True, seed=55)
    ref_out, ref_lse = ref_attention(p.q, p.k, p.v, **p.oracle_kw())
    pd = p.to(cuda_device)
    base, base_lse, _ = capi.fwd(pd.q, pd.k, pd.v, route=TC, check=True, **pd.capi_kw())
    kw = dict(pd.capi_kw(), max_seqlen_k=1 << 22)
    md = _metadata_for(p, cuda_device, max_seqlen_k=kw["max_seqlen_k"])
    assert int(md[9]) == TC
    for extra in ({}, {"scheduler_metadata": md}):
        out, lse, _ = capi.fwd(pd.q, pd.k, pd.v, route=TC, check=True, **kw, **extra)
        assert torch.equal(out, base) and torch.equal(lse, base_lse)
    assert (base.float().cpu() - ref_out).abs().max().item() <= 2e-2
    assert (base_lse.cpu() - ref_lse).abs().max().item() <= 2e-3


@pytest.mark.parametrize("reqs,page", [([(1, 0)], 0), ([(2, 0), (0, 0)], 0), ([(448, 0)], 0),     # K/V without a key
                                       ([(0, 20)], 4), ([(0, 0), (0, 5)], 16), ([(0, 191)], 256)])  # no query row
def test_batches_without_keys_or_without_queries(reqs, page, cuda_device):
    """Tensors without elements have no address.  A contiguous K/V without a single key gives zeros and the LSE of
    the sink alone (or -inf); a batch without a query row is a call that writes nothing; both leave a clean status."""
    for sink in (False, True):
        p = W.make_problem("nothing", reqs, hq=4, hkv=2, hd=128, causal=True, sink=sink, page_size=page, seed=61)
        ref_out, ref_lse = ref_attention(p.q, p.k, p.v, **p.oracle_kw())
        pd = p.to(cuda_device)
        out, lse, _ = capi.fwd(pd.q, pd.k, pd.v, check=True, **pd.capi_kw())
        assert out.shape == ref_out.shape and lse.shape == ref_lse.shape
        if out.numel():
            assert torch.equal(out.float().cpu(), ref_out)              # zeros
            fin = torch.isfinite(ref_lse)
            assert torch.equal(torch.isfinite(lse.cpu()), fin)
            torch.testing.assert_close(lse.cpu()[fin], ref_lse[fin], atol=1e-5, rtol=1e-5)


def test_metadata_is_left_unread_on_the_general_route(cuda_device):
    """The metadata call knows one element type.  For 16-bit queries over an e4m3 cache with many query rows it plans
    a tensor-core prefill, while `fwd` (which sees both types) takes the general kernel: that kernel does not read the
    list, so the call goes through with it."""
    p = W.make_problem("md_general", [(169, 437), (192, 840)], hq=8, hkv=1, hd=128, dtype="fp16", kv_dtype="fp8",
                       causal=False, sink=True, page_size=128, seed=60)
    md = _metadata_for(p, cuda_device)
    _check(p, cuda_device, AUTO, 6e-2, scheduler_metadata=md)


@pytest.mark.parametrize("kind", ["decode", "prefill"])
def test_metadata_of_another_problem_is_refused(kind, cuda_device):
    """Metadata built for batch 5 handed to a batch-3 call.  It is long enough that no read could leave the
    tensor; the kernel must still not index it: the header check records the mismatch, the kernel produces
    nothing, and the status call reports FA_ERR_BAD_METADATA."""
    if kind == "decode":
        big = W.make_problem("md5", [(1, 500)] * 5, hq=8, hkv=2, hd=128, causal=True, page_size=64, seed=52)
        small = W.make_problem("md3", [(1, 500)] * 3, hq=8, hkv=2, hd=128, causal=True, page_size=64, seed=53)
    else:
        big = W.make_problem("mp5", [(300, 300)] * 5, hq=4, hkv=2, hd=128, causal=True, seed=52)
        small = W.make_problem("mp3", [(300, 300)] * 3, hq=4, hkv=2, hd=128, causal=True, seed=53)
    md_big = _metadata_for(big, cuda_device)
    pd = small.to(cuda_device)
    # stated length: refused on the host
    with pytest.raises(capi.FaError) as ei:
        capi.fwd(pd.q, pd.k, pd.v, scheduler_metadata=md_big, **pd.capi_kw())
    assert ei.value.code == capi.FA_ERR_BAD_METADATA
    # length not stated (a binding that passes only the pointer): refused on the device
    out = torch.zeros(pd.q.shape[0], pd.q.shape[1], 128, device=cuda_device, dtype=torch.bfloat16)   # kept alive: the
    lse = torch.zeros(pd.q.shape[1], pd.q.shape[0], device=cuda_device)                              # call is asynchronous
    p_, keep = capi.make_params(pd.q, pd.k, pd.v, out, lse, scheduler_metadata=md_big, **pd.capi_kw())
    p_.scheduler_metadata_len = 0
    import ctypes as C
    lib = capi.load()
    ws = torch.empty(max(lib.fa_b200_fwd_workspace_bytes(C.byref(p_)), 256), device=cuda_device, dtype=torch.uint8)
    rc = lib.fa_b200_fwd(C.byref(p_), ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream)
    assert rc == capi.FA_OK
    with pytest.raises(capi.FaError) as ei:
        capi.check_status(ws)
    assert ei.value.code == capi.FA_ERR_BAD_METADATA, f"status detail {getattr(ei.value, 'detail', 0):#x}"
    # the library is still usable and the same call without the foreign metadata is right
    _check(small, cuda_device, AUTO, 2e-2)


def test_metadata_round_trip_same_problem_decode(cuda_device):
    p = W.paged_decode(B=9, ctx_lo=100, ctx_hi=5000)
    md = _metadata_for(p, cuda_device)
    assert int(md[9]) == DEC
    _check(p, cuda_device, AUTO, 2e-2, scheduler_metadata=md)


# ---------------------------------------------------------------------------------------------------------
# bounded waits
# ---------------------------------------------------------------------------------------------------------
def test_a_wait_nobody_satisfies_gives_up_with_an_error_code(cuda_device):
    """One thread block waits (with the wait routine of the attention kernels) on a barrier that never
    completes, with a budget of 2e5 SM cycles; it must return by itself and leave DEV_ERR_TIMEOUT with the
    self-test role in the status word.  Nothing is in flight and nothing faults; the context stays usable."""
    with torch.cuda.device(cuda_device):
        ws = capi.selftest_timeout(cuda_device, max_cycles=200_000)
        with pytest.raises(capi.FaError) as ei:
            capi.check_status(ws)
        assert ei.value.code == capi.FA_ERR_DEVICE_TIMEOUT
        assert (ei.value.detail >> 24) == 7 and (ei.value.detail & 0xFFFFFF) == 0
        # the device is fine afterwards
        p = W.causal_gqa_prefill(B=1, S=256)
        _check(p, cuda_device, AUTO, 2e-2)


def test_maxima_may_be_upper_bounds(cuda_device):
    """max_seqlen_q / max_seqlen_k are only bounds: larger values change the launch geometry, not the result."""
    p = W.make_problem("bounds", [(100, 100), (300, 400)], hq=4, hkv=2, hd=128, causal=True, seed=54)
    ref_out, _ = ref_attention(p.q, p.k, p.v, **p.oracle_kw())
    pd = p.to(cuda_device)
    kw = dict(pd.capi_kw(), max_seqlen_q=pd.q.shape[0], max_seqlen_k=pd.k.shape[0])
    for route in (AUTO, GEN):
        out, _, _ = capi.fwd(pd.q, pd.k, pd.v, route=route, check=True, **kw)
        assert (out.float().cpu() - ref_out).abs().max().item() <= 2e-2
