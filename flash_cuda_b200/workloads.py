"""Seeded synthetic attention problems: a general builder plus the five benchmark configurations.

Inputs are drawn on the CPU from `torch.Generator().manual_seed(seed)` in a fixed order (integer
lengths / leftpad, page permutation, Q, K, V, s_aux) so that every GPU and the CPU oracle see identical
bits.  The very large long-context pool is the one exception: it is drawn on the device (see
`long_context`), and only the slices an oracle check needs are copied back.

Layouts follow the op boundary: q (total_q, hq, hd); contiguous k/v (total_k, hkv, hd|hdv) with
cu_seqlens_k; paged k/v (num_pages, page, hkv, hd|hdv) with page_table (B, max_pages) and seqused_k.
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import List, Optional, Sequence, Tuple

import torch

_DT = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp8": torch.float8_e4m3fn}


@dataclass
class Problem:
    name: str
    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor
    cu_seqlens_q: torch.Tensor
    cu_seqlens_k: Optional[torch.Tensor]
    seqused_k: Optional[torch.Tensor]
    page_table: Optional[torch.Tensor]
    leftpad_k: Optional[torch.Tensor]
    q_descale: Optional[torch.Tensor]
    k_descale: Optional[torch.Tensor]
    v_descale: Optional[torch.Tensor]
    s_aux: Optional[torch.Tensor]
    max_seqlen_q: int
    max_seqlen_k: int
    softmax_scale: float
    causal: bool
    window_left: int = -1
    window_right: int = -1
    softcap: float = 0.0
    q_lens: List[int] = field(default_factory=list)
    k_lens: List[int] = field(default_factory=list)

    _TENSORS = ("q", "k", "v", "cu_seqlens_q", "cu_seqlens_k", "seqused_k", "page_table", "leftpad_k",
                "q_descale", "k_descale", "v_descale", "s_aux")

    def to(self, device) -> "Problem":
        return replace(self, **{n: (None if getattr(self, n) is None else getattr(self, n).to(device))
                                for n in self._TENSORS})

    def pin(self) -> "Problem":
        return replace(self, **{n: (None if getattr(self, n) is None else getattr(self, n).pin_memory())
                                for n in self._TENSORS})

    # -- argument packs --------------------------------------------------------------------
    def semantics(self) -> dict:
        return dict(softmax_scale=self.softmax_scale, causal=self.causal, window_left=self.window_left,
                    window_right=self.window_right, softcap=self.softcap)

    def tensors_kw(self) -> dict:
        return dict(cu_seqlens_q=self.cu_seqlens_q, cu_seqlens_k=self.cu_seqlens_k, seqused_k=self.seqused_k,
                    page_table=self.page_table, leftpad_k=self.leftpad_k, q_descale=self.q_descale,
                    k_descale=self.k_descale, v_descale=self.v_descale, s_aux=self.s_aux)

    def capi_kw(self) -> dict:
        """Keyword arguments of flash_cuda_b200.capi.fwd / ops.call_fwd."""
        return dict(self.tensors_kw(), max_seqlen_q=self.max_seqlen_q, max_seqlen_k=self.max_seqlen_k,
                    **self.semantics())

    def oracle_kw(self) -> dict:
        """Keyword arguments of oracle.ref_attention.ref_attention."""
        return dict(self.tensors_kw(), **self.semantics())

    # -- algorithmic work --------------------------------------------------------------------
    def unmasked_pairs(self) -> int:
        """Number of (query, key) pairs that are not masked, per q head."""
        lp = [0] * len(self.q_lens) if self.leftpad_k is None else [int(x) for x in self.leftpad_k.tolist()]
        total = 0
        for ql, kl, pad in zip(self.q_lens, self.k_lens, lp):
            qpos = torch.arange(kl - ql, kl, dtype=torch.int64)
            lo = torch.full_like(qpos, pad)
            hi = torch.full_like(qpos, kl - 1)
            if self.causal:
                hi = torch.minimum(hi, qpos)
            if self.window_right >= 0:
                hi = torch.minimum(hi, qpos + self.window_right)
            if self.window_left >= 0:
                lo = torch.maximum(lo, qpos - self.window_left)
            total += int(torch.clamp(hi - lo + 1, min=0).sum())
        return total

    def flops(self) -> float:
        hq, hd = self.q.shape[1], self.q.shape[2]
        hdv = self.v.shape[-1]
        return 2.0 * (hd + hdv) * hq * self.unmasked_pairs()

    def kv_bytes(self) -> int:
        """Bytes of K and V the unmasked keys occupy: sum_b (k_len_b - leftpad_b) * hkv * (hd + hdv) * elt."""
        lp = [0] * len(self.k_lens) if self.leftpad_k is None else [int(x) for x in self.leftpad_k.tolist()]
        hkv = self.k.shape[-2]
        hd, hdv = self.k.shape[-1], self.v.shape[-1]
        keys = sum(max(0, kl - pad) for kl, pad in zip(self.k_lens, lp))
        return keys * hkv * (hd + hdv) * self.k.element_size()


def _quant_fp8(x: torch.Tensor, descale: torch.Tensor) -> torch.Tensor:
    return (x.float() / descale).to(torch.float8_e4m3fn)


def make_problem(name: str, reqs: Sequence[Tuple[int, int]], *, hq: int, hkv: int, hd: int, hdv: Optional[int] = None,
                 dtype: str = "bf16", kv_dtype: Optional[str] = None, causal: bool = True, window_left: int = -1,
                 window_right: int = -1, softcap: float = 0.0, sink: bool = False, page_size: int = 0,
                 leftpad: Optional[Sequence[int]] = None, permute_pages: bool = True, spare_pages: int = 3,
                 fp8_scales: str = "per_head", seed: int = 0) -> Problem:
    """reqs = [(q_len, k_len), ...].  dtype in bf16|fp16|fp8 (fp8 = all of Q, K, V in e4m3 with
    descale = amax/448); kv_dtype='fp8' with a 16-bit dtype gives a 16-bit Q over an fp8 KV cache.
    fp8_scales: 'per_head' = one descale per (batch, kv head), 'tensor' = one per tensor."""
    g = torch.Generator().manual_seed(seed)
    hdv = hd if hdv is None else hdv
    q_lens = [int(a) for a, _ in reqs]
    k_lens = [int(b) for _, b in reqs]
    B = len(reqs)
    total_q = sum(q_lens)
    q_is_fp8 = dtype == "fp8"
    kv_is_fp8 = q_is_fp8 or kv_dtype == "fp8"
    gen_dt = torch.bfloat16 if q_is_fp8 else _DT[dtype]

    page_table = seqused_k = cu_k = None
    if page_size > 0:
        npages = [(kl + page_size - 1) // page_size for kl in k_lens]
        total_pages = sum(npages) + spare_pages
        perm = torch.randperm(total_pages, generator=g) if permute_pages else torch.arange(total_pages)
        page_table = torch.zeros(B, max(max(npages), 1), dtype=torch.int32)
        o = 0
        for i, n in enumerate(npages):
            page_table[i, :n] = perm[o:o + n].to(torch.int32)
            o += n
        seqused_k = torch.tensor(k_lens, dtype=torch.int32)
    q = torch.randn(total_q, hq, hd, generator=g, dtype=torch.float32)
    if page_size > 0:
        k = torch.randn(total_pages, page_size, hkv, hd, generator=g, dtype=torch.float32)
        v = torch.randn(total_pages, page_size, hkv, hdv, generator=g, dtype=torch.float32)
    else:
        total_k = sum(k_lens)
        k = torch.randn(total_k, hkv, hd, generator=g, dtype=torch.float32)
        v = torch.randn(total_k, hkv, hdv, generator=g, dtype=torch.float32)
        cu_k = torch.tensor([0] + list(torch.tensor(k_lens).cumsum(0).tolist()), dtype=torch.int32)
    s_aux = torch.randn(hq, generator=g, dtype=torch.float32).to(torch.bfloat16) if sink else None

    qd = kd = vd = None
    if kv_is_fp8:
        def scales(x, per_batch_rows):
            # descale = amax / 448 per tensor, or per (batch, kv head) over that batch's rows
            if fp8_scales == "tensor":
                return (x.abs().amax() / 448.0).reshape(1, 1).expand(B, hkv).contiguous()
            out = torch.empty(B, hkv)
            for b, rows in enumerate(per_batch_rows):
                xb = x[rows]
                out[b] = xb.abs().reshape(-1, hkv, xb.shape[-1]).amax(dim=(0, 2)) / 448.0 if xb.numel() else 1.0
            return out.clamp_min(1e-8)

        if page_size > 0:
            rows = [page_table[b, :(k_lens[b] + page_size - 1) // page_size].long() for b in range(B)]
        else:
            rows = [slice(int(cu_k[b]), int(cu_k[b + 1])) for b in range(B)]
        kd, vd = scales(k, rows), scales(v, rows)

        def apply(x, d):
            xq = torch.empty_like(x, dtype=torch.float8_e4m3fn)
            if fp8_scales == "tensor":
                return _quant_fp8(x, d[0, 0])
            xq.copy_(_quant_fp8(x, d.mean()))      # pages no sequence owns: any finite value
            for b, r in enumerate(rows):
                shape = (1, 1, hkv, 1) if page_size > 0 else (1, hkv, 1)
                xq[r] = _quant_fp8(x[r], d[b].view(shape))
            return xq

        k, v = apply(k, kd), apply(v, vd)
        if q_is_fp8:
            cu = [0] + list(torch.tensor(q_lens).cumsum(0).tolist())
            if fp8_scales == "tensor":
                qd = (q.abs().amax() / 448.0).reshape(1, 1).expand(B, hkv).contiguous()
                q = _quant_fp8(q, qd[0, 0])
            else:
                rep = hq // hkv
                qd = torch.empty(B, hkv)
                qq = torch.empty_like(q, dtype=torch.float8_e4m3fn)
                for b in range(B):
                    qb = q[cu[b]:cu[b + 1]].reshape(-1, hkv, rep, hd)
                    qd[b] = (qb.abs().amax(dim=(0, 2, 3)) / 448.0) if qb.numel() else 1.0
                    qq[cu[b]:cu[b + 1]] = _quant_fp8(qb, qd[b].clamp_min(1e-8).view(1, hkv, 1, 1)).reshape(-1, hq, hd)
                qd = qd.clamp_min(1e-8)
                q = qq
        else:
            q = q.to(gen_dt)
    else:
        q, k, v = q.to(gen_dt), k.to(gen_dt), v.to(gen_dt)

    lp = None if leftpad is None else torch.tensor([int(x) for x in leftpad], dtype=torch.int32)
    cu_q = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0).tolist()), dtype=torch.int32)
    return Problem(name=name, q=q, k=k, v=v, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k, seqused_k=seqused_k,
                   page_table=page_table, leftpad_k=lp, q_descale=qd, k_descale=kd, v_descale=vd, s_aux=s_aux,
                   max_seqlen_q=max(q_lens), max_seqlen_k=max(k_lens), softmax_scale=hd ** -0.5, causal=causal,
                   window_left=window_left, window_right=window_right, softcap=softcap, q_lens=q_lens, k_lens=k_lens)


# --------------------------------------------------------------------------------------------------
# The five benchmark configurations (scale < 1 shrinks sequence lengths / batch for quick tests).
# --------------------------------------------------------------------------------------------------
def dense_noncausal(seed: int = 0, B: int = 2, H: int = 8, S: int = 512) -> Problem:
    """Dense non-causal MHA, bf16: B=2, H=8, S_q=S_kv=512, head_dim 128."""
    return make_problem("dense_nc_b2_h8_s512", [(S, S)] * B, hq=H, hkv=H, hd=128, causal=False, seed=seed)


def causal_gqa_prefill(seed: int = 0, B: int = 4, S: int = 4096, dtype: str = "bf16") -> Problem:
    """Causal GQA prefill (Llama-3-8B-shaped): B=4, Hq=32, Hkv=8, S=4096, head_dim 128; dtype bf16 or fp8
    (fp8: per-tensor descale = amax/448)."""
    return make_problem(f"causal_gqa_prefill_{dtype}_b{B}_s{S}", [(S, S)] * B, hq=32, hkv=8, hd=128, dtype=dtype,
                        causal=True, fp8_scales="tensor", seed=seed)


def varlen_lengths(seed: int = 0, n: int = 16, lo: int = 128, hi: int = 8192) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return [int(x) for x in torch.randint(lo, hi + 1, (n,), generator=g).tolist()]


def varlen_window_softcap_sink(seed: int = 0, n: int = 16, lo: int = 128, hi: int = 8192, window: int = 4096) -> Problem:
    """Varlen packed causal prefill, bf16: 16 sequences with lengths uniform in [128, 8192], Hq=32, Hkv=8,
    head_dim 128, sliding window 4096, softcap 30, sink logits ~ N(0,1) per head."""
    lens = varlen_lengths(seed, n, lo, hi)
    return make_problem(f"varlen_n{n}_win{window}_cap30_sink", [(L, L) for L in lens], hq=32, hkv=8, hd=128,
                        causal=True, window_left=window, window_right=0, softcap=30.0, sink=True, seed=seed + 1)


def paged_decode(seed: int = 0, B: int = 128, ctx_lo: int = 1024, ctx_hi: int = 32768, kv_dtype: str = "bf16",
                 page_size: int = 64) -> Problem:
    """Paged-KV decode: batch 128, q_len 1, context uniform in [1024, 32768], page 64, block table a seeded
    random permutation of the physical pages, Hq=32, Hkv=8, head_dim 128, cache_leftpad uniform in [0, 63];
    KV cache bf16, or fp8 with a descale per (batch, kv head)."""
    g = torch.Generator().manual_seed(seed)
    ctx = torch.randint(ctx_lo, ctx_hi + 1, (B,), generator=g).tolist()
    pad = torch.randint(0, 64, (B,), generator=g).tolist()
    pad = [min(int(p), int(c) - 1) for p, c in zip(pad, ctx)]
    return make_problem(f"paged_decode_{kv_dtype}_b{B}", [(1, int(c)) for c in ctx], hq=32, hkv=8, hd=128,
                        dtype="bf16", kv_dtype=("fp8" if kv_dtype == "fp8" else None), causal=True,
                        page_size=page_size, leftpad=pad, seed=seed + 1)


def paged_decode_on_device(device, seed: int = 0, B: int = 128, ctx_lo: int = 1024, ctx_hi: int = 32768,
                           kv_dtype: str = "bf16", page_size: int = 64) -> Problem:
    """The paged-decode configuration with the KV pool drawn ON THE DEVICE (the pool is 8.5 GB in bf16; drawing
    it on the host costs 17 GB of fp32 per process, too much when 8 ranks share one host).  Lengths, leftpad and
    the page permutation are the same seeded host draws as `paged_decode`; K/V/Q values come from the device
    generator.  Returns a Problem whose tensors already live on `device`."""
    g = torch.Generator().manual_seed(seed)
    ctx = [int(c) for c in torch.randint(ctx_lo, ctx_hi + 1, (B,), generator=g).tolist()]
    pad = torch.randint(0, 64, (B,), generator=g).tolist()
    pad = [min(int(p), c - 1) for p, c in zip(pad, ctx)]
    g2 = torch.Generator().manual_seed(seed + 1)
    hq, hkv, hd = 32, 8, 128
    npages = [(c + page_size - 1) // page_size for c in ctx]
    total_pages = sum(npages) + 3
    perm = torch.randperm(total_pages, generator=g2)
    page_table = torch.zeros(B, max(npages), dtype=torch.int32)
    o = 0
    for i, n in enumerate(npages):
        page_table[i, :n] = perm[o:o + n].to(torch.int32)
        o += n
    gd = torch.Generator(device=device).manual_seed(seed * 104729 + 7)
    q = torch.randn(B, hq, hd, generator=gd, device=device, dtype=torch.float32).to(torch.bfloat16)
    k = torch.empty(total_pages, page_size, hkv, hd, device=device, dtype=torch.bfloat16)
    v = torch.empty_like(k)
    for p0 in range(0, total_pages, 2048):
        p1 = min(total_pages, p0 + 2048)
        k[p0:p1] = torch.randn(p1 - p0, page_size, hkv, hd, generator=gd, device=device, dtype=torch.bfloat16)
        v[p0:p1] = torch.randn(p1 - p0, page_size, hkv, hd, generator=gd, device=device, dtype=torch.bfloat16)
    kd = vd = None
    pt_dev = page_table.to(device)
    if kv_dtype == "fp8":
        k8 = torch.empty(k.shape, device=device, dtype=torch.float8_e4m3fn)
        v8 = torch.empty_like(k8)
        k8.copy_((k.float() / 0.01).clamp(-448, 448))      # pages no sequence owns: any finite value
        v8.copy_((v.float() / 0.01).clamp(-448, 448))
        kd = torch.empty(B, hkv, device=device, dtype=torch.float32)
        vd = torch.empty_like(kd)
        for b in range(B):
            rows = pt_dev[b, :npages[b]].long()
            for src, dst, dsc in ((k, k8, kd), (v, v8, vd)):
                xb = src[rows].float()
                d = (xb.abs().amax(dim=(0, 1, 3)) / 448.0).clamp_min(1e-8)
                dsc[b] = d
                dst[rows] = (xb / d.view(1, 1, hkv, 1)).to(torch.float8_e4m3fn)
        k, v = k8, v8
    return Problem(name=f"paged_decode_{kv_dtype}_b{B}", q=q, k=k, v=v,
                   cu_seqlens_q=torch.arange(B + 1, device=device, dtype=torch.int32), cu_seqlens_k=None,
                   seqused_k=torch.tensor(ctx, device=device, dtype=torch.int32), page_table=pt_dev,
                   leftpad_k=torch.tensor(pad, device=device, dtype=torch.int32), q_descale=None, k_descale=kd,
                   v_descale=vd, s_aux=None, max_seqlen_q=1, max_seqlen_k=max(ctx), softmax_scale=hd ** -0.5,
                   causal=True, q_lens=[1] * B, k_lens=ctx)


def long_context(device, seed: int = 0, q_len: int = 4096, k_len: int = 524288, heads: int = 128, hd: int = 192,
                 hdv: int = 128, page_size: int = 64, k_begin: int = 0, k_end: Optional[int] = None) -> Problem:
    """Long-context prefill: B=1, a chunk of q_len query rows against a paged KV of k_len tokens, Hq=Hkv=heads,
    head_dim 192 / head_dim_v 128, causal, bf16.  The pool is drawn ON THE DEVICE (it is tens of GB at full
    size); [k_begin, k_end) selects the key range one KV shard holds (pages outside it are not allocated)."""
    k_end = k_len if k_end is None else k_end
    assert k_begin % page_size == 0 and (k_end % page_size == 0 or k_end == k_len)
    g = torch.Generator(device=device).manual_seed(seed)
    q = torch.randn(q_len, heads, hd, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    n_local = k_end - k_begin
    npages = (n_local + page_size - 1) // page_size
    # each shard seeds its own slice so that a shard's pool does not depend on the shard count
    gk = torch.Generator(device=device).manual_seed(seed * 7919 + 1 + k_begin // page_size)
    k = torch.empty(npages, page_size, heads, hd, device=device, dtype=torch.bfloat16)
    v = torch.empty(npages, page_size, heads, hdv, device=device, dtype=torch.bfloat16)
    step = max(1, 256)
    for p0 in range(0, npages, step):
        p1 = min(npages, p0 + step)
        k[p0:p1] = torch.randn(p1 - p0, page_size, heads, hd, generator=gk, device=device, dtype=torch.bfloat16)
        v[p0:p1] = torch.randn(p1 - p0, page_size, heads, hdv, generator=gk, device=device, dtype=torch.bfloat16)
    page_table = torch.arange(npages, device=device, dtype=torch.int32).view(1, npages)
    return Problem(name=f"long_context_q{q_len}_k{k_len}", q=q, k=k, v=v,
                   cu_seqlens_q=torch.tensor([0, q_len], device=device, dtype=torch.int32), cu_seqlens_k=None,
                   seqused_k=torch.tensor([n_local], device=device, dtype=torch.int32), page_table=page_table,
                   leftpad_k=None, q_descale=None, k_descale=None, v_descale=None, s_aux=None, max_seqlen_q=q_len,
                   max_seqlen_k=n_local, softmax_scale=hd ** -0.5, causal=True, q_lens=[q_len], k_lens=[n_local])
