"""fp32 CPU attention oracle (TEST INFRASTRUCTURE ONLY — never imported by the product path).

A restatement, in plain torch fp32 on the host, of the reference's `ref_fp32`
(bench/scenarios.py:943-1024), with the three things that function lacks and the CUDA path needs
checked:

  * a per-batch `leftpad_k` vector (the reference oracle only has one scalar, bench/scenarios.py:1003-1006;
    per-batch semantics follow kernels/fa3_hopper.cu:1084 — keys with index < leftpad_k[b] are ignored,
    the causal/window geometry is unchanged);
  * the log-sum-exp output, natural log, shape (hq, total_q), -inf for rows that see no key and no sink,
    the sink included (kernels/fa4_blackwell.cu:5942-5955, 5984);
  * evaluation of a subset of query rows / heads, so that full-size workloads can be spot-checked exactly
    without materialising the whole score matrix.

Conventions (all from bench/scenarios.py):
  q (total_q, hq, hd); non-paged k/v (total_k, hkv, hd|hdv) with cu_seqlens_k; paged k/v
  (num_pages, page, hkv, hd|hdv) with page_table (B, max_pages) int32 and seqused_k (B) (:758-776).
  Query rows of a sequence are its LAST q_len positions: qpos = k_len - q_len + row (:994).
  causal masks kpos > qpos (:998); window_left >= 0 masks kpos < qpos - wl (:1000); window_right >= 0
  masks kpos > qpos + wr (:1002).  softcap: s = cap * tanh(s / cap) after the softmax scale (:1010-1012).
  s_aux: one extra logit per q head joins the softmax and is dropped from the output (:1014-1017).
  fp8: x_fp8.float() * descale, descale per (batch, kv head) or scalar (:969-992).
  Rows with every key masked give 0 (:1020-1021).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch


def _descale(d: Optional[torch.Tensor], b: int) -> Optional[torch.Tensor]:
    """Row `b` of a (B, hkv) descale table, or the scalar; fp32 1-D (hkv) or 0-D."""
    if d is None:
        return None
    d = d.detach().to("cpu", torch.float32)
    if d.numel() == 1:
        return d.reshape(())
    return d[b]


def ref_attention(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *,
    cu_seqlens_q: torch.Tensor,
    cu_seqlens_k: Optional[torch.Tensor] = None,
    seqused_k: Optional[torch.Tensor] = None,
    page_table: Optional[torch.Tensor] = None,
    leftpad_k: Optional[torch.Tensor] = None,
    q_descale: Optional[torch.Tensor] = None,
    k_descale: Optional[torch.Tensor] = None,
    v_descale: Optional[torch.Tensor] = None,
    softmax_scale: float,
    causal: bool,
    window_left: int = -1,
    window_right: int = -1,
    softcap: float = 0.0,
    s_aux: Optional[torch.Tensor] = None,
    q_rows: Optional[Sequence[int]] = None,
    heads: Optional[Sequence[int]] = None,
    q_chunk: int = 256,
    round_to: Optional[torch.dtype] = None,
):
    """Returns (out fp32 (total_q, hq, hdv), lse fp32 (hq, total_q)).

    With `q_rows` (global row indices into q) and/or `heads` (q-head indices) only those entries are
    computed; every other entry of the returned tensors is NaN.

    `round_to` (bfloat16 / float16) turns this into the BASELINE of the reference harness' error criterion
    (bench/scenarios.py:681-687, bench/eval.py:1269-1273; there the baseline is another kernel, in the test suite
    that criterion comes from it is this: the same plain attention evaluated in the input dtype, without
    upcasting): scores, probabilities and output are each rounded to that dtype.  A kernel passes when its
    error against the fp32 result is at most twice (three times with softcap) the error of this baseline.
    """
    q = q.detach().cpu()
    k = k.detach().cpu()
    v = v.detach().cpu()
    paged = page_table is not None
    total_q, hq, hd = q.shape
    hkv = k.shape[2] if paged else k.shape[1]
    hdv = v.shape[3] if paged else v.shape[2]
    rep = hq // hkv
    cu_q = [int(x) for x in cu_seqlens_q.tolist()]
    B = len(cu_q) - 1
    if paged:
        page = k.shape[1]
        k_lens = [int(x) for x in seqused_k.tolist()]
        pt = page_table.detach().cpu().long()
    else:
        cu_k = [int(x) for x in cu_seqlens_k.tolist()]
        k_lens = [cu_k[i + 1] - cu_k[i] for i in range(B)]
        if seqused_k is not None:
            k_lens = [int(x) for x in seqused_k.tolist()]
    lp = [0] * B if leftpad_k is None else [int(x) for x in leftpad_k.tolist()]
    sink = None if s_aux is None else s_aux.detach().to("cpu", torch.float32)

    subset = (q_rows is not None) or (heads is not None)
    fill = float("nan") if subset else 0.0
    out = torch.full((total_q, hq, hdv), fill, dtype=torch.float32)
    lse = torch.full((hq, total_q), fill, dtype=torch.float32)
    head_list = list(range(hq)) if heads is None else sorted(set(int(h) for h in heads))
    kv_heads = sorted(set(h // rep for h in head_list))
    rows_sel = None if q_rows is None else torch.as_tensor(sorted(set(int(r) for r in q_rows)), dtype=torch.long)

    for b in range(B):
        q0, q1 = cu_q[b], cu_q[b + 1]
        ql, kl = q1 - q0, k_lens[b]
        if ql == 0:
            continue
        if rows_sel is None:
            rows = torch.arange(q0, q1)
        else:
            rows = rows_sel[(rows_sel >= q0) & (rows_sel < q1)]
            if rows.numel() == 0:
                continue
        qd, kd, vd = _descale(q_descale, b), _descale(k_descale, b), _descale(v_descale, b)
        for hk in kv_heads:
            hs = [h for h in head_list if h // rep == hk]
            # K, V of this (batch, kv head): (kl, hd), (kl, hdv), fp32, descaled
            if paged:
                npg = (kl + page - 1) // page
                pages = pt[b, :npg]
                Kb = k[pages, :, hk, :].to(torch.float32).reshape(npg * page, hd)[:kl]
                Vb = v[pages, :, hk, :].to(torch.float32).reshape(npg * page, hdv)[:kl]
            else:
                k0 = cu_k[b]
                Kb = k[k0:k0 + kl, hk, :].to(torch.float32)
                Vb = v[k0:k0 + kl, hk, :].to(torch.float32)
            if kd is not None:
                Kb = Kb * (kd if kd.dim() == 0 else kd[hk])
            if vd is not None:
                Vb = Vb * (vd if vd.dim() == 0 else vd[hk])
            kpos = torch.arange(kl).view(1, kl)
            for c0 in range(0, rows.numel(), q_chunk):
                rr = rows[c0:c0 + q_chunk]
                Qc = q[rr][:, hs, :].to(torch.float32)              # (n, nh, hd)
                if qd is not None:
                    Qc = Qc * (qd if qd.dim() == 0 else qd[hk])
                n = rr.numel()
                qpos = (rr - q0 + (kl - ql)).view(n, 1)
                mask = kpos >= kl                                   # all False, shape (1, kl)
                mask = mask.expand(n, kl).clone()
                if causal:
                    mask |= kpos > qpos
                if window_left >= 0:
                    mask |= kpos < (qpos - window_left)
                if window_right >= 0:
                    mask |= kpos > (qpos + window_right)
                if lp[b] > 0:
                    mask |= kpos < lp[b]
                s = torch.einsum("nhd,kd->nhk", Qc, Kb) * softmax_scale
                if round_to is not None:
                    s = s.to(round_to).to(torch.float32)
                if softcap and softcap > 0:
                    s = softcap * torch.tanh(s / softcap)
                s = s.masked_fill(mask.view(n, 1, kl), float("-inf"))
                m = s.max(dim=-1).values if kl > 0 else torch.full((n, len(hs)), float("-inf"))
                if sink is not None:
                    sk = sink[hs].view(1, len(hs))
                    m = torch.maximum(m, sk.expand_as(m))
                m_safe = torch.where(torch.isinf(m) & (m < 0), torch.zeros_like(m), m)
                p = torch.exp(s - m_safe.unsqueeze(-1))
                l = p.sum(dim=-1)
                if sink is not None:
                    l = l + torch.exp(sk - m_safe)
                inv = torch.where(l > 0, 1.0 / l, torch.zeros_like(l))
                if round_to is None:
                    o = torch.einsum("nhk,kd->nhd", p, Vb) * inv.unsqueeze(-1)
                else:
                    a = (p * inv.unsqueeze(-1)).to(round_to).to(torch.float32)
                    o = torch.einsum("nhk,kd->nhd", a, Vb).to(round_to).to(torch.float32)
                ls = torch.where(l > 0, m_safe + torch.log(l), torch.full_like(l, float("-inf")))
                out[rr.view(-1, 1), torch.tensor(hs).view(1, -1)] = o
                lse[torch.tensor(hs).view(-1, 1), rr.view(1, -1)] = ls.t()
    return out, lse


def combine_partials(o_part: torch.Tensor, lse_part: torch.Tensor, s_aux: Optional[torch.Tensor] = None):
    """CPU restatement of the split-KV merge (kernels/fa4_blackwell.cu:5964-5985).

    o_part (S, total_q, hq, hdv) fp32, each split normalised by its own denominator; lse_part
    (S, hq, total_q) fp32 natural log, -inf for a split that saw no key.  The sink joins once, here.
    Returns (out fp32 (total_q, hq, hdv), lse fp32 (hq, total_q)).
    """
    o_part = o_part.detach().to("cpu", torch.float32)
    lse_part = lse_part.detach().to("cpu", torch.float32)
    S, total_q, hq, hdv = o_part.shape
    G = lse_part.max(dim=0).values                                   # (hq, total_q)
    if s_aux is not None:
        sk = s_aux.detach().to("cpu", torch.float32).view(hq, 1)
        G = torch.maximum(G, sk.expand_as(G))
    G_safe = torch.where(torch.isinf(G) & (G < 0), torch.zeros_like(G), G)
    w = torch.exp(lse_part - G_safe.unsqueeze(0))                     # (S, hq, total_q); exp(-inf) = 0
    L = w.sum(dim=0)
    if s_aux is not None:
        L = L + torch.exp(sk - G_safe)
    # a split with weight 0 must contribute exactly 0 even when its partial holds garbage
    # (kernels/fa3_hopper.cu:3107-3111)
    wq = w.permute(0, 2, 1).unsqueeze(-1)                             # (S, total_q, hq, 1)
    acc = torch.where(wq > 0, wq * o_part, torch.zeros_like(o_part)).sum(dim=0)
    Lq = L.t().unsqueeze(-1)
    out = torch.where(Lq > 0, acc / Lq, torch.zeros_like(acc))
    lse = torch.where(L > 0, G_safe + torch.log(L), torch.full_like(L, float("-inf")))
    return out, lse
