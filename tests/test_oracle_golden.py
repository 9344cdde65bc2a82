"""The CPU oracle against the reference's own numbers (fixtures made from the reference's `ref_fp32`)."""
import pytest
import torch

import _golden
from oracle.ref_attention import ref_attention, combine_partials


@pytest.mark.parametrize("name", _golden.NAMES)
def test_oracle_matches_reference_fixture(name):
    d = _golden.load(name)
    out, lse = ref_attention(d["q"], d["k"], d["v"], **_golden.oracle_kwargs(d))
    ref = d["ref_out"]
    assert out.shape == ref.shape
    # both are fp32 evaluations of the same formula; only summation order differs
    torch.testing.assert_close(out, ref, atol=2e-5, rtol=1e-4)
    assert lse.shape == (d["q"].shape[1], d["q"].shape[0])
    assert not torch.isnan(lse).any()


def test_oracle_row_subset_is_exact_restriction():
    d = _golden.load("g_win_cap_sink")
    kw = _golden.oracle_kwargs(d)
    full, lse_full = ref_attention(d["q"], d["k"], d["v"], **kw)
    rows, heads = [0, 5, 59, 60, 83, 100], [1, 2]
    sub, lse_sub = ref_attention(d["q"], d["k"], d["v"], q_rows=rows, heads=heads, **kw)
    for r in rows:
        for h in heads:
            torch.testing.assert_close(sub[r, h], full[r, h], atol=1e-6, rtol=1e-6)
            torch.testing.assert_close(lse_sub[h, r], lse_full[h, r], atol=1e-6, rtol=1e-6)
    assert torch.isnan(sub[1, 1]).all() and torch.isnan(sub[0, 0]).all()


def test_oracle_lse_is_logsumexp_and_empty_rows():
    # causal with q_len > k_len: the first q_len-k_len rows see no key -> out 0, lse -inf
    d = _golden.load("g_causal_q_gt_k")
    out, lse = ref_attention(d["q"], d["k"], d["v"], **_golden.oracle_kwargs(d))
    assert torch.all(out[:17] == 0) and torch.all(torch.isinf(lse[:, :17]) & (lse[:, :17] < 0))
    assert torch.isfinite(lse[:, 17:50]).all()
    # direct check of one row
    q, k = d["q"].float(), d["k"].float()
    s = (q[49, 1] @ k[:33, 1].t()) * d["softmax_scale"]
    torch.testing.assert_close(lse[1, 49], torch.logsumexp(s, 0), atol=1e-5, rtol=1e-5)


def test_per_batch_leftpad_vector():
    d = _golden.load("g_paged_decode_leftpad")
    kw = _golden.oracle_kwargs(d)
    base, _ = ref_attention(d["q"], d["k"], d["v"], **kw)
    kw2 = dict(kw)
    kw2["leftpad_k"] = torch.tensor([5, 0, 5, 7], dtype=torch.int32)
    out2, _ = ref_attention(d["q"], d["k"], d["v"], **kw2)
    torch.testing.assert_close(out2[0], base[0])
    torch.testing.assert_close(out2[2], base[2])
    assert not torch.allclose(out2[1], base[1]) and not torch.allclose(out2[3], base[3])


def test_split_merge_reproduces_unsplit():
    """Attention over the whole key range == merge of attention over disjoint key sub-ranges."""
    d = _golden.load("g_causal_gqa_mix")
    kw = _golden.oracle_kwargs(d)
    full, lse_full = ref_attention(d["q"], d["k"], d["v"], **kw)
    # non-causal split on a single-sequence problem: use g_fp8_scalar_scales (1 seq, 160 keys)
    d = _golden.load("g_fp8_scalar_scales")
    kw = _golden.oracle_kwargs(d)
    full, lse_full = ref_attention(d["q"], d["k"], d["v"], **kw)
    parts_o, parts_l = [], []
    for a, b in ((0, 64), (64, 128), (128, 160)):
        kw2 = dict(kw)
        kw2["cu_seqlens_k"] = torch.tensor([0, b - a], dtype=torch.int32)
        o, l = ref_attention(d["q"], d["k"][a:b], d["v"][a:b], **kw2)
        parts_o.append(o)
        parts_l.append(l)
    # an empty split must be ignored even if its partial is garbage
    parts_o.append(torch.full_like(parts_o[0], float("nan")))
    parts_l.append(torch.full_like(parts_l[0], float("-inf")))
    out, lse = combine_partials(torch.stack(parts_o), torch.stack(parts_l))
    torch.testing.assert_close(out, full, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(lse, lse_full, atol=1e-5, rtol=1e-5)
