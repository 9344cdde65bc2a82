"""Append-KV + rotary (the op's `k_new` / `v_new` / `rotary_*` arguments), through the C ABI and through the torch op,
against the CPU restatement in oracle/append_oracle.py.  Cache bytes, rotated queries and the new key counts are
integer / byte results of exactly specified fp32 arithmetic: they must match BIT FOR BIT.  The attention that follows is
checked with the usual tolerances against the fp32 oracle run on the oracle's own updated cache."""
import pytest
import torch

from flash_cuda_b200 import capi, ops
from oracle.append_oracle import append_kv_reference
from oracle.ref_attention import ref_attention

pytestmark = pytest.mark.gpu


def _case(dtype, page, hd, rd, seed, hq=8, hkv=2, used=(100, 5, 63, 64, 0), new=(3, 0, 1, 17, 2), q_lens=None):
    g = torch.Generator().manual_seed(seed)
    B = len(used)
    q_lens = list(new) if q_lens is None else list(q_lens)
    room = [u + n for u, n in zip(used, new)]
    npg = [(r + page - 1) // page + 1 for r in room]
    total_pages = sum(npg) + 2
    perm = torch.randperm(total_pages, generator=g)
    pt = torch.zeros(B, max(npg), dtype=torch.int32)
    o = 0
    for b, n in enumerate(npg):
        pt[b, :n] = perm[o:o + n].to(torch.int32)
        o += n
    kc = torch.randn(total_pages, page, hkv, hd, generator=g).to(dtype)
    vc = torch.randn(total_pages, page, hkv, hd, generator=g).to(dtype)
    kn = torch.randn(sum(new), hkv, hd, generator=g).to(dtype)
    vn = torch.randn(sum(new), hkv, hd, generator=g).to(dtype)
    q = torch.randn(sum(q_lens), hq, hd, generator=g).to(dtype)
    ang = torch.rand(4096, rd // 2, generator=g) * 6.283
    cu = lambda xs: torch.tensor([0] + list(torch.tensor(list(xs)).cumsum(0).tolist()), dtype=torch.int32)
    return dict(q=q, k_cache=kc, v_cache=vc, k_new=kn, v_new=vn, page_table=pt,
                seqused_k=torch.tensor(list(used), dtype=torch.int32), cu_seqlens_k_new=cu(new), cu_seqlens_q=cu(q_lens),
                rotary_cos=torch.cos(ang).to(dtype), rotary_sin=torch.sin(ang).to(dtype))


def _bits(t):
    return t.view(torch.int16) if t.element_size() == 2 else t.view(torch.uint8)


@pytest.mark.parametrize("interleaved", [True, False])
@pytest.mark.parametrize("dtype,page,hd,rd", [(torch.bfloat16, 64, 128, 128), (torch.float16, 16, 128, 64),
                                             (torch.bfloat16, 1, 64, 32), (torch.bfloat16, 256, 192, 96 + 32)])
def test_append_and_rotary_are_bit_exact(dtype, page, hd, rd, interleaved, cuda_device):
    c = _case(dtype, page, hd, rd, seed=61)
    for advance, use_rot_lens in ((True, False), (False, True)):
        rot_lens = torch.tensor([7, 0, 1000, 3, 2], dtype=torch.int32) if use_rot_lens else None
        want_q, want_k, want_v, want_n = append_kv_reference(
            c["k_new"], c["v_new"], c["k_cache"], c["v_cache"], page_table=c["page_table"], seqused_k=c["seqused_k"],
            cu_seqlens_k_new=c["cu_seqlens_k_new"], q=c["q"], cu_seqlens_q=c["cu_seqlens_q"], rotary_cos=c["rotary_cos"],
            rotary_sin=c["rotary_sin"], seqlens_rotary=rot_lens, rotary_interleaved=interleaved, q_positions_advance=advance)
        d = {k: v.to(cuda_device) for k, v in c.items()}
        q_rot, n_out = capi.append_kv(d["k_new"], d["v_new"], d["k_cache"], d["v_cache"], page_table=d["page_table"],
                                      seqused_k=d["seqused_k"], cu_seqlens_k_new=d["cu_seqlens_k_new"], q=d["q"],
                                      cu_seqlens_q=d["cu_seqlens_q"], rotary_cos=d["rotary_cos"], rotary_sin=d["rotary_sin"],
                                      seqlens_rotary=None if rot_lens is None else rot_lens.to(cuda_device),
                                      rotary_interleaved=interleaved, q_positions_advance=advance)
        torch.cuda.synchronize()
        assert n_out.cpu().tolist() == want_n.tolist()
        assert torch.equal(_bits(d["k_cache"].cpu()), _bits(want_k)), "K cache bytes differ"
        assert torch.equal(_bits(d["v_cache"].cpu()), _bits(want_v)), "V cache bytes differ"
        assert torch.equal(_bits(q_rot.cpu()), _bits(want_q)), "rotated q differs"
        assert torch.equal(_bits(d["q"].cpu()), _bits(c["q"])), "q itself must not be modified"


@pytest.mark.parametrize("used,new,q_lens", [((0, 399), (0, 0), (0, 3)),      # nothing to append, queries still rotate
                                             ((473,), (11,), (0,)),            # keys appended, no query row at all
                                             ((0,), (0,), (0,))])              # nothing of either
def test_append_steps_without_new_keys_or_without_queries(used, new, q_lens, cuda_device):
    """Empty `k_new` / `q` tensors have no address: the call must take them for what they are."""
    c = _case(torch.float16, 8, 64, 32, seed=65, hq=4, hkv=4, used=used, new=new, q_lens=q_lens)
    want_q, want_k, want_v, want_n = append_kv_reference(
        c["k_new"], c["v_new"], c["k_cache"], c["v_cache"], page_table=c["page_table"], seqused_k=c["seqused_k"],
        cu_seqlens_k_new=c["cu_seqlens_k_new"], q=c["q"], cu_seqlens_q=c["cu_seqlens_q"], rotary_cos=c["rotary_cos"],
        rotary_sin=c["rotary_sin"], rotary_interleaved=True, q_positions_advance=False)
    d = {k: v.to(cuda_device) for k, v in c.items()}
    q_rot, n_out = capi.append_kv(d["k_new"], d["v_new"], d["k_cache"], d["v_cache"], page_table=d["page_table"],
                                  seqused_k=d["seqused_k"], cu_seqlens_k_new=d["cu_seqlens_k_new"], q=d["q"],
                                  cu_seqlens_q=d["cu_seqlens_q"], rotary_cos=d["rotary_cos"], rotary_sin=d["rotary_sin"],
                                  rotary_interleaved=True, q_positions_advance=False)
    torch.cuda.synchronize()
    assert n_out.cpu().tolist() == want_n.tolist()
    assert torch.equal(_bits(d["k_cache"].cpu()), _bits(want_k)) and torch.equal(_bits(d["v_cache"].cpu()), _bits(want_v))
    assert torch.equal(_bits(q_rot.cpu()), _bits(want_q))


def test_append_without_rotary_into_e4m3_cache_is_a_byte_copy(cuda_device):
    c = _case(torch.bfloat16, 32, 128, 128, seed=62)
    f8 = lambda t: (t.float() * 8).to(torch.float8_e4m3fn)
    kc, vc, kn, vn = f8(c["k_cache"]), f8(c["v_cache"]), f8(c["k_new"]), f8(c["v_new"])
    _, want_k, want_v, want_n = append_kv_reference(kn, vn, kc, vc, page_table=c["page_table"], seqused_k=c["seqused_k"],
                                                   cu_seqlens_k_new=c["cu_seqlens_k_new"])
    dk, dv = kc.to(cuda_device), vc.to(cuda_device)
    _, n_out = capi.append_kv(kn.to(cuda_device), vn.to(cuda_device), dk, dv, page_table=c["page_table"].to(cuda_device),
                              seqused_k=c["seqused_k"].to(cuda_device), cu_seqlens_k_new=c["cu_seqlens_k_new"].to(cuda_device))
    torch.cuda.synchronize()
    assert n_out.cpu().tolist() == want_n.tolist()
    assert torch.equal(_bits(dk.cpu()), _bits(want_k)) and torch.equal(_bits(dv.cpu()), _bits(want_v))


def _op_args(d, *, k_new, v_new, cu_new, cos, sin, rot_lens, interleaved, causal, page_table, kv_batch_idx=None,
             seqused_k=None, max_k=None):
    B = d["cu_seqlens_q"].numel() - 1
    max_q = int((d["cu_seqlens_q"][1:] - d["cu_seqlens_q"][:-1]).max())
    return (d["q"], d["k_cache"], d["v_cache"], k_new, v_new, None, None, d["cu_seqlens_q"], None, cu_new, None,
            d["seqused_k"] if seqused_k is None else seqused_k, max_q, max_k, page_table, kv_batch_idx, None, cos, sin,
            rot_lens, None, None, None, d["q"].shape[-1] ** -0.5, causal, -1, -1, 0.0, interleaved, None, 0, None, 0,
            None, 1, 0, None)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("interleaved", [True, False])
def test_fwd_op_with_k_new_and_rotary(interleaved, causal, cuda_device):
    """The whole op: append + rotate + attention over cache and new keys, against the oracle chain."""
    c = _case(torch.bfloat16, 64, 128, 64, seed=63, used=(100, 5, 63, 300), new=(3, 1, 1, 17))
    want_q, want_k, want_v, want_n = append_kv_reference(
        c["k_new"], c["v_new"], c["k_cache"], c["v_cache"], page_table=c["page_table"], seqused_k=c["seqused_k"],
        cu_seqlens_k_new=c["cu_seqlens_k_new"], q=c["q"], cu_seqlens_q=c["cu_seqlens_q"], rotary_cos=c["rotary_cos"],
        rotary_sin=c["rotary_sin"], rotary_interleaved=interleaved, q_positions_advance=causal)
    ref_out, ref_lse = ref_attention(want_q, want_k, want_v, cu_seqlens_q=c["cu_seqlens_q"], seqused_k=want_n,
                                     page_table=c["page_table"], softmax_scale=128 ** -0.5, causal=causal)
    d = {k: v.to(cuda_device) for k, v in c.items()}
    res = ops.fwd(*_op_args(d, k_new=d["k_new"], v_new=d["v_new"], cu_new=d["cu_seqlens_k_new"], cos=d["rotary_cos"],
                            sin=d["rotary_sin"], rot_lens=None, interleaved=interleaved, causal=causal,
                            page_table=d["page_table"]))
    torch.cuda.synchronize()
    assert torch.equal(_bits(d["k_cache"].cpu()), _bits(want_k)) and torch.equal(_bits(d["v_cache"].cpu()), _bits(want_v))
    assert (res[0].float().cpu() - ref_out).abs().max().item() <= 2e-2
    fin = torch.isfinite(ref_lse)
    torch.testing.assert_close(res[1].cpu()[fin], ref_lse[fin], atol=5e-3, rtol=1e-2)


def test_batch_layout_cache_with_kv_batch_idx_and_batched_k_new(cuda_device):
    """A cache laid out (batch_cache, seqlen_cache, hkv, d) with `kv_batch_idx`, and k_new as (batch, seqlen_new, ...)."""
    g = torch.Generator().manual_seed(64)
    Bc, S, hkv, hq, hd, B, s_new = 5, 192, 2, 4, 128, 3, 2
    kc = torch.randn(Bc, S, hkv, hd, generator=g).to(torch.bfloat16)
    vc = torch.randn(Bc, S, hkv, hd, generator=g).to(torch.bfloat16)
    idx = torch.tensor([4, 0, 2], dtype=torch.int32)
    used = torch.tensor([100, 7, 190], dtype=torch.int32)
    kn = torch.randn(B, s_new, hkv, hd, generator=g).to(torch.bfloat16)
    vn = torch.randn(B, s_new, hkv, hd, generator=g).to(torch.bfloat16)
    q = torch.randn(B * s_new, hq, hd, generator=g).to(torch.bfloat16)
    cu_q = torch.arange(0, (B + 1) * s_new, s_new, dtype=torch.int32)
    pt = idx.view(B, 1)
    _, want_k, want_v, want_n = append_kv_reference(kn.reshape(-1, hkv, hd), vn.reshape(-1, hkv, hd), kc, vc, page_table=pt,
                                                   seqused_k=used, cu_seqlens_k_new=cu_q)
    ref_out, _ = ref_attention(q, want_k, want_v, cu_seqlens_q=cu_q, seqused_k=want_n, page_table=pt,
                               softmax_scale=hd ** -0.5, causal=True)
    dev = cuda_device
    d = dict(q=q.to(dev), k_cache=kc.to(dev), v_cache=vc.to(dev), cu_seqlens_q=cu_q.to(dev), seqused_k=used.to(dev))
    res = ops.fwd(*_op_args(d, k_new=kn.to(dev), v_new=vn.to(dev), cu_new=None, cos=None, sin=None, rot_lens=None,
                            interleaved=True, causal=True, page_table=None, kv_batch_idx=idx.to(dev)))
    torch.cuda.synchronize()
    assert torch.equal(_bits(d["k_cache"].cpu()), _bits(want_k)) and torch.equal(_bits(d["v_cache"].cpu()), _bits(want_v))
    assert (res[0].float().cpu() - ref_out).abs().max().item() <= 2e-2
