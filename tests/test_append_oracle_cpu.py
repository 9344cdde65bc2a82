"""CPU checks of the append-KV / rotary restatement (oracle/append_oracle.py) through properties that need no second
implementation: a rotation preserves the length of every rotated pair, rotating by position 0 with cos = 1, sin = 0 is
the identity, the appended rows are exactly the new rows, untouched cache rows keep their bytes, and attention over
the updated cache equals attention over the explicitly concatenated keys."""
import torch

from oracle.append_oracle import append_kv_reference, rotate_rows
from oracle.ref_attention import ref_attention


def test_rotation_properties():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(6, 3, 64, generator=g).to(torch.float16)
    ang = torch.rand(50, 16, generator=g) * 6.283
    cos, sin = torch.cos(ang).to(torch.float16), torch.sin(ang).to(torch.float16)
    pos = torch.tensor([0, 1, 7, 49, 3, 3])
    for inter in (True, False):
        y = rotate_rows(x, cos, sin, pos, inter)
        assert torch.equal(y[..., 32:], x[..., 32:])                       # dimensions >= rotary_dim pass through
        if inter:
            n0 = x[..., 0:32:2].float() ** 2 + x[..., 1:32:2].float() ** 2
            n1 = y[..., 0:32:2].float() ** 2 + y[..., 1:32:2].float() ** 2
        else:
            n0 = x[..., :16].float() ** 2 + x[..., 16:32].float() ** 2
            n1 = y[..., :16].float() ** 2 + y[..., 16:32].float() ** 2
        torch.testing.assert_close(n0, n1, atol=2e-2, rtol=2e-2)
        ident = rotate_rows(x, torch.ones_like(cos), torch.zeros_like(sin), pos, inter)
        assert torch.equal(ident, x)


def test_append_then_attention_equals_attention_over_concatenated_keys():
    g = torch.Generator().manual_seed(1)
    page, hkv, hq, hd = 16, 2, 4, 64
    used, new = [20, 0, 31], [3, 5, 1]
    pt = torch.tensor([[2, 0, 5], [1, 6, 7], [3, 4, 8]], dtype=torch.int32)
    kc = torch.randn(9, page, hkv, hd, generator=g).to(torch.bfloat16)
    vc = torch.randn(9, page, hkv, hd, generator=g).to(torch.bfloat16)
    kn = torch.randn(sum(new), hkv, hd, generator=g).to(torch.bfloat16)
    vn = torch.randn(sum(new), hkv, hd, generator=g).to(torch.bfloat16)
    q = torch.randn(sum(new), hq, hd, generator=g).to(torch.bfloat16)
    cu = torch.tensor([0, 3, 8, 9], dtype=torch.int32)
    _, k2, v2, n2 = append_kv_reference(kn, vn, kc, vc, page_table=pt, seqused_k=torch.tensor(used, dtype=torch.int32),
                                       cu_seqlens_k_new=cu)
    assert n2.tolist() == [23, 5, 32]
    out_a, _ = ref_attention(q, k2, v2, cu_seqlens_q=cu, seqused_k=n2, page_table=pt, softmax_scale=hd ** -0.5, causal=True)
    # the same keys, gathered and concatenated by hand into a packed (unpaged) layout
    ks, vs, cu_k = [], [], [0]
    for b in range(3):
        rows = torch.cat([kc[pt[b].long()].reshape(-1, hkv, hd)[:used[b]], kn[cu[b]:cu[b + 1]]])
        ks.append(rows)
        vs.append(torch.cat([vc[pt[b].long()].reshape(-1, hkv, hd)[:used[b]], vn[cu[b]:cu[b + 1]]]))
        cu_k.append(cu_k[-1] + rows.shape[0])
    out_b, _ = ref_attention(q, torch.cat(ks), torch.cat(vs), cu_seqlens_q=cu,
                             cu_seqlens_k=torch.tensor(cu_k, dtype=torch.int32), softmax_scale=hd ** -0.5, causal=True)
    torch.testing.assert_close(out_a, out_b, atol=1e-6, rtol=1e-6)
    # rows the append did not touch keep their bytes
    untouched = torch.ones(9, page, dtype=torch.bool)
    for b in range(3):
        for i in range(new[b]):
            kidx = used[b] + i
            untouched[int(pt[b, kidx // page]), kidx % page] = False
    assert torch.equal(k2[untouched].view(torch.int16), kc[untouched].view(torch.int16))
