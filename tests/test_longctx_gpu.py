"""Long-context configuration (head_dim 192 / head_dim_v 128, paged, causal chunk against a long KV):
a reduced size against the full oracle, and the full 524288-key size on sampled rows and heads."""
import pytest
import torch

from flash_cuda_b200 import capi, workloads as W
from oracle.ref_attention import ref_attention

pytestmark = pytest.mark.gpu


def test_long_context_reduced_full_check(cuda_device):
    p = W.long_context(cuda_device, seed=3, q_len=300, k_len=4096, heads=4)
    out, lse, _ = capi.fwd(p.q, p.k, p.v, check=True, **p.capi_kw())
    pc = p.to("cpu")
    ref_out, ref_lse = ref_attention(pc.q, pc.k, pc.v, **pc.oracle_kw())
    assert (out.float().cpu() - ref_out).abs().max().item() <= 2e-2
    torch.testing.assert_close(lse.cpu(), ref_lse, atol=5e-3, rtol=1e-2)


def test_long_context_full_size_sampled_rows(cuda_device):
    free, _ = torch.cuda.mem_get_info(cuda_device)
    if free < 60e9:
        pytest.skip("needs ~45 GB of device memory")
    q_len, k_len, heads = 4096, 524288, 128
    p = W.long_context(cuda_device, seed=0, q_len=q_len, k_len=k_len, heads=heads)
    out, lse, _ = capi.fwd(p.q, p.k, p.v, check=True, **p.capi_kw())
    rows, hs = [0, 1, 127, 128, 2049, 4095], [0, 77, 127]
    # oracle on the sampled heads only: gather those heads to the host as a 3-head problem
    k_s = p.k[:, :, hs, :].cpu()
    v_s = p.v[:, :, hs, :].cpu()
    q_s = p.q[:, hs, :].cpu()
    ref_out, ref_lse = ref_attention(q_s, k_s, v_s, cu_seqlens_q=p.cu_seqlens_q.cpu(), seqused_k=p.seqused_k.cpu(),
                                     page_table=p.page_table.cpu(), softmax_scale=p.softmax_scale, causal=True,
                                     q_rows=rows)
    got = out[:, hs, :].float().cpu()
    for r in rows:
        assert (got[r] - ref_out[r]).abs().max().item() <= 2e-2, f"row {r}"
        torch.testing.assert_close(lse[hs, r].cpu(), ref_lse[:, r], atol=5e-3, rtol=1e-2)
    assert torch.isfinite(out.float()).all()
