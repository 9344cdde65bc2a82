"""CPU-side checks of the drop-in boundary: the C-ABI library loads and exports every symbol the header
declares, struct layouts agree, host-only planning agrees with the integer oracle, and the torch-op
library registers the two schemas.  No compute call is made (there is no GPU here)."""
import ctypes
import os
import re

import pytest
import torch

from flash_cuda_b200 import build, capi
from oracle import sched_oracle as SO

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    with open(os.path.join(ROOT, "include", "fa_b200.h")) as f:
        text = f.read()
    return sorted(set(re.findall(r"\b(fa_b200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = capi.load()
    names = _declared_symbols()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/fa_b200.h but not exported"
    assert set(names) == set(capi.EXPORTS)


def test_struct_layouts_match():
    lib = capi.load()
    assert lib.fa_b200_sizeof_fwd_params() == ctypes.sizeof(capi.FaFwdParams)
    assert lib.fa_b200_sizeof_sched_params() == ctypes.sizeof(capi.FaSchedParams)
    assert lib.fa_b200_version() >= 1
    assert lib.fa_b200_strerror(capi.FA_ERR_UNSUPPORTED).decode().startswith("unsupported")


def test_no_gpu_means_error_not_fallback():
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = capi.load()
    p = capi.FaFwdParams()
    # a structurally valid problem; pointers are never dereferenced on the host
    for n in ("q", "k", "v", "out", "lse", "cu_seqlens_q", "cu_seqlens_k"):
        setattr(p, n, 4096)
    p.batch, p.total_q, p.total_k, p.hq, p.hkv, p.hd, p.hdv = 1, 8, 8, 2, 2, 128, 128
    p.max_seqlen_q = p.max_seqlen_k = 8
    for n in ("q_row_stride", "k_row_stride", "v_row_stride", "o_row_stride"):
        setattr(p, n, 256)
    for n in ("q_head_stride", "k_head_stride", "v_head_stride", "o_head_stride"):
        setattr(p, n, 128)
    rc = lib.fa_b200_fwd(ctypes.byref(p), 4096, 1 << 20, None)
    assert rc == capi.FA_ERR_NO_DEVICE


PLAN_CASES = [
    dict(batch=128, max_seqlen_q=1, max_seqlen_k=32768, hq=32, hkv=8, hd=128, hdv=128, page_size=64),
    dict(batch=1, max_seqlen_q=1, max_seqlen_k=32768, hq=32, hkv=8, hd=128, hdv=128, page_size=64),
    dict(batch=2, max_seqlen_q=4, max_seqlen_k=5000, hq=16, hkv=2, hd=128, hdv=128, page_size=16),
    dict(batch=4, max_seqlen_q=4096, max_seqlen_k=4096, hq=32, hkv=8, hd=128, hdv=128, page_size=0),
    dict(batch=1, max_seqlen_q=100, max_seqlen_k=100000, hq=4, hkv=4, hd=256, hdv=256, page_size=0),
    dict(batch=3, max_seqlen_q=1, max_seqlen_k=700, hq=8, hkv=8, hd=64, hdv=64, page_size=1),
    dict(batch=1, max_seqlen_q=4096, max_seqlen_k=524288, hq=128, hkv=128, hd=192, hdv=128, page_size=64),
]


@pytest.mark.parametrize("num_splits", [0, 1, 5])
@pytest.mark.parametrize("case", PLAN_CASES)
def test_host_plan_matches_integer_oracle(case, num_splits):
    lib = capi.load()
    plan = SO.make_plan(num_splits=num_splits, num_sms_device=148, **case)
    p = capi.FaFwdParams()
    for k_, v_ in case.items():
        if hasattr(p, k_):
            setattr(p, k_, v_)
    p.page_table = 4096 if case["page_size"] else None
    p.num_pages = 1024
    # packed layouts: heads back to back inside a token row, pages back to back
    p.q_head_stride, p.k_head_stride, p.v_head_stride = case["hd"], case["hd"], case["hdv"]
    p.q_row_stride, p.k_row_stride = case["hq"] * case["hd"], case["hkv"] * case["hd"]
    p.v_row_stride = case["hkv"] * case["hdv"]
    p.k_page_stride, p.v_page_stride = case["page_size"] * p.k_row_stride, case["page_size"] * p.v_row_stride
    p.num_splits = num_splits
    p.total_q = case["batch"] * case["max_seqlen_q"]
    assert lib.fa_b200_num_splits(ctypes.byref(p)) == plan.nsplits
    sp = capi.sched_params(dtype=torch.bfloat16, num_splits=num_splits, **case)
    assert lib.fa_b200_scheduler_metadata_len(ctypes.byref(sp)) == SO.HEADER + 4 * case["batch"] * plan.max_mtiles


def test_index_arithmetic_properties():
    # every key a row may attend lies inside the block range; split ranges tile the range exactly
    import random
    rnd = random.Random(0)
    for _ in range(300):
        sk, sq = rnd.randint(0, 700), rnd.randint(1, 300)
        tn = rnd.choice([64, 128])
        causal = rnd.random() < 0.5
        wl = rnd.choice([-1, 0, 5, 100])
        wr = rnd.choice([-1, 0, 7])
        pad = rnd.choice([0, 0, 3, 64, 200])
        r0 = rnd.randint(0, sq - 1)
        r1 = min(sq - 1, r0 + rnd.randint(0, 255))
        lo, hi = SO.nblock_range(sk, pad, sk - sq + r0, sk - sq + r1, causal, wl, wr, tn)
        assert 0 <= lo <= hi <= SO.cdiv(sk, tn)
        for r in (r0, r1):
            qp = sk - sq + r
            for kk in range(sk):
                ok = kk >= pad and (not causal or kk <= qp) and (wl < 0 or kk >= qp - wl) and (wr < 0 or kk <= qp + wr)
                if ok:
                    assert lo <= kk // tn < hi
        ns = rnd.randint(1, 9)
        cover = []
        for s in range(ns):
            a, b = SO.split_range(lo, hi, s, ns)
            assert lo <= a <= b <= hi
            cover += list(range(a, b))
        assert cover == list(range(lo, hi))
    assert SO.page_row([7, 2, 9], 70, 64) == 2 * 64 + 6


def test_torch_op_library_registers_reference_schemas():
    from flash_cuda_b200 import ops
    ns = ops.load()
    fwd_schema = str(ns.fwd.default._schema)
    assert fwd_schema.count(",") == 36 and "Tensor[]" in fwd_schema and "s_aux" in fwd_schema
    md_schema = str(ns.get_scheduler_metadata.default._schema)
    assert md_schema.count(",") == 22 and md_schema.endswith("-> Tensor")
    assert os.path.isfile(build.TORCH_SO) and os.path.isfile(build.CAPI_SO)
