"""Generates the golden fixtures in this directory from the reference's own Python code.

Run in a checkout that has the reference mounted (it is imported, never copied):

    python tests/golden/make_golden.py --ref <reference checkout>

For each small scenario below it calls the reference's `make_inputs(cfg, seed, device="cpu")`
(bench/scenarios.py:741-819) and its fp32 oracle `ref_fp32` (bench/scenarios.py:943-1024) and stores
inputs + expected output in `<name>.npz`.  bf16/fp16 tensors are stored as their int16 bit patterns,
fp8-e4m3 as uint8, so the fixtures are bit-exact and need no reference at test time.
The scenarios are ours (small shapes that exercise every feature the op boundary takes); the numbers
in the fixtures are the reference's.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _bits(t: torch.Tensor):
    if t is None:
        return None, None
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.contiguous().view(torch.int16).numpy(), str(t.dtype).replace("torch.", "")
    if t.dtype == torch.float8_e4m3fn:
        return t.contiguous().view(torch.uint8).numpy(), "float8_e4m3fn"
    return t.contiguous().numpy(), str(t.dtype).replace("torch.", "")


def scenarios(S):
    C = S.Config
    return [
        # name, phase, dtype, hd, hq, hkv, ...
        C("g_dense_nc_mha", "prefill", "bf16", 128, 2, 2, causal=False, paged=False, batch=2, q_len=40, k_len=40),
        C("g_causal_gqa_mix", "prefill", "bf16", 128, 4, 2, causal=True, paged=False,
          mix=((30, 30), (17, 150), (40, 40), (1, 40))),
        C("g_causal_q_gt_k", "prefill", "fp16", 128, 2, 2, causal=True, paged=False, batch=2, q_len=50, k_len=33),
        C("g_win_cap_sink", "prefill", "bf16", 128, 4, 2, causal=True, paged=False, window_left=37, window_right=0,
          softcap=30.0, sink=True, mix=((60, 60), (24, 200), (17, 17))),
        C("g_local_two_sided", "prefill", "bf16", 64, 4, 1, causal=False, paged=False, window_left=20, window_right=11,
          batch=2, q_len=45, k_len=130),
        C("g_paged_decode_leftpad", "decode", "bf16", 128, 8, 2, causal=True, paged=True, block_size=16, leftpad=5,
          mix=((1, 77), (1, 300), (1, 16), (1, 129))),
        C("g_paged_decode_p64_sink", "decode", "bf16", 128, 8, 2, causal=True, paged=True, block_size=64, sink=True,
          mix=((1, 300), (1, 64), (1, 191))),
        C("g_paged_spec_q4", "decode", "fp16", 128, 8, 2, causal=True, paged=True, block_size=32,
          mix=((4, 260), (4, 97))),
        C("g_paged_prefill_chunk", "prefill", "bf16", 128, 4, 2, causal=True, paged=True, block_size=16,
          mix=((24, 200), (66, 66))),
        C("g_fp8_qkv_causal", "prefill", "fp8e4m3", 128, 4, 2, causal=True, paged=False, batch=2, q_len=50, k_len=50),
        C("g_fp8kv_paged_decode", "decode", "bf16q_fp8kv", 128, 8, 2, causal=True, paged=True, block_size=64, leftpad=9,
          mix=((1, 333), (1, 70), (1, 128))),
        C("g_fp8_scalar_scales", "prefill", "fp8e4m3", 128, 2, 2, causal=False, paged=False, batch=1, q_len=64, k_len=160,
          fp8_scales="scalar"),
        C("g_hd192_dv128", "prefill", "bf16", 192, 2, 2, causal=True, paged=False, head_dim_v=128, batch=2, q_len=36,
          k_len=136),
        C("g_hd64_mqa", "prefill", "bf16", 64, 4, 1, causal=True, paged=False, batch=2, q_len=70, k_len=70),
        C("g_hd96_pad", "prefill", "bf16", 96, 4, 2, causal=True, paged=False, batch=1, q_len=65, k_len=65),
        C("g_hd256", "prefill", "bf16", 256, 2, 1, causal=True, paged=False, batch=1, q_len=40, k_len=72),
    ]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="path of the reference checkout (read-only)")
    a = ap.parse_args()
    sys.path.insert(0, a.ref)
    from bench import scenarios as S  # the reference's module, imported from where it lies

    torch.set_num_threads(max(1, os.cpu_count() or 1))
    index = []
    for i, cfg in enumerate(scenarios(S)):
        inp = S.make_inputs(cfg, seed=100 + i, device="cpu")
        ref = S.ref_fp32(inp)
        arrs, meta = {}, {"cfg": cfg.to_dict(), "seed": 100 + i, "dtypes": {},
                          "max_seqlen_q": inp.max_seqlen_q, "max_seqlen_k": inp.max_seqlen_k,
                          "softmax_scale": inp.softmax_scale}
        for name in ("q", "k", "v", "cu_seqlens_q", "cu_seqlens_k", "seqused_k", "page_table",
                     "q_descale", "k_descale", "v_descale", "s_aux", "leftpad_k"):
            t = getattr(inp, name)
            if t is None:
                continue
            arr, dt = _bits(t)
            arrs[name] = arr
            meta["dtypes"][name] = dt
        arrs["ref_out"] = ref.numpy()
        arrs["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
        path = os.path.join(HERE, cfg.name + ".npz")
        np.savez_compressed(path, **arrs)
        index.append(cfg.name)
        print(f"{cfg.name}: q{tuple(inp.q.shape)} k{tuple(inp.k.shape)} -> {os.path.getsize(path)} B")
    with open(os.path.join(HERE, "INDEX.json"), "w") as f:
        json.dump(index, f, indent=1)


if __name__ == "__main__":
    main()
