#!/usr/bin/env python
"""Benchmark of the hot path: one `fwd` call over one synthetic batch per step.

  python bench.py --gpus N --steps K --warmup W            our CUDA path (rank 0 prints ONE JSON line)
  python bench.py --impl reference ...                      the reference's own CPU implementation of the path
                                                            (its fp32 attention, restated in oracle/), host cores

Headline workload (`config.workload`): causal GQA prefill, bf16, B=4, Hq=32, Hkv=8, S=4096, head_dim 128
(seeded N(0,1) inputs, softmax scale 1/sqrt(128)); metric = prefill TFLOP/s, algorithmic FLOPs
2*(hd+hdv)*Hq*unmasked_pairs.  A second object, `decode`, reports the paged-KV decode workload (batch 128,
context 1k..32k, page 64, leftpad 0..63, bf16 KV) as achieved HBM GB/s.

For N > 1 the (batch, kv-head) work items are independent, so every rank runs its own batch (weak scaling,
no collective on the data path); value = total FLOPs of all ranks / max-over-ranks device time.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

# DRAM traffic per launch measured once with ncu (dram__bytes_read.sum + dram__bytes_write.sum); the captures and
# their commands are summarised under profiles/.  Prefill was captured at B=2 (133.2 MB) and grows in proportion to B.
NCU_PREFILL_TRAFFIC_PER_BATCH = 66.6e6
NCU_DECODE_TRAFFIC = {"bf16": 8.59e9, "fp8": 4.307e9}
METRIC = "prefill TFLOP/s per job (causal GQA bf16 B=4 Hq=32 Hkv=8 S=4096 d=128); decode HBM GB/s in `decode`"
L2_BYTES = 126 * 1024 * 1024


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                    bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


# ----------------------------------------------------------------------------------------------------
# clocks during the timed region
# ----------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ln in self.lines:
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[1]))
                mx = float(parts[2])
            except ValueError:
                continue
            for n, v in zip(names, parts[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": (sm[len(sm) // 2] if sm else None), "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# ----------------------------------------------------------------------------------------------------
# CPU arm: the reference's fp32 attention on the host cores, on a bounded sample of the workload
# ----------------------------------------------------------------------------------------------------
def _cpu_sample_problem(seed: int = 0):
    """One (batch, kv head) slice of the prefill workload: S=4096, the 4 q heads of kv head 0."""
    from flash_cuda_b200 import workloads as W
    return W.make_problem("prefill_sample_b1_hq4_hkv1_s4096", [(4096, 4096)], hq=4, hkv=1, hd=128, causal=True,
                          seed=seed)


def cpu_baseline(budget_s: float = 10.0) -> dict:
    """The CPU port on one slice of the workload, repeated for about `budget_s` seconds of CPU work."""
    from oracle.ref_attention import ref_attention
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    p = _cpu_sample_problem()
    fl = p.flops()
    ref_attention(p.q[:256], p.k, p.v, **dict(p.oracle_kw(), cu_seqlens_q=torch.tensor([0, 256], dtype=torch.int32)))
    ts = []
    t_begin = time.perf_counter()
    while len(ts) < 3 or (time.perf_counter() - t_begin < budget_s and len(ts) < 500):
        t0 = time.perf_counter()
        ref_attention(p.q, p.k, p.v, **p.oracle_kw())
        ts.append(time.perf_counter() - t0)
    reps = len(ts)
    total = sum(ts)
    ts.sort()
    t = ts[len(ts) // 2]
    return {"value": fl / t / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"1 of the 32 (batch, kv-head) slices of the workload (S=4096, 4 q heads, {fl / 1e9:.1f} GFLOP), "
                      f"median of {reps} repetitions ({total:.1f} s of CPU work), {t * 1e3:.0f} ms each", "ms_per_sample": t * 1e3}


def run_reference(args) -> None:
    """`--impl reference`: rank 0 times the CPU implementation; other ranks exit without work."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle.ref_attention import ref_attention
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    p = _cpu_sample_problem()
    fl = p.flops()
    for _ in range(max(1, min(args.warmup, 3))):
        ref_attention(p.q, p.k, p.v, **p.oracle_kw())
    t0 = time.perf_counter()
    for _ in range(args.steps):
        ref_attention(p.q, p.k, p.v, **p.oracle_kw())
    dt = (time.perf_counter() - t0) / args.steps
    val = fl / dt / 1e12
    sample = (f"each step = 1 of the 32 (batch, kv-head) slices of the workload (S=4096, 4 q heads, "
              f"{fl / 1e9:.1f} GFLOP)")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic (seeded N(0,1))",
        "config": {"workload": "causal GQA prefill B=4 Hq=32 Hkv=8 S=4096 d=128 (CPU: bounded sample per step)"},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ----------------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------------
def _time_steps(fn, steps, dist, world):
    """Barrier + synchronize on both sides, CUDA events on the current stream; returns ms per step, max over ranks."""
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(steps):
        fn(i)
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / steps
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
        ms = float(t.item())
    return ms


def _tensor_bytes(*ts):
    return int(sum(t.numel() * t.element_size() for t in ts if t is not None))


def run_ours(args) -> None:
    from flash_cuda_b200 import capi, ops, workloads as W

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    dist = None
    if world > 1:
        import torch.distributed as dist  # noqa: F811
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device for --impl ours (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    ops.load(build_if_missing=False)
    peaks = _peaks()

    # ---- prefill workload: R rotating copies so that no step re-reads lines a recent step left in L2 ----
    host = W.causal_gqa_prefill(seed=rank, B=args.batch).pin()
    flops = host.flops()
    R = 4
    sets = [host.to(dev) for _ in range(R)]
    outs = [torch.empty(host.q.shape[0], host.q.shape[1], host.v.shape[-1], device=dev, dtype=torch.bfloat16)
            for _ in range(R)]
    in_bytes = _tensor_bytes(host.q, host.k, host.v)

    def step(i):
        p = sets[i % R]
        ops.call_fwd(p.q, p.k, p.v, out=outs[i % R], **p.capi_kw())

    for i in range(max(args.warmup, 3)):
        step(i)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    ms = _time_steps(step, args.steps, dist, world)
    clocks = sampler.stop() if rank == 0 else {}
    value = flops * world / (ms * 1e-3) / 1e12
    per_gpu = flops / (ms * 1e-3) / 1e12

    # ---- end to end: pinned host inputs -> device, op, result -> pinned host, all inside the timed region ----
    # Every step copies its inputs from pinned host memory and reads its result back.  The three legs of a step run
    # on three streams (copy-in, the op on the current stream, copy-out) with two buffer sets, so step i+1's inputs
    # travel while step i computes and step i-1's result travels back; events order the legs of one step and
    # protect each buffer until its previous user is done.
    e2e = None
    if not args.no_e2e:
        s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        cur = torch.cuda.current_stream(dev)
        dbuf = [(torch.empty_like(sets[0].q), torch.empty_like(sets[0].k), torch.empty_like(sets[0].v)) for _ in range(2)]
        obuf = [torch.empty_like(outs[0]) for _ in range(2)]
        h_out = [torch.empty(outs[0].shape, dtype=outs[0].dtype).pin_memory() for _ in range(2)]
        kw = dict(sets[0].capi_kw())

        def e2e_run(n):
            ev_in = [None, None]     # inputs of the step that last used buffer set b have landed
            ev_op = [None, None]     # the op that last used buffer set b has finished
            ev_out = [None, None]    # the result in obuf[b] has been copied out
            for i in range(n):
                b = i & 1
                with torch.cuda.stream(s_in):
                    if ev_op[b] is not None:
                        s_in.wait_event(ev_op[b])          # the op two steps back has read these inputs
                    dbuf[b][0].copy_(host.q, non_blocking=True)
                    dbuf[b][1].copy_(host.k, non_blocking=True)
                    dbuf[b][2].copy_(host.v, non_blocking=True)
                    ev_in[b] = torch.cuda.Event()
                    ev_in[b].record(s_in)
                cur.wait_event(ev_in[b])
                if ev_out[b] is not None:
                    cur.wait_event(ev_out[b])              # obuf[b] has been read back
                ops.call_fwd(dbuf[b][0], dbuf[b][1], dbuf[b][2], out=obuf[b], **kw)
                ev_op[b] = torch.cuda.Event()
                ev_op[b].record(cur)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_op[b])
                    h_out[b].copy_(obuf[b], non_blocking=True)
                    ev_out[b] = torch.cuda.Event()
                    ev_out[b].record(s_out)
            for e in ev_out:
                if e is not None:
                    cur.wait_event(e)                      # the timed region ends when the last result is on the host

        e2e_run(3)
        n_e2e = max(4, min(20, args.steps // 4))
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        e2e_run(n_e2e)
        t1.record()
        torch.cuda.synchronize()
        e2e_ms = t0.elapsed_time(t1) / n_e2e
        if world > 1:
            tt = torch.tensor([e2e_ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            dist.barrier()
            e2e_ms = float(tt.item())
        e2e = {"value": flops * world / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": in_bytes, "d2h_bytes_per_step": _tensor_bytes(h_out[0]),
               "overlap": "copy-in, op and copy-out of consecutive steps on three streams, two buffer sets"}

    # ---- decode workload (secondary objects: bf16 KV cache, and e4m3 KV cache with --decode-fp8) ----
    def decode_leg(kv_dtype):
        try:
            dp = W.paged_decode_on_device(dev, seed=rank, kv_dtype=kv_dtype)   # the 8.5 GB pool is drawn on the GPU
            kvb = dp.kv_bytes()
            dout = torch.empty(dp.q.shape[0], dp.q.shape[1], dp.v.shape[-1], device=dev, dtype=torch.bfloat16)
            nspl = capi.num_splits(dp.q, dp.k, dp.v, **dp.capi_kw())

            def dstep(i):
                ops.call_fwd(dp.q, dp.k, dp.v, out=dout, **dp.capi_kw())

            for i in range(max(args.warmup, 3)):
                dstep(i)
            dms = _time_steps(dstep, max(3, min(args.steps, 100)), dist, world)
            gbs = kvb / (dms * 1e-3) / 1e9
            return {
                "metric": f"paged decode HBM GB/s (B=128 q_len=1 ctx 1k..32k page 64 Hq=32 Hkv=8 d=128 {kv_dtype} KV, "
                          "leftpad 0..63)",
                "value": gbs * world, "unit": "GB/s", "ms_per_step": dms, "kv_bytes_per_step": kvb,
                "num_splits": nspl,
                "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                             "frac": gbs / peaks["hbm_gbs"], "traffic": NCU_DECODE_TRAFFIC[kv_dtype],
                             "traffic_source": "ncu dram__bytes_read+write per launch of this configuration (profiles/)",
                             "peak_source": peaks["source"]},
                "l2": f"KV pool ({kvb / 1e9:.2f} GB) larger than L2",
            }
        except Exception as e:  # reported, never hidden
            return {"error": repr(e)}

    decode = None if args.no_decode else decode_leg("bf16")
    decode_fp8 = decode_leg("fp8") if args.decode_fp8 else None

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    cpu = cpu_baseline() if (world == 1 and not args.no_cpu) else None
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded N(0,1), random-permuted page table for decode)",
        "config": {"workload": f"causal GQA prefill B={args.batch} Hq=32 Hkv=8 S=4096 d=128 bf16 per GPU",
                   "parallelism": f"(batch, kv-head) items sharded over {world} GPU(s), no collective",
                   "l2": f"{R} rotating input sets of {in_bytes / 1e6:.0f} MB each (> L2 {L2_BYTES / 1e6:.0f} MB)",
                   "flops_per_step_per_gpu": flops},
        "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": per_gpu / peaks["bf16_tflops"], "traffic": NCU_PREFILL_TRAFFIC_PER_BATCH * args.batch,
                     "traffic_source": "ncu dram__bytes_read+write of a B=2 launch, scaled by B (profiles/)",
                     "peak_source": peaks["source"], "kernel": "fwd_prefill_tc_kernel", "launch_ms": ms},
        "e2e": e2e, "gpu_launches": args.steps, "clocks": clocks, "decode": decode, "decode_fp8": decode_fp8, "cpu_baseline": cpu,
        "kernels_per_step": {"prefill": ["fwd_prefill_tc_kernel"], "decode": ["sched_kernel", "fwd_decode_kernel"]},
    }
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_longctx(args) -> None:
    """`--workload longctx`: B=1, a chunk of 4096 query rows against a paged KV of 524288 tokens (page 64),
    128 heads, head_dim 192 / head_dim_v 128, causal, bf16.  The key range is split evenly over the ranks
    (strong scaling); partial O / LSE are merged with ONE all-gather + the merge kernel, inside the timed region."""
    from flash_cuda_b200 import multi_gpu as MG, ops, workloads as W

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    dist = None
    if world > 1:
        import torch.distributed as dist  # noqa: F811
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    ops.load(build_if_missing=False)
    peaks = _peaks()
    q_len, k_len, heads = 4096, args.longctx_keys, 128
    per = k_len // world
    p = W.long_context(dev, seed=0, q_len=q_len, k_len=k_len, heads=heads, k_begin=rank * per, k_end=(rank + 1) * per)
    # unmasked pairs per head of the WHOLE problem: sum_i (k_len - q_len + i + 1)
    pairs = q_len * (k_len - q_len) + q_len * (q_len + 1) // 2
    flops = 2.0 * (192 + 128) * heads * pairs

    def step(i):
        MG.fwd_kv_sharded(p.q, p.k, p.v, page_table_local=p.page_table, seqused_k_local=p.seqused_k,
                          cu_seqlens_q=p.cu_seqlens_q, max_seqlen_q=q_len, max_seqlen_k_local=per,
                          softmax_scale=p.softmax_scale, causal=True, rank=rank, world=world)

    for i in range(max(args.warmup, 3)):
        step(i)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    steps = max(1, min(args.steps, 10))
    ms = _time_steps(step, steps, dist, world)
    clocks = sampler.stop() if rank == 0 else {}
    if rank == 0:
        val = flops / (ms * 1e-3) / 1e12
        print(json.dumps({
            "metric": "long-context prefill TFLOP/s (q 4096 x paged KV 524288, 128 heads, hd192/hdv128, causal, bf16), whole job",
            "value": val, "unit": "TFLOP/s", "n_gpus": world, "steps": steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (N(0,1) drawn on the device, seeded)",
            "config": {"workload": f"long-context prefill q={q_len} k={k_len} heads={heads} hd192/hdv128 page 64",
                       "parallelism": f"KV range split over {world} GPU(s); one all-gather of [O|LSE] + merge kernel",
                       "l2": f"KV shard {p.k.numel() * 2 / 1e9 + p.v.numel() * 2 / 1e9:.1f} GB per GPU (> L2)"},
            "roofline": {"bound": "tensor", "achieved": val / world, "peak": peaks["bf16_tflops_sustained"],
                         "unit": "TFLOP/s", "frac": val / world / peaks["bf16_tflops_sustained"], "traffic": None,
                         "peak_source": peaks["source"] + " (sustained: seconds-long step)"},
            "gpu_launches": steps * (1 if world == 1 else 2), "clocks": clocks}))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-decode", action="store_true", help="skip the decode workload")
    ap.add_argument("--decode-fp8", action="store_true", help="also time the decode workload with an e4m3 KV cache")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--batch", type=int, default=4, help="prefill batch per GPU (4 = the benchmark configuration; "
                    "smaller values are for profiler captures only)")
    ap.add_argument("--workload", default="prefill", choices=["prefill", "longctx"],
                    help="prefill = the headline configuration (+ decode object); longctx = KV-range sharded long context")
    ap.add_argument("--longctx-keys", type=int, default=524288)
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "longctx":
        run_longctx(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
