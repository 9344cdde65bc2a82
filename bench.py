#!/usr/bin/env python
"""Benchmark of the hot path: one `fwd` call over one synthetic batch per step.

  python bench.py --gpus N --steps K --warmup W            our CUDA path (rank 0 prints ONE JSON line)
  python bench.py --impl reference ...                      the reference's own CPU implementation of the path
                                                            (its fp32 attention, restated in oracle/), host cores

Headline workload (`config.workload`): causal GQA prefill, bf16, B=4, Hq=32, Hkv=8, S=4096, head_dim 128
(seeded N(0,1) inputs, softmax scale 1/sqrt(128)); metric = prefill TFLOP/s, algorithmic FLOPs
2*(hd+hdv)*Hq*unmasked_pairs.  Further objects of the same JSON line report the other benchmark configurations:
`c1` (dense non-causal, latency), `c2_fp8` (the headline in e4m3), `c3` (varlen + window + softcap + sink),
`decode` / `decode_fp8` (paged decode, batch 128, context 1k..32k, page 64, leftpad 0..63, bf16 / e4m3 cache, as
achieved HBM GB/s) and `c5` (long context: q 4096 x paged KV 524288, hd192/128, KV range sharded over the GPUs).

For N > 1 the headline is ONE shared problem of N x 4 sequences whose kv heads are sharded over the ranks by
`multi_gpu.fwd_head_sharded` (per-GPU work = the 1-GPU configuration: weak scaling, no collective);
value = total FLOPs / max-over-ranks device time.  `c5` is strong scaling through `multi_gpu.fwd_kv_sharded`
(one all-gather of the partial results + the merge kernel inside the timed region).
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
# their commands are summarised under profiles/.  Prefill was captured at B=2 (137.6 MB) and grows in proportion to B.
NCU_PREFILL_TRAFFIC_PER_BATCH = 68.8e6
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
# optional arm: the reference's own sm_100a kernel beside ours, same tensors, same loop (one GPU)
# ----------------------------------------------------------------------------------------------------
AB_SHAPES = ("c2", "c1", "c4")
# Shapes the reference's kernel is not run on: it did not return within the limit on the first of them (the child
# process was ended by the host-side timeout, the GPU kept answering); the second was never reached.
AB_SHAPES_STALLED = ("h16_s4k", "h16_s8k")


def _ab_problem(name):
    from flash_cuda_b200 import workloads as W
    if name == "c2":
        return W.causal_gqa_prefill()
    if name == "c1":
        return W.dense_noncausal()
    if name == "h16_s4k":
        return W.make_problem("dense_c_d128_s4k", [(4096, 4096)] * 4, hq=16, hkv=16, hd=128, causal=True)
    if name == "h16_s8k":
        return W.make_problem("dense_c_d128_s8k", [(8192, 8192)] * 2, hq=16, hkv=16, hd=128, causal=True)
    if name == "c4":
        p = W.paged_decode()
        p.leftpad_k = None      # the reference's kernel reads only leftpad_k[0] (kernels/fa4_blackwell.cu:10126-10127)
        return p
    raise SystemExit(f"unknown A/B shape {name!r}; choose from {AB_SHAPES + AB_SHAPES_STALLED}")


def run_ab_one(name: str) -> None:
    """One shape, in a process of its own: ours and the reference's kernel on the same device tensors, alternating
    over 4 rotating input copies, median of 20 CUDA-event timings each; numerics of one against the other."""
    from dataclasses import replace
    from flash_cuda_b200 import ops
    so = os.path.join(ROOT, "oracle", "_ref", "fa4_ref.so")
    if not os.path.isfile(so):
        print(json.dumps({"shape": name, "unavailable": "oracle/_ref/fa4_ref.so is not built (python oracle/build_ref.py)"}))
        return
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    ops.load(build_if_missing=False)
    torch.ops.load_library(so)
    ref = torch.ops.fa4_ref.fwd
    p = _ab_problem(name)
    fl, by = p.flops(), p.kv_bytes()
    p0 = p.to(dev)
    R = 4 if name != "c4" else 1       # the decode pool (8.5 GB) is larger than L2 by itself
    ps = [p0] + [replace(p0, q=p0.q.clone(), k=p0.k.clone(), v=p0.v.clone()) for _ in range(R - 1)]
    kws = [x.capi_kw() for x in ps]

    def ours(i):
        x = ps[i % R]
        return ops.call_fwd(x.q, x.k, x.v, **kws[i % R])

    def theirs(i):
        x = ps[i % R]
        return ref(x.q, x.k, x.v, None, None, None, None, x.cu_seqlens_q, x.cu_seqlens_k, None, None, x.seqused_k,
                   x.max_seqlen_q, x.max_seqlen_k, x.page_table, None, x.leftpad_k, None, None, None, None, None, None,
                   x.softmax_scale, x.causal, x.window_left, x.window_right, x.softcap, True, None, 0, None, 0,
                   x.s_aux, 1, 0, None)

    def med(fn, n=20, warm=5):
        for i in range(warm):
            fn(i)
        torch.cuda.synchronize()
        ts = []
        for i in range(n):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn(i)
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        ts.sort()
        return ts[len(ts) // 2]

    o1, l1 = ours(0)
    r = theirs(0)
    torch.cuda.synchronize()
    fin = torch.isfinite(l1)
    t_o, t_r = med(ours), med(theirs)
    t_o2, t_r2 = med(ours), med(theirs)          # second pass: the order of the two does not decide the result
    t_o, t_r = min(t_o, t_o2), min(t_r, t_r2)
    print(json.dumps({"shape": name, "ours_ms": t_o, "reference_kernel_ms": t_r, "speedup": t_r / t_o,
                      "ours_TFLOPs": fl / t_o / 1e9, "reference_TFLOPs": fl / t_r / 1e9,
                      "ours_GBs": by / t_o / 1e6, "reference_GBs": by / t_r / 1e6,
                      "max_abs_dout": (o1.float() - r[0].float()).abs().max().item(),
                      "max_abs_dlse": (l1[fin] - r[1][fin]).abs().max().item()}))


def run_ab(args) -> None:
    """`--impl reference-kernel`: the reference's own `kernels/fa4_blackwell.cu` (built by oracle/build_ref.py into
    oracle/_ref/fa4_ref.so, never on the product path) against ours, shape by shape, each in a child process with a
    wall-clock limit (the reference's device waits are unbounded).  Shapes the reference cannot run are left out: the
    varlen + softcap configuration (its kernel for it has a recorded hang class, bench/scenarios.py:630-638), e4m3
    (unsupported there) and the long-context configuration (its launch asks for more shared memory than the GPU has)."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    shapes = [x for x in args.ab_shapes.split(",") if x]
    rows = []
    for name in shapes:
        if name in AB_SHAPES_STALLED:
            rows.append({"shape": name, "unavailable": "the reference's kernel did not return on this shape (recorded stall); not run again"})
            continue
        try:
            r = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference-kernel", "--ab-one", name],
                               stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=args.ab_timeout)
            line = [ln for ln in r.stdout.strip().splitlines() if ln.startswith("{")]
            rows.append(json.loads(line[-1]) if line else {"shape": name, "error": (r.stderr or r.stdout)[-400:]})
        except subprocess.TimeoutExpired:
            rows.append({"shape": name, "error": f"no result within {args.ab_timeout} s; child process ended"})
            break      # do not go on after a stall
    print(json.dumps({"impl": "reference-kernel", "n_gpus": 1, "rows": rows,
                      "method": "same device tensors, 4 rotating input copies, median of 20 CUDA-event timings, best of two passes"}))


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
    _time_steps.last_min = ms
    if world > 1:
        t = torch.tensor([ms, -ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
        ms, _time_steps.last_min = float(t[0].item()), -float(t[1].item())
    return ms


def _build_record():
    from flash_cuda_b200 import build as B
    try:
        return B.build_record()
    except Exception as e:
        return {"error": repr(e)}


def _tensor_bytes(*ts):
    return int(sum(t.numel() * t.element_size() for t in ts if t is not None))


def _repeat_batch(p, n):
    """The problem with its batch repeated n times (contiguous K/V, equal lengths): the shared problem of an
    n-GPU run, identical on every rank."""
    from dataclasses import replace
    if n == 1:
        return p
    B = len(p.q_lens)
    cu = lambda lens: torch.tensor([0] + list(torch.tensor(lens * n).cumsum(0).tolist()), dtype=torch.int32,
                                   device=p.q.device)
    rep = lambda t: None if t is None else t.repeat(n, *([1] * (t.dim() - 1)))
    return replace(p, q=rep(p.q), k=rep(p.k), v=rep(p.v), cu_seqlens_q=cu(p.q_lens), cu_seqlens_k=cu(p.k_lens),
                   q_descale=rep(p.q_descale), k_descale=rep(p.k_descale), v_descale=rep(p.v_descale),
                   q_lens=p.q_lens * n, k_lens=p.k_lens * n, name=f"{p.name}_x{n}")


def _tensor_roofline(tflops, peaks, dtype="bf16", sustained=False):
    """Tensor-bound roofline object.  The fp8 peak is DERIVED: twice the measured bf16 figure (the tensor cores'
    e4m3 rate is twice their bf16 rate); no fp8 GEMM was measured on this pool."""
    base = peaks["bf16_tflops_sustained"] if sustained else peaks["bf16_tflops"]
    peak = 2.0 * base if dtype == "fp8" else base
    src = peaks["source"] + (" (sustained: step of hundreds of ms)" if sustained else " (burst)")
    if dtype == "fp8":
        src += ", fp8 peak derived as 2 x bf16"
    return {"bound": "tensor", "achieved": tflops, "peak": peak, "unit": "TFLOP/s", "frac": tflops / peak,
            "peak_source": src}


def run_decode_only(args) -> None:
    """`--decode-only`: the two decode legs alone on one GPU, for profiler captures on a small pool."""
    from flash_cuda_b200 import capi, ops, workloads as W
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    ops.load(build_if_missing=False)
    res = {}
    for kv_dtype in ("bf16", "fp8"):
        dp = W.paged_decode_on_device(dev, seed=0, kv_dtype=kv_dtype, B=args.decode_batch, ctx_hi=args.decode_ctx_max)
        dout = torch.empty(dp.q.shape[0], dp.q.shape[1], dp.v.shape[-1], device=dev, dtype=torch.bfloat16)
        kw = dp.capi_kw()
        for _ in range(max(args.warmup, 3)):
            ops.call_fwd(dp.q, dp.k, dp.v, out=dout, **kw)
        ms = _time_steps(lambda i: ops.call_fwd(dp.q, dp.k, dp.v, out=dout, **kw), args.steps, None, 1)
        res[kv_dtype] = {"ms_per_step": ms, "GB/s": dp.kv_bytes() / (ms * 1e-3) / 1e9, "kv_bytes": dp.kv_bytes()}
        del dp, dout
        torch.cuda.empty_cache()
    print(json.dumps({"decode_only": res, "batch": args.decode_batch, "ctx_max": args.decode_ctx_max, "steps": args.steps}))


def run_ours(args) -> None:
    from flash_cuda_b200 import capi, multi_gpu as MG, ops, workloads as W

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
    warm = max(args.warmup, 10)      # untimed steps actually run before every timed region (reported as warmup_steps_run)

    # ---- headline: causal GQA prefill.  One SHARED problem of world x B sequences (the B-sequence batch of the
    # benchmark configuration repeated `world` times, identical on every rank); each rank computes its block of
    # kv heads through multi_gpu.fwd_head_sharded, so per-GPU work is that of the 1-GPU configuration (weak
    # scaling) and there is no collective.  R rotating copies: no step re-reads lines a recent step left in L2.
    host = W.causal_gqa_prefill(seed=0, B=args.batch)
    flops = host.flops()                       # per GPU: world x B sequences x (32 / world) heads
    R = 4
    from dataclasses import replace
    first = _repeat_batch(host.to(dev), world)
    sets = [first] + [replace(first, q=first.q.clone(), k=first.k.clone(), v=first.v.clone()) for _ in range(R - 1)]
    hq_loc = host.q.shape[1] // world
    outs = [torch.empty(sets[0].q.shape[0], hq_loc, host.v.shape[-1], device=dev, dtype=torch.bfloat16)
            for _ in range(R)]
    in_bytes = _tensor_bytes(host.q, host.k, host.v)

    def step(i):
        p = sets[i % R]
        MG.fwd_head_sharded(p.q, p.k, p.v, rank=rank, world=world, out=outs[i % R], **p.capi_kw())

    for i in range(warm):
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
    # Every step copies this rank's shard (its heads of every sequence) from pinned host memory and reads its
    # result back.  The three legs of a step run on three streams (copy-in, the op on the current stream, copy-out)
    # with two buffer sets, so step i+1's inputs travel while step i computes and step i-1's result travels back;
    # events order the legs of one step and protect each buffer until its previous user is done.
    e2e = None
    if not args.no_e2e:
        qs, ks = MG.head_slice(host.q.shape[1], host.k.shape[1], rank, world)
        hq_h = host.q[:, qs, :].repeat(world, 1, 1).contiguous().pin_memory()
        hk_h = host.k[:, ks, :].repeat(world, 1, 1).contiguous().pin_memory()
        hv_h = host.v[:, ks, :].repeat(world, 1, 1).contiguous().pin_memory()
        s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        cur = torch.cuda.current_stream(dev)
        dbuf = [(torch.empty(hq_h.shape, device=dev, dtype=hq_h.dtype), torch.empty(hk_h.shape, device=dev, dtype=hk_h.dtype),
                 torch.empty(hv_h.shape, device=dev, dtype=hv_h.dtype)) for _ in range(2)]
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
                    dbuf[b][0].copy_(hq_h, non_blocking=True)
                    dbuf[b][1].copy_(hk_h, non_blocking=True)
                    dbuf[b][2].copy_(hv_h, non_blocking=True)
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
               "h2d_bytes_per_step": _tensor_bytes(hq_h, hk_h, hv_h), "d2h_bytes_per_step": _tensor_bytes(h_out[0]),
               "overlap": "copy-in, op and copy-out of consecutive steps on three streams, two buffer sets"}
        del dbuf, obuf, h_out, hq_h, hk_h, hv_h
    del sets, outs
    torch.cuda.empty_cache()

    # ---- the other benchmark configurations, one object each (every rank runs its own copy; per-GPU figures,
    # `value` = per-GPU figure x ranks) ----
    def timed_leg(make, steps, rotate, work, unit_scale, extra):
        """make() -> problem on the host; `rotate` device copies are cycled so that no step finds its inputs in L2
        (or the one copy is larger than L2)."""
        try:
            p0 = make().to(dev)
            ps = [p0] + [replace(p0, q=p0.q.clone(), k=p0.k.clone(), v=p0.v.clone()) for _ in range(rotate - 1)]
            os_ = [torch.empty(p.q.shape[0], p.q.shape[1], p.v.shape[-1], device=dev, dtype=torch.bfloat16) for p in ps]
            kws = [p.capi_kw() for p in ps]

            def leg_step(i):
                j = i % rotate
                ops.call_fwd(ps[j].q, ps[j].k, ps[j].v, out=os_[j], **kws[j])

            for i in range(warm):
                leg_step(i)
            lms = _time_steps(leg_step, steps, dist, world)
            res = {"ms_per_step": lms, "ms_fastest_rank": _time_steps.last_min, "steps": steps, "work_per_step": work(ps[0]),
                   "per_gpu": work(ps[0]) / (lms * 1e-3) / unit_scale}
            res.update(extra(ps[0], res))
            del ps, os_
            torch.cuda.empty_cache()
            return res
        except Exception as e:  # reported, never hidden
            torch.cuda.empty_cache()
            return {"error": repr(e)}

    nsteps = max(3, min(args.steps, 100))
    legs = {}
    if not args.headline_only:
        # C1: dense non-causal B=2 H=8 S=512 (8 MB per copy: 32 rotating copies = 268 MB > L2); a latency figure
        legs["c1"] = timed_leg(lambda: W.dense_noncausal(seed=0), nsteps, 32, lambda p: p.flops(), 1e12,
                               lambda p, r: {"workload": "dense non-causal MHA bf16 B=2 H=8 S=512 d=128", "us_per_step": r["ms_per_step"] * 1e3,
                                             "unit": "TFLOP/s", "roofline": _tensor_roofline(r["per_gpu"], peaks),
                                             "kernels_per_step": ["fwd_prefill_tc_kernel"], "l2": "32 rotating copies (268 MB)",
                                             "note": "32 work items on 148 SMs: launch- and latency-bound, the TFLOP/s figure is informational"})
        # C2 in e4m3 (per-tensor descale)
        legs["c2_fp8"] = timed_leg(lambda: W.causal_gqa_prefill(seed=0, B=args.batch, dtype="fp8"), nsteps, 4,
                                   lambda p: p.flops(), 1e12,
                                   lambda p, r: {"workload": f"causal GQA prefill e4m3 (Q, K, V; per-tensor descale) B={args.batch} Hq=32 Hkv=8 S=4096 d=128",
                                                 "unit": "TFLOP/s", "roofline": _tensor_roofline(r["per_gpu"], peaks, "fp8"),
                                                 "kernels_per_step": ["fwd_prefill_tc_kernel (kind::f8f6f4)"], "l2": "4 rotating copies"})
        # C3: varlen + window + softcap + sink (468 MB of Q alone: larger than L2)
        legs["c3"] = timed_leg(lambda: W.varlen_window_softcap_sink(seed=0), max(3, min(args.steps, 30)), 1,
                               lambda p: p.flops(), 1e12,
                               lambda p, r: {"workload": "varlen packed causal prefill bf16, 16 sequences 128..8192, Hq=32 Hkv=8 d=128, window 4096, softcap 30, sink",
                                             "unit": "TFLOP/s", "roofline": _tensor_roofline(r["per_gpu"], peaks),
                                             "kernels_per_step": ["fwd_prefill_tc_kernel"], "l2": "inputs (0.7 GB) larger than L2",
                                             "note": "one tanh and one exp2 per score share the special-function unit"})

    # ---- decode workload: bf16 KV cache and e4m3 KV cache ----
    def decode_leg(kv_dtype):
        try:
            dp = W.paged_decode_on_device(dev, seed=rank, kv_dtype=kv_dtype, B=args.decode_batch)   # the pool is drawn on the GPU
            kvb = dp.kv_bytes()
            dout = torch.empty(dp.q.shape[0], dp.q.shape[1], dp.v.shape[-1], device=dev, dtype=torch.bfloat16)
            nspl = capi.num_splits(dp.q, dp.k, dp.v, **dp.capi_kw())

            def dstep(i):
                ops.call_fwd(dp.q, dp.k, dp.v, out=dout, **dp.capi_kw())

            for i in range(warm):
                dstep(i)
            dms = _time_steps(dstep, nsteps, dist, world)
            gbs = kvb / (dms * 1e-3) / 1e9
            res = {
                "metric": f"paged decode HBM GB/s (B={args.decode_batch} q_len=1 ctx 1k..32k page 64 Hq=32 Hkv=8 d=128 {kv_dtype} KV, "
                          "leftpad 0..63)",
                "value": gbs * world, "unit": "GB/s", "ms_per_step": dms, "kv_bytes_per_step": kvb,
                "num_splits": nspl,
                "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                             "frac": gbs / peaks["hbm_gbs"], "traffic": NCU_DECODE_TRAFFIC[kv_dtype],
                             "traffic_source": "ncu dram__bytes_read+write per launch of this configuration (profiles/)",
                             "peak_source": peaks["source"]},
                "kernels_per_step": ["sched_kernel", "fwd_decode_kernel"],
                "l2": f"KV pool ({kvb / 1e9:.2f} GB) larger than L2",
            }
            del dp, dout
            torch.cuda.empty_cache()
            return res
        except Exception as e:  # reported, never hidden
            torch.cuda.empty_cache()
            return {"error": repr(e)}

    decode = None if (args.no_decode or args.headline_only) else decode_leg("bf16")
    decode_fp8 = None if (args.no_decode or args.headline_only) else decode_leg("fp8")

    # ---- long context (C5): KV range sharded over the ranks, strong scaling, through multi_gpu.fwd_kv_sharded ----
    longctx = None
    if not (args.no_longctx or args.headline_only):
        try:
            longctx = _longctx_leg(args, dist, rank, world, dev, peaks)
        except Exception as e:
            torch.cuda.empty_cache()
            longctx = {"error": repr(e)}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    for name, leg in legs.items():
        if "per_gpu" in leg:
            leg["value"] = leg["per_gpu"] * world
    cpu = cpu_baseline() if (world == 1 and not args.no_cpu) else None
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded N(0,1), random-permuted page table for decode)",
        "config": {"workload": f"causal GQA prefill B={args.batch} Hq=32 Hkv=8 S=4096 d=128 bf16 per GPU",
                   "parallelism": (f"one shared problem of {world}x{args.batch} sequences; the 8 kv heads (and their q heads) "
                                   f"sharded over {world} GPU(s) by multi_gpu.fwd_head_sharded, no collective"),
                   "global_batch": world * args.batch,
                   "l2": f"{R} rotating input sets of {in_bytes * world / 1e6:.0f} MB each (> L2 {L2_BYTES / 1e6:.0f} MB)",
                   "flops_per_step_per_gpu": flops},
        "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": per_gpu / peaks["bf16_tflops"], "traffic": NCU_PREFILL_TRAFFIC_PER_BATCH * args.batch,
                     "traffic_source": "ncu dram__bytes_read+write of a B=2 launch, scaled by B (profiles/)",
                     "peak_source": peaks["source"], "kernel": "fwd_prefill_tc_kernel", "launch_ms": ms},
        "e2e": e2e, "gpu_launches": args.steps, "clocks": clocks, "decode": decode, "decode_fp8": decode_fp8,
        "c1": legs.get("c1"), "c2_fp8": legs.get("c2_fp8"), "c3": legs.get("c3"), "c5": longctx, "longctx": longctx,
        "cpu_baseline": cpu,
        "kernels_per_step": {"prefill": ["fwd_prefill_tc_kernel"], "decode": ["sched_kernel", "fwd_decode_kernel"]},
        "build": _build_record(),
    }
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def _longctx_leg(args, dist, rank, world, dev, peaks, merge="auto"):
    """B=1, a chunk of 4096 query rows against a paged KV of 524288 tokens (page 64), 128 heads, head_dim 192 /
    head_dim_v 128, causal, bf16.  The key range is split evenly over the ranks (strong scaling); each rank's kernel
    writes its fp32 partial into the gather buffer, ONE all-gather + the merge kernel finish the step, all inside
    the timed region; the time between the end of the attention kernel and the end of the merge is reported apart."""
    from flash_cuda_b200 import multi_gpu as MG, workloads as W
    q_len, k_len, heads = 4096, args.longctx_keys, 128
    merge = MG.resolve_merge(merge, world, q_len)
    per = k_len // world
    p = W.long_context(dev, seed=0, q_len=q_len, k_len=k_len, heads=heads, k_begin=rank * per, k_end=(rank + 1) * per)
    pairs = q_len * (k_len - q_len) + q_len * (q_len + 1) // 2     # unmasked pairs per head of the WHOLE problem
    flops = 2.0 * (192 + 128) * heads * pairs
    marks = []

    def step(i, rec=None):
        MG.fwd_kv_sharded(p.q, p.k, p.v, page_table_local=p.page_table, seqused_k_local=p.seqused_k,
                          cu_seqlens_q=p.cu_seqlens_q, max_seqlen_q=q_len, max_seqlen_k_local=per,
                          softmax_scale=p.softmax_scale, causal=True, rank=rank, world=world, merge=merge, marks=rec)

    for i in range(2):
        step(i)
    steps = max(1, min(args.steps, 3))
    ms = _time_steps(lambda i: step(i, marks), steps, dist, world)
    # Time from the end of a rank's attention kernel to the end of its merge.  On a rank whose kernel ends early
    # (the last rank is causal on its shard, and GPUs differ by a few per cent) that span also holds the wait for the
    # slowest kernel; the rank whose kernel ends last waits for nobody, so the MINIMUM over ranks is what the
    # collective and the merge add to the step.  The maximum is reported beside it.
    merge_ms = merge_ms_max = 0.0
    if world > 1:
        mine = sum(marks[2 * i].elapsed_time(marks[2 * i + 1]) for i in range(steps)) / steps
        t = torch.tensor([mine, -mine], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        merge_ms, merge_ms_max = float(t[0].item()), -float(t[1].item())
    val = flops / (ms * 1e-3) / 1e12
    kvgb = (p.k.numel() + p.v.numel()) * 2 / 1e9
    del p
    torch.cuda.empty_cache()
    return {"metric": "long-context prefill TFLOP/s, whole job (q 4096 x paged KV 524288, 128 heads, hd192/hdv128, causal, bf16)",
            "value": val, "unit": "TFLOP/s", "ms_per_step": ms, "steps": steps, "scaling": "strong",
            "gather_and_merge_ms": merge_ms, "gather_and_merge_frac": merge_ms / ms if ms > 0 else None,
            "gather_and_merge_ms_max_over_ranks": merge_ms_max,
            "parallelism": (f"KV range split over {world} GPU(s) by multi_gpu.fwd_kv_sharded; fp32 partials written into the "
                            f"gather buffer by the kernel, one all-gather (in place), merge kernel reads it in place"
                            if merge == "all_gather" else
                            f"KV range split over {world} GPU(s); partial rows exchanged by all-to-all, merged per row block, result all-gathered"),
            "roofline": _tensor_roofline(val / world, peaks, sustained=True),
            "merge": merge if world > 1 else None,
            "kernels_per_step": ["fwd_prefill_tc_kernel"] + ([] if world == 1 else
                                 ["ncclAllGather (NCCL)", "combine_kernel"] if merge == "all_gather" else
                                 ["ncclSendRecv x2 (NCCL all-to-all)", "combine_kernel", "ncclAllGather x2 (NCCL)"]),
            "l2": f"KV shard {kvgb:.1f} GB per GPU (> L2)"}


def run_longctx(args) -> None:
    """`--workload longctx`: only the long-context leg (see _longctx_leg), as the headline of its own JSON line."""
    from flash_cuda_b200 import ops
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
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    leg = _longctx_leg(args, dist, rank, world, dev, peaks, merge=args.longctx_merge)
    clocks = sampler.stop() if rank == 0 else {}
    if rank == 0:
        print(json.dumps(dict(leg, n_gpus=world, warmup=2, higher_is_better=True, vs_baseline=None, dtype="bf16",
                              data="synthetic (N(0,1) drawn on the device, seeded)",
                              config={"workload": f"long-context prefill q=4096 k={args.longctx_keys} heads=128 hd192/hdv128 page 64",
                                      "merge": args.longctx_merge},
                              gpu_launches=leg["steps"] * (1 if world == 1 else 2), clocks=clocks)))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-kernel"])
    ap.add_argument("--ab-shapes", default=",".join(AB_SHAPES), help="--impl reference-kernel: shapes to compare")
    ap.add_argument("--ab-one", default=None, help=argparse.SUPPRESS)
    ap.add_argument("--ab-timeout", type=float, default=240.0, help="--impl reference-kernel: seconds per shape")
    ap.add_argument("--no-decode", action="store_true", help="skip the decode workloads")
    ap.add_argument("--no-longctx", action="store_true", help="skip the long-context (KV-sharded) leg")
    ap.add_argument("--headline-only", action="store_true", help="only the headline prefill leg (profiler captures)")
    ap.add_argument("--decode-only", action="store_true", help="only the two decode legs (profiler captures)")
    ap.add_argument("--decode-ctx-max", type=int, default=32768, help="--decode-only: longest context (captures use a smaller pool)")
    ap.add_argument("--decode-batch", type=int, default=128, help="decode batch (128 = the benchmark configuration; "
                    "smaller values are for profiler captures only)")
    ap.add_argument("--longctx-merge", default="auto", choices=["auto", "all_gather", "all_to_all"])
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
    elif args.impl == "reference-kernel":
        run_ab_one(args.ab_one) if args.ab_one else run_ab(args)
    elif args.workload == "longctx":
        run_longctx(args)
    elif args.decode_only:
        run_decode_only(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
