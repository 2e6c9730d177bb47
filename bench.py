#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline ("step" = one forward pass over one synthetic batch): dense causal
bf16 prefill, B=4, H=32, S=4096, D=128 per GPU (benchmark config 2), reported
as whole-job TFLOP/s with the causal FLOP count 4*D*S(S+1)/2 per (b, h).
For N > 1 launch under torchrun; every rank runs its own batch of 4 sequences
(weak scaling, no collective on the data path) and the slowest rank's time is
used.  The same line carries the GQA decoding (config 3), block-sparse prefill
(config 4) and block-sparse decoding (config 5) results under "other".

`--impl reference` times the reference's CPU path (its naive torch attention,
restated in oracle/attention_oracle.py because the reference checkout does
not exist on the GPU box) on the host cores.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "prefill attn TFLOP/s & decode KV HBM GB/s per B200, at 1/2/4/8 GPUs"
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the
# ncu captures summarised under profiles/ (same workloads as below)
TRAFFIC = {"cfg2": 409.803520e6 + 120.196096e6, "cfg3": 1.301270e9 + 6.896384e6, "cfg2_backward": 809.810176e6 + 491.803392e6,
           "cfg4": 619.421184e6 + 128.075264e6, "cfg5": 2.148035e9 + 14.810368e6}
WORKLOAD = "cfg2: dense causal prefill bf16 B=4 H=32 S=4096 D=128 per GPU"


# ----------------------------------------------------------------------------
def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(tflops=d["bf16_tflops"], tflops_sustained=d.get("bf16_tflops_sustained"),
                    gbs=d["hbm_gbs"], source="measured")
    return dict(tflops=1590.0, tflops_sustained=1400.0, gbs=6650.0, source="fallback")


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 100 ms while timing."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for n, val in zip(names, f[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def time_steps(fn, steps, warmup, stream_sync, barrier):
    """Warm up, then time exactly `steps` calls with CUDA events on the current
    stream, bracketed by barrier + synchronize.  Returns ms per step."""
    for _ in range(warmup):
        fn()
    stream_sync(); barrier(); stream_sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    stream_sync(); barrier(); stream_sync()
    return e0.elapsed_time(e1) / steps


# ----------------------------------------------------------------------------
def cpu_prefill_sample(seconds_hint=12.0):
    """The reference's CPU path (flash_attn_torch restated) on a bounded sample of
    config 2: whole 4096-token, 32-head sequences, repeated until the time hint
    is used up (at least one)."""
    from oracle import attention_oracle as orc
    from tritonops_b200 import workloads
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    S, D, H = 4096, 128, 32
    g = torch.Generator().manual_seed(1)
    q = torch.randn(1, S, H, D, generator=g).to(torch.bfloat16)
    k = torch.randn(1, S, H, D, generator=g).to(torch.bfloat16)
    v = torch.randn(1, S, H, D, generator=g).to(torch.bfloat16)
    cu = torch.tensor([0, S], dtype=torch.int32)
    n, t0 = 0, time.perf_counter()
    while True:
        orc.dense_prefill_refpath(q, k, v, cu)
        n += 1
        dt = time.perf_counter() - t0
        if dt >= seconds_hint or n >= 64:
            break
    flops = workloads.causal_flops([S], H, D) * n
    return dict(value=flops / dt / 1e12, unit="TFLOP/s", cores=threads, kind="port",
                sample=f"{n} sequence(s) of cfg2 (S=4096, H=32, D=128, causal bf16; the full step has 4), "
                       f"{dt:.1f} s, naive torch attention of flash_attn_triton.py:877-915 restated",
                seconds=dt)


def run_reference(args, rank, world):
    """Reference arm: the reference's own CPU implementation of the path (port)."""
    if rank != 0:
        return
    vals = []
    # seconds of CPU work per step; the environment override only exists so that the contract
    # test of this arm can run in a few seconds
    budget = float(os.environ.get("B200ATTN_BENCH_CPU_SECONDS", "12"))
    cpu_prefill_sample(min(2.0, budget))                  # warm-up (thread pool, allocator)
    steps = max(1, min(args.steps, 3))
    last = None
    for _ in range(steps):
        last = cpu_prefill_sample(budget)
        vals.append(last)
    val = sum(v["value"] for v in vals) / len(vals)
    ms = sum(v["seconds"] for v in vals) / len(vals) * 1e3
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": 1, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic N(0,1), seeded", "config": {"workload": WORKLOAD,
                                                       "note": "each step is a bounded sample of the workload on host cores"},
        "cpu_baseline": {k: last[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    line["cpu_baseline"]["value"] = val
    print(json.dumps(line))


# ----------------------------------------------------------------------------
def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist
    from tritonops_b200 import ops, workloads
    from tritonops_b200.flash_attn_triton.flash_attn_triton import flash_attn_triton_fwd
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    pk = peaks()

    def sync():
        torch.cuda.synchronize(dev)

    def barrier():
        if world > 1:
            dist.barrier()

    def reduce_max(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sampler = ClockSampler(local_rank)
    LOG2E = 1.4426950408889634
    if args.only != "all":
        return run_single(args, dev, sync, barrier, pk)

    # ---------------- headline: config 2, each rank its own 4 sequences (seed 1 + rank)
    w = workloads.dense_causal(4, 32, 4096, 128, 1 + rank, dev, name="cfg2")
    sm_scale = w.scale * LOG2E

    def step():
        return flash_attn_triton_fwd(w.q, w.k, w.v, w.cu_seqlens, sm_scale, max_seqlen=w.max_seqlen)

    l0 = ops.launch_counter
    step()
    launches = (ops.launch_counter - l0) * args.steps     # kernels of ours per timed region
    sampler.start()
    ms = reduce_max(time_steps(step, args.steps, args.warmup, sync, barrier))
    total_flops = w.flops * world
    value = total_flops / ms / 1e9                       # TFLOP/s, whole job
    per_launch_tflops = w.flops / ms / 1e9               # this GPU's kernel (1 launch per step)

    # ---------------- end to end: pinned host buffers in, O + LSE back out, every step
    hq, hk, hv = (t.cpu().pin_memory() for t in (w.q, w.k, w.v))
    ho = torch.empty(w.q.shape, dtype=w.q.dtype).pin_memory()
    hl = torch.empty(w.q.shape[:3], dtype=torch.float32).pin_memory()
    dq, dk, dv = (torch.empty_like(t) for t in (w.q, w.k, w.v))

    # the package's host-buffer entry point: per sequence copy in / attend / copy out on three
    # streams, so the PCIe transfers overlap the kernels and each other (same arithmetic as above)
    from tritonops_b200.host import HostPrefill
    pipe = HostPrefill(dev)
    cu_host = [int(x) for x in w.cu_seqlens.cpu()]
    del dq, dk, dv

    def e2e_step():
        pipe.run(hq, hk, hv, cu_host, ho, hl, scale=sm_scale, scale_has_log2e=True, causal=True, lse_base2=True)

    e2e_steps = max(3, min(args.steps, 10))
    ms_e2e = reduce_max(time_steps(e2e_step, e2e_steps, 3, sync, barrier))
    h2d = 3 * w.q.numel() * w.q.element_size() if w.k.shape == w.q.shape else \
        (w.q.numel() + 2 * w.k.numel()) * w.q.element_size()
    d2h = ho.numel() * ho.element_size() + hl.numel() * 4
    del hq, hk, hv, ho, hl, pipe

    other = {}
    # ---------------- config 3: GQA decoding (HBM bound)
    try:
        w3 = workloads.cfg3(dev)
        f3 = lambda: ops.decode(w3.q, w3.k_cache, w3.v_cache, cu_seqlens=w3.cu_seqlens,
                                max_seqlen=w3.max_seqlen)
        ms3 = reduce_max(time_steps(f3, max(args.steps, 10), 3, sync, barrier))
        gbs = w3.kv_bytes / ms3 / 1e6
        f3b = lambda: ops.decode(w3.q, w3.k_cache, w3.v_cache, cu_seqlens=w3.cu_seqlens,
                                 max_seqlen=w3.max_seqlen, chunk=512)
        gbs512 = w3.kv_bytes / reduce_max(time_steps(f3b, max(args.steps, 10), 3, sync, barrier)) / 1e6
        other["cfg3_gqa_decode"] = {
            "value": gbs * world, "unit": "GB/s", "ms_per_step": ms3,
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": pk["gbs"], "unit": "GB/s",
                         "frac": gbs / pk["gbs"], "frac_of_nominal_8TBs": gbs / 8000.0,
                         "traffic": TRAFFIC["cfg3"], "algorithmic_bytes": w3.kv_bytes},
            "config": {"workload": "cfg3: GQA decode bf16 B=64 Hq=32 Hkv=8 D=128, cache 8192, "
                                   "len U[1024,8192] seed 2, split chunks chosen by the library (2048 here)",
                       "with_512_key_chunks_GBs": gbs512,
                       "l2": "2.6 GB of KV streamed per step, far larger than L2"}}
        del w3
    except Exception as e:  # keep the headline even if a secondary config fails
        other["cfg3_gqa_decode"] = {"error": repr(e)}
    # ---------------- config 2 backward (dQ, dK, dV; 2.5x the forward FLOPs)
    try:
        o2, lse2 = flash_attn_triton_fwd(w.q, w.k, w.v, w.cu_seqlens, sm_scale, max_seqlen=w.max_seqlen)
        do2 = torch.randn(w.q.shape, device=dev, dtype=torch.float32).to(w.q.dtype)
        fb = lambda: ops.prefill_bwd(w.q, w.k, w.v, o2, do2, lse2, cu_seqlens=w.cu_seqlens,
                                     max_seqlen=w.max_seqlen, scale=sm_scale, scale_has_log2e=True,
                                     lse_base2=True)
        msb = reduce_max(time_steps(fb, max(args.steps // 2, 5), 3, sync, barrier))
        tfb = 2.5 * w.flops / msb / 1e9
        other["cfg2_backward"] = {
            "value": tfb * world, "unit": "TFLOP/s", "ms_per_step": msb,
            "roofline": {"bound": "tensor", "achieved": tfb, "peak": pk["tflops"], "unit": "TFLOP/s",
                         "frac": tfb / pk["tflops"], "traffic": TRAFFIC["cfg2_backward"]},
            "config": {"workload": "backward of cfg2 (dense causal bf16 B=4 H=32 S=4096 D=128): dQ, dK, dV",
                       "flops": "2.5 x the causal forward count (five products instead of two)"}}
        del o2, lse2, do2
    except Exception as e:
        other["cfg2_backward"] = {"error": repr(e)}
    # ---------------- config 4: block-sparse causal prefill (tensor bound, gathered KV blocks)
    try:
        from tritonops_b200.flash_attn_triton.flash_attn_sparse_attn_triton import flash_attn_block_sparse
        w4 = workloads.cfg4(dev)
        f4 = lambda: flash_attn_block_sparse(w4.q, w4.k, w4.v, w4.cu_seqlens, w4.block_idx, w4.block_cnt,
                                             max_seqlen=w4.max_seqlen)
        ms4 = reduce_max(time_steps(f4, max(args.steps, 10), 3, sync, barrier))
        tf4 = w4.flops / ms4 / 1e9
        other["cfg4_block_sparse_prefill"] = {
            "value": tf4 * world, "unit": "TFLOP/s", "ms_per_step": ms4,
            "roofline": {"bound": "tensor", "achieved": tf4, "peak": pk["tflops"], "unit": "TFLOP/s",
                         "frac": tf4 / pk["tflops"], "frac_of_nominal_2250": tf4 / 2250.0,
                         "traffic": TRAFFIC["cfg4"]},
            "config": {"workload": "cfg4: block-sparse causal prefill bf16 B=2 H=16 S=16384 D=128, 64x64 "
                                   "blocks, 8-block window + Bernoulli(0.1) earlier blocks seed 3",
                       "flops": "4*D per visible (query,key) pair of the listed blocks only"}}
        del w4
    except Exception as e:
        other["cfg4_block_sparse_prefill"] = {"error": repr(e)}
    # ---------------- config 5: top-k block decoding (HBM bound, gathered blocks)
    try:
        w5 = workloads.cfg5(dev)
        f5 = lambda: ops.decode(w5.q, w5.k_cache, w5.v_cache, seqlens=w5.seqlens,
                                sparsity=ops.BLOCK_LIST, block_idx=w5.block_idx, block_size=64)
        ms5 = reduce_max(time_steps(f5, max(args.steps, 10), 3, sync, barrier))
        gbs5 = w5.kv_bytes / ms5 / 1e6
        other["cfg5_block_sparse_decode"] = {
            "value": gbs5 * world, "unit": "GB/s", "ms_per_step": ms5,
            "roofline": {"bound": "hbm", "achieved": gbs5, "peak": pk["gbs"], "unit": "GB/s",
                         "frac": gbs5 / pk["gbs"], "frac_of_nominal_8TBs": gbs5 / 8000.0,
                         "traffic": TRAFFIC["cfg5"], "algorithmic_bytes": w5.kv_bytes},
            "config": {"workload": "cfg5: block-sparse decode bf16 B=32 H=32 D=128, KV 32768 = 512 "
                                   "blocks of 64, 64 blocks per (b,h) seed 4"}}
        del w5
    except Exception as e:
        other["cfg5_block_sparse_decode"] = {"error": repr(e)}
    # ---------------- rows either side of the hot path: paged decoding and RMSNorm (HBM bound)
    try:
        w3 = workloads.cfg3(dev)
        page, B3, cap = 64, w3.k_cache.shape[0], w3.k_cache.shape[1]
        n_pages = B3 * cap // page
        gperm = torch.Generator(device="cpu").manual_seed(7)
        table = torch.randperm(n_pages, generator=gperm).to(torch.int32).view(B3, cap // page).to(dev)
        # scatter the padded caches into pools so that page table[b][i] holds keys i*page.. of sequence b
        kp = torch.empty(n_pages, page, *w3.k_cache.shape[2:], device=dev, dtype=w3.k_cache.dtype)
        vp = torch.empty_like(kp)
        kp[table.view(-1).long()] = w3.k_cache.view(n_pages, page, *w3.k_cache.shape[2:])
        vp[table.view(-1).long()] = w3.v_cache.view(n_pages, page, *w3.v_cache.shape[2:])
        fpg = lambda: ops.paged_decode(w3.q, kp, vp, table, w3.seqlens, max_seqlen=w3.max_seqlen)
        same = bool(torch.equal(fpg(), ops.decode(w3.q, w3.k_cache, w3.v_cache, seqlens=w3.seqlens,
                                                  max_seqlen=w3.max_seqlen)))
        msp = reduce_max(time_steps(fpg, max(args.steps, 10), 3, sync, barrier))
        gbp = w3.kv_bytes / msp / 1e6
        other["cfg3_paged_decode"] = {
            "value": gbp * world, "unit": "GB/s", "ms_per_step": msp,
            "roofline": {"bound": "hbm", "achieved": gbp, "peak": pk["gbs"], "unit": "GB/s", "frac": gbp / pk["gbs"],
                         "traffic": None, "algorithmic_bytes": w3.kv_bytes},
            "config": {"workload": "config 3's sequences in 64-key pages scattered at random over a pool, found "
                                   "through a page table", "bit_identical_to_padded_decode": same}}
        del w3, kp, vp, table
    except Exception as e:
        other["cfg3_paged_decode"] = {"error": repr(e)}
    try:
        rows_n, dim_n = 65536, 4096
        xn = torch.randn(rows_n, dim_n, device=dev, dtype=torch.bfloat16)
        wn = torch.ones(dim_n, device=dev, dtype=torch.bfloat16)
        dyn = torch.randn_like(xn)
        _, rstd_n = ops.rmsnorm_fwd(xn, wn, 1e-6)
        nbytes = xn.numel() * 2
        msf = reduce_max(time_steps(lambda: ops.rmsnorm_fwd(xn, wn, 1e-6), max(args.steps, 10), 3, sync, barrier))
        msb = reduce_max(time_steps(lambda: ops.rmsnorm_bwd(dyn, xn, wn, rstd_n), max(args.steps, 10), 3, sync, barrier))
        other["rmsnorm_bf16_65536x4096"] = {
            "value": 2 * nbytes / msf / 1e6 * world, "unit": "GB/s", "ms_per_step": msf,
            "roofline": {"bound": "hbm", "achieved": 2 * nbytes / msf / 1e6, "peak": pk["gbs"], "unit": "GB/s",
                         "frac": 2 * nbytes / msf / 1e6 / pk["gbs"], "traffic": None, "algorithmic_bytes": 2 * nbytes},
            "backward": {"value": 3 * nbytes / msb / 1e6 * world, "unit": "GB/s", "ms_per_step": msb,
                         "frac": 3 * nbytes / msb / 1e6 / pk["gbs"], "algorithmic_bytes": 3 * nbytes},
            "config": {"workload": "RMSNorm forward (x in, y out) and backward (dy, x in, dx out) over 65536 rows "
                                   "of 4096 bf16"}}
        del xn, wn, dyn, rstd_n
    except Exception as e:
        other["rmsnorm_bf16_65536x4096"] = {"error": repr(e)}
    # ---------------- config 1: the reference's own small case (latency bound), in microseconds
    try:
        w1 = workloads.cfg1(dev)
        f1 = lambda: ops.prefill(w1.q, w1.k, w1.v, cu_seqlens=w1.cu_seqlens, max_seqlen=w1.max_seqlen,
                                 causal=False, scale=w1.scale)
        us_call = reduce_max(time_steps(f1, 200, 20, sync, barrier)) * 1e3      # call rate incl. the Python host path
        graph_us = None
        try:
            side = torch.cuda.Stream(dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                f1()
                g1 = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g1, stream=side):
                    for _ in range(20):
                        f1()
            torch.cuda.current_stream(dev).wait_stream(side)
            graph_us = reduce_max(time_steps(g1.replay, 50, 5, sync, barrier)) * 1e3 / 20
            del g1
        except Exception:
            graph_us = None
        other["cfg1_small_noncausal"] = {
            "value": graph_us if graph_us is not None else us_call, "unit": "us per call",
            "per_call_with_python_host_path_us": us_call, "per_launch_replayed_from_a_cuda_graph_us": graph_us,
            "config": {"workload": "cfg1: non-causal fp16 B=1 H=2 S=128 D=64 (8.4 MFLOP, 128 KiB): launch-latency "
                                   "bound, one CTA"}}
        del w1
    except Exception as e:
        other["cfg1_small_noncausal"] = {"error": repr(e)}
    clocks = sampler.stop()          # sampled over every timed region above
    torch.cuda.empty_cache()

    if rank != 0:
        return
    cpu = cpu_prefill_sample(12.0)
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic N(0,1), seeded",
        "config": {"workload": WORKLOAD, "global_batch": 4 * world, "sharding": "by sequence, no collective",
                   "flops_per_gpu_step": w.flops,
                   "l2": "inputs+outputs 514 MiB per step, larger than the 126 MB L2; no flush",
                   "api": "flash_attn_triton_fwd(q,k,v,cu_seq_lens,sm_scale) -> (o, lse2)"},
        "roofline": {"bound": "tensor", "achieved": per_launch_tflops, "peak": pk["tflops"],
                     "unit": "TFLOP/s", "frac": per_launch_tflops / pk["tflops"],
                     "peak_source": pk["source"] + " cuBLAS bf16 burst",
                     "frac_of_sustained": per_launch_tflops / pk["tflops_sustained"] if pk["tflops_sustained"] else None,
                     "frac_of_nominal_2250": per_launch_tflops / 2250.0,
                     "traffic": TRAFFIC["cfg2"], "traffic_unit": "bytes per launch (ncu)",
                     "algorithmic_bytes": 4 * w.q.numel() * 2 + w.q.numel() // 128 * 4},
        "cpu_baseline": {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": total_flops / ms_e2e / 1e9, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "api": "tritonops_b200.host.HostPrefill.run(pinned q, k, v -> pinned o, lse2), one sequence per "
                       "copy-in / kernel / copy-out stage on three streams"},
        "gpu_launches": launches,
        "clocks": clocks,
        "other": other,
    }
    print(json.dumps(line))


def run_single(args, dev, sync, barrier, pk):
    """One kernel's loop only (used for ncu captures; prints a short JSON line)."""
    from tritonops_b200 import ops, workloads
    if args.only == "prefill":
        w = workloads.dense_causal(4, 32, 4096, 128, 1, dev, name="cfg2")
        fn = lambda: ops.prefill(w.q, w.k, w.v, cu_seqlens=w.cu_seqlens, max_seqlen=w.max_seqlen)
        work, unit, peak = w.flops / 1e9, "TFLOP/s", pk["tflops"]
    elif args.only == "decode":
        w = workloads.cfg3(dev)
        fn = lambda: ops.decode(w.q, w.k_cache, w.v_cache, cu_seqlens=w.cu_seqlens, max_seqlen=w.max_seqlen)
        work, unit, peak = w.kv_bytes / 1e6, "GB/s", pk["gbs"]
    elif args.only == "backward":
        w = workloads.dense_causal(4, 32, 4096, 128, 1, dev, name="cfg2")
        o, lse = ops.prefill(w.q, w.k, w.v, cu_seqlens=w.cu_seqlens, max_seqlen=w.max_seqlen)
        d_o = torch.randn(o.shape, device=dev, dtype=torch.float32).to(o.dtype)
        fn = lambda: ops.prefill_bwd(w.q, w.k, w.v, o, d_o, lse, cu_seqlens=w.cu_seqlens, max_seqlen=w.max_seqlen)
        work, unit, peak = 2.5 * w.flops / 1e9, "TFLOP/s", pk["tflops"]
    elif args.only == "sparse_prefill":
        w = workloads.cfg4(dev)
        fn = lambda: ops.prefill(w.q, w.k, w.v, cu_seqlens=w.cu_seqlens, max_seqlen=w.max_seqlen,
                                 sparsity=ops.BLOCK_LIST, block_idx=w.block_idx, block_cnt=w.block_cnt)
        work, unit, peak = w.flops / 1e9, "TFLOP/s", pk["tflops"]
    else:
        # (sparse_decode_small: a quarter of config 5's batch, 4.3 GB of cache, for ncu captures)
        w = workloads.cfg5(dev, B=8) if args.only == "sparse_decode_small" else workloads.cfg5(dev)
        fn = lambda: ops.decode(w.q, w.k_cache, w.v_cache, seqlens=w.seqlens, sparsity=ops.BLOCK_LIST,
                                block_idx=w.block_idx, block_size=64)
        work, unit, peak = w.kv_bytes / 1e6, "GB/s", pk["gbs"]
    ms = time_steps(fn, args.steps, args.warmup, sync, barrier)
    print(json.dumps({"only": args.only, "ms_per_step": ms, "value": work / ms, "unit": unit,
                      "frac_of_measured_peak": work / ms / peak}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--only", default="all",
                    choices=["all", "prefill", "decode", "backward", "sparse_prefill", "sparse_decode", "sparse_decode_small"],
                    help="profiling aid: run one kernel's timed loop and print a short line")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
