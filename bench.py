#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline ("step" = one forward pass over one synthetic batch): dense causal bf16 prefill,
B=4, H=32, S=4096, D=128 (benchmark config 2), reported as whole-job TFLOP/s with the causal
FLOP count 4*D*S(S+1)/2 per (b, h).  For N > 1 launch under torchrun: the batch's 128
(sequence x KV head) units are split contiguously over the ranks (strong scaling, no collective
on the data path), the slowest rank's time is used, and the gathered outputs are compared bit
for bit with one GPU's.  The K-step region is repeated and the median region is the headline;
a region of at least two seconds gives the figure the board sustains at its power cap.

The same line carries, as entries of `roofline`, the GQA decoding (config 3), block-sparse
prefill (config 4), block-sparse decoding (config 5), the backward of config 2, paged decoding
and RMSNorm, each with its fraction of the measured peak and a max-abs error against fp32 math
computed outside the timed region; `cpu_baseline` holds the reference's CPU path for every
config, timed on the host cores before any GPU work, and `roofline.reference_triton_gpu` the
reference's own Triton kernels timed on the same GPU.

`--impl reference` times the reference's CPU path (its naive torch attention, restated in
oracle/attention_oracle.py because the reference checkout does not exist on the GPU box) on the
host cores.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "prefill attn TFLOP/s & decode KV HBM GB/s per B200, at 1/2/4/8 GPUs"
WORKLOAD = "cfg2: dense causal prefill bf16 B=4 H=32 S=4096 D=128"
CFG2 = dict(B=4, H=32, S=4096, D=128)
LOG2E = 1.4426950408889634
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the named kernel and the ncu summary
# the figure comes from (same workload unless the summary says it was scaled)
TRAFFIC = {
    "cfg2": (412.162816e6 + 119.906816e6, "profiles/prefill_cfg2_ncu.md"),
    "cfg3": (1.301250e9 + 6.312448e6, "profiles/decode_cfg3_ncu.md"),
    "cfg2_backward": (824.896512e6 + 490.286848e6, "profiles/backward_cfg2_ncu.md"),
    "cfg4": (614.754816e6 + 124.699136e6, "profiles/sparse_prefill_cfg4_ncu.md"),
    "cfg5": (4 * (537.079552e6 + 4.031488e6), "profiles/sparse_decode_cfg5_ncu.md (batch 8 capture x 4)"),
    "paged_cfg3": (1.301388e9 + 6.204160e6, "profiles/paged_decode_cfg3_ncu.md"),
    "rmsnorm_fwd": (537.041920e6 + 480.131072e6, "profiles/rmsnorm_ncu.md (one cold launch: 57 MB of the output still in L2)"),
    "rmsnorm_bwd": (1.074061e9 + 480.250624e6, "profiles/rmsnorm_ncu.md (one cold launch)"),
}


def traffic(key):
    b, src = TRAFFIC[key]
    return {"traffic": b, "traffic_source": src}


def static_config():
    """What both arms print as `config`: the workload, independent of who measures it."""
    c = CFG2
    return {"workload": WORKLOAD, "global_batch": c["B"], "heads": c["H"], "seq_len": c["S"], "head_dim": c["D"],
            "causal": True,
            "flops_per_step": 4.0 * c["B"] * c["H"] * c["D"] * c["S"] * (c["S"] + 1) / 2,
            "sharding": "N=1: one GPU.  N>1: the 128 (sequence x KV head) units split contiguously over the "
                        "ranks (strong scaling), no collective on the data path",
            "l2": "inputs + outputs 514 MiB per step, larger than the 126 MB L2; no flush",
            "api": "flash_attn_triton_fwd(q, k, v, cu_seq_lens, sm_scale) -> (o, lse2)"}


# ----------------------------------------------------------------------------
def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(tflops=d["bf16_tflops"], tflops_sustained=d.get("bf16_tflops_sustained"),
                    gbs=d["hbm_gbs"], source="measured")
    return dict(tflops=1590.0, tflops_sustained=1400.0, gbs=6650.0, source="fallback")


class ClockSampler:
    """SM clock, power and clock-event reasons of one GPU, read through NVML every few
    milliseconds on a thread while the benchmark runs; `window(t0, t1)` summarises the samples
    taken between two host times.  Reading only: no setting of the GPU is touched."""
    REASONS = (("hw_slowdown", 0x8), ("sw_power_cap", 0x4), ("hw_thermal_slowdown", 0x40),
               ("sw_thermal_slowdown", 0x20), ("hw_power_brake", 0x80))

    def __init__(self, device_index, period_s=0.004):
        self.samples, self.period, self.stop_flag, self.thread, self.h, self.nv = [], period_s, False, None, None, None
        self.max_mhz = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            try:
                uuid = str(torch.cuda.get_device_properties(device_index).uuid)
                self.h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.h = None

    def start(self):
        if self.h is None:
            return
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def _run(self):
        nv = self.nv
        while not self.stop_flag:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    rs = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    rs = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                pw = nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0
                self.samples.append((time.perf_counter(), float(mhz), int(rs), pw))
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self.stop_flag = True
        if self.thread is not None:
            self.thread.join(timeout=1.0)

    def window(self, t0, t1):
        if self.h is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["nvml unavailable"]}
        sel = [s for s in self.samples if t0 <= s[0] <= t1]
        if not sel and self.samples:     # a region shorter than the sampling period: the nearest sample
            mid = 0.5 * (t0 + t1)
            sel = [min(self.samples, key=lambda s: abs(s[0] - mid))]
        mhz = sorted(s[1] for s in sel)
        bits = 0
        for s in sel:
            bits |= s[2]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": self.max_mhz, "samples": len(sel),
                "power_w_max": max((s[3] for s in sel), default=None),
                "reasons": [n for n, b in self.REASONS if bits & b]}


def timed(fn, steps, sync, barrier):
    """Time exactly `steps` calls with CUDA events on the current stream, bracketed by
    synchronize + barrier on both sides: (ms per step, host time window of the region)."""
    sync(); barrier(); sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    sync()
    t1 = time.perf_counter()
    barrier(); sync()
    return e0.elapsed_time(e1) / steps, (t0, t1)


def time_steps(fn, steps, warmup, sync, barrier):
    for _ in range(max(warmup, 3)):
        fn()
    return timed(fn, steps, sync, barrier)[0]


# ----------------------------------------------------------------------------
# the reference's CPU path, config by config, on bounded samples (kind "port": the restated
# naive torch functions of oracle/attention_oracle.py, each pinned bit for bit to the reference)
# ----------------------------------------------------------------------------
def _threads():
    n = os.cpu_count() or 1
    torch.set_num_threads(n)
    return n


def cpu_prefill_sample(seconds_hint=12.0):
    """flash_attn_torch (flash_attn_triton.py:877-915) restated, on whole 4096-token, 32-head
    sequences of config 2, repeated until the time hint is used up (at least one)."""
    from oracle import attention_oracle as orc
    from tritonops_b200 import workloads
    threads = _threads()
    S, D, H = CFG2["S"], CFG2["D"], CFG2["H"]
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(1, S, H, D, generator=g).to(torch.bfloat16) for _ in range(3))
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


def cpu_other_configs(budget_s=4.0):
    """CPU baselines of configs 1, 3, 4 and 5: each the reference's own naive torch function for
    that path (restated), on a stated subset of the workload sized for a few seconds."""
    from oracle import attention_oracle as orc
    from tritonops_b200 import workloads
    threads, out = _threads(), {}

    def loop(fn, hint):
        fn()
        n, t0 = 0, time.perf_counter()
        while True:
            fn()
            n += 1
            dt = time.perf_counter() - t0
            if dt >= hint or n >= 1000:
                return n, dt

    # config 1: the tutorial's non-causal einsum math (tutorial/4.3.multi_head_attention.py:11-19)
    w1 = workloads.cfg1("cpu")
    n, dt = loop(lambda: _tutorial_full_attention(w1.q, w1.k, w1.v), min(budget_s, 1.0))
    out["cfg1"] = dict(value=dt / n * 1e6, unit="us per call", cores=threads, kind="port",
                       sample=f"{n} calls of the tutorial's torch_full_attention math on cfg1 (fp16, B=1 H=2 S=128 D=64)")
    # config 3: flash_attn_decoding_torch (flash_attn_decoding.py:339-368) on packed, head-expanded KV
    B3 = 4
    w3 = workloads.decode_work(B3, 32, 8, 128, 8192, 1024, 8192, 2, "cpu")
    lens = w3.seqlens.tolist()
    kp = torch.cat([w3.k_cache[b, :lens[b]] for b in range(B3)])[None].repeat_interleave(4, dim=2)
    vp = torch.cat([w3.v_cache[b, :lens[b]] for b in range(B3)])[None].repeat_interleave(4, dim=2)
    n, dt = loop(lambda: orc.decoding_refpath(w3.q, kp, vp, w3.cu_seqlens), budget_s)
    out["cfg3"] = dict(value=w3.kv_bytes * n / dt / 1e9, unit="GB/s", cores=threads, kind="port",
                       sample=f"{n} passes over {B3} of cfg3's 64 sequences (lengths {lens}, drawn as cfg3's are), KV "
                              f"bytes before the head expansion, {dt:.1f} s, flash_attn_decoding.py:339-368 restated")
    del w3, kp, vp
    # config 4: the dense masked per-(b, h) loop of flash_attn_sparse_torch
    # (flash_attn_sparse_attn_triton.py:391-442) with the mask from the block lists; one head
    S4 = 16384
    g = torch.Generator().manual_seed(3)
    q, k, v = (torch.randn(1, S4, 1, 128, generator=g).to(torch.bfloat16) for _ in range(3))
    idx, cnt = workloads.block_sparse_lists(1, 1, S4 // 64, 8, 0.1, 3)
    cu = torch.tensor([0, S4], dtype=torch.int32)
    t0 = time.perf_counter()
    orc.block_sparse_prefill_refpath(q, k, v, cu, idx, cnt)
    dt = time.perf_counter() - t0
    fl = workloads.block_sparse_flops(idx, cnt, 64, 128, S4)
    out["cfg4"] = dict(value=fl / dt / 1e12, unit="TFLOP/s", cores=threads, kind="port",
                       sample=f"1 of cfg4's 32 (b, h) heads (S=16384, lists drawn as cfg4's are), listed FLOPs only "
                              f"(the loop computes the dense 16384^2 scores), {dt:.1f} s, "
                              f"flash_attn_sparse_attn_triton.py:391-442 restated with a block-list mask")
    del q, k, v
    # config 5: gather the listed blocks, then the sparse flash_attn_decoding_torch math
    # (flash_attn_decoding_sparse.py:368-406); one sequence of the batch
    w5 = workloads.decode_work(1, 32, 32, 128, 32768, 32768, 32768, 4, "cpu")
    sel = workloads.topk_block_lists(1, 32, 512, 64, 4)
    n, dt = loop(lambda: orc.block_sparse_decoding_refpath(w5.q, w5.k_cache, w5.v_cache, sel), budget_s)
    nbytes = 32 * 64 * 64 * 128 * 2 * 2
    out["cfg5"] = dict(value=nbytes * n / dt / 1e9, unit="GB/s", cores=threads, kind="port",
                       sample=f"{n} passes over 1 of cfg5's 32 sequences (32 heads x 64 blocks of 64 keys gathered), "
                              f"{dt:.1f} s, gather + flash_attn_decoding_sparse.py:368-406 restated")
    return out


def _tutorial_full_attention(q, k, v):
    """softmax(Q K^T / sqrt(D)) V in the input dtype, layout [B, H, N, D]: the math of the
    tutorial's torch_full_attention (tutorial/4.3.multi_head_attention.py:11-19)."""
    qh, kh, vh = (t.permute(0, 2, 1, 3) for t in (q, k, v))
    s = torch.einsum("bhqd,bhkd->bhqk", qh, kh) / math.sqrt(q.shape[-1])
    return torch.einsum("bhqk,bhkd->bhqd", torch.softmax(s, dim=-1), vh)


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
        "higher_is_better": True, "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic N(0,1), seeded", "config": static_config(),
        "cpu_baseline": {k: last[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "each step is a bounded sample of the workload on the host cores (rank 0 only)",
    }
    line["cpu_baseline"]["value"] = val
    print(json.dumps(line))


# ----------------------------------------------------------------------------
# max-abs error of sampled rows against fp32 math on the device (outside any timed region)
# ----------------------------------------------------------------------------
def err_dense_heads(q, k, v, o, lse2, S, scale, samples):
    tril = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()
    eo = el = 0.0
    for b, h in samples:
        sl = slice(b * S, (b + 1) * S)
        s = (q[0, sl, h].float() @ k[0, sl, h].float().T) * scale
        s = s.masked_fill(~tril, -math.inf)
        ref = torch.softmax(s, -1) @ v[0, sl, h].float()
        eo = max(eo, (o[0, sl, h].float() - ref).abs().max().item())
        el = max(el, (lse2[0, sl, h] / LOG2E - torch.logsumexp(s, -1)).abs().max().item())
    return eo, el


def err_decode_rows(w, o, rows):
    e = 0.0
    for b in rows:
        n = int(w.seqlens[b])
        g = w.q.shape[1] // w.k_cache.shape[2]
        kk = w.k_cache[b, :n].float().permute(1, 0, 2).repeat_interleave(g, 0)      # [Hq, n, D]
        vv = w.v_cache[b, :n].float().permute(1, 0, 2).repeat_interleave(g, 0)
        p = torch.softmax(torch.einsum("hd,hkd->hk", w.q[b].float(), kk) * w.scale, -1)
        e = max(e, (o[b].float() - torch.einsum("hk,hkd->hd", p, vv)).abs().max().item())
    return e


def err_block_decode(w, o, samples):
    e = 0.0
    off = torch.arange(64, device=w.q.device)
    for b, h in samples:
        rows = (w.block_idx[b, h].long()[:, None] * 64 + off[None, :]).reshape(-1)
        kk, vv = w.k_cache[b, rows, h].float(), w.v_cache[b, rows, h].float()
        p = torch.softmax((kk @ w.q[b, h].float()) * w.scale, 0)
        e = max(e, (o[b, h].float() - p @ vv).abs().max().item())
    return e


def err_block_prefill(w, o, S, samples):
    """(b, h, query block): the 64 rows of that block against dense masked fp32 math."""
    e = 0.0
    for b, h, qb in samples:
        sl = slice(b * S, (b + 1) * S)
        rows = slice(b * S + qb * 64, b * S + qb * 64 + 64)
        s = (w.q[0, rows, h].float() @ w.k[0, sl, h].float().T) * w.scale          # [64, S]
        vis = torch.zeros(S // 64, dtype=torch.bool, device=w.q.device)
        lst = w.block_idx[b, h, qb, :int(w.block_cnt[b, h, qb])].long()
        vis[lst[lst >= 0]] = True
        mask = vis.repeat_interleave(64)[None, :].expand(64, S).clone()
        qi = torch.arange(qb * 64, qb * 64 + 64, device=w.q.device)
        mask &= torch.arange(S, device=w.q.device)[None, :] <= qi[:, None]
        ref = torch.softmax(s.masked_fill(~mask, -math.inf), -1) @ w.v[0, sl, h].float()
        e = max(e, (o[0, rows, h].float() - ref).abs().max().item())
    return e


def err_backward(w, do, grads, S, samples):
    tril = torch.ones(S, S, dtype=torch.bool, device=w.q.device).tril()
    e = [0.0, 0.0, 0.0]
    for b, h in samples:
        sl = slice(b * S, (b + 1) * S)
        qq, kk, vv = (t[0, sl, h].float().requires_grad_(True) for t in (w.q, w.k, w.v))
        s = ((qq @ kk.T) * w.scale).masked_fill(~tril, -math.inf)
        (torch.softmax(s, -1) @ vv * do[0, sl, h].float()).sum().backward()
        for i, (gr, ref) in enumerate(zip(grads, (qq.grad, kk.grad, vv.grad))):
            e[i] = max(e[i], (gr[0, sl, h].float() - ref).abs().max().item())
    return {"dq": e[0], "dk": e[1], "dv": e[2]}


# ----------------------------------------------------------------------------
def run_ours(args, rank, world, local_rank, cpu_base):
    import torch.distributed as dist
    from tritonops_b200 import ops, sharding, workloads
    from tritonops_b200.flash_attn_triton.flash_attn_triton import flash_attn_triton_fwd
    from tritonops_b200.host import HostPrefill
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

    if args.only != "all":
        return run_single(args, dev, sync, barrier, pk)
    sampler = ClockSampler(local_rank)
    sampler.start()
    windows = []          # host time windows of every timed region (for the overall clocks record)

    def region(fn, steps, warmup=3):
        for _ in range(warmup):
            fn()
        ms, win = timed(fn, steps, sync, barrier)
        windows.append(win)
        return reduce_max(ms), win

    def graph_region(fn, steps, per_graph=10):
        """The same steps replayed from a CUDA graph (10 calls per graph): what a decoding loop that
        captures its launches sees.  A step of tens of microseconds is otherwise timed together with
        the host's launch path.  None if the capture fails."""
        try:
            side = torch.cuda.Stream(dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                fn()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    for _ in range(per_graph):
                        fn()
            torch.cuda.current_stream(dev).wait_stream(side)
            ms, _ = region(g.replay, max(1, steps // per_graph))
            return ms / per_graph
        except Exception:
            return None

    def with_graph(entry, fn, steps, nbytes):
        """Adds the graph-replayed time to a decoding entry and makes the better of the two the
        entry's figure (both stay in the entry)."""
        ms_g = graph_region(fn, steps)
        entry["ms_per_step_eager"] = entry["ms_per_step"]
        entry["ms_per_step_graph"] = ms_g
        entry["timed_as"] = "eager launches"
        if ms_g is not None and ms_g < entry["ms_per_step"]:
            gb = nbytes / ms_g / 1e6
            entry.update({"value": gb, "ms_per_step": ms_g, "achieved": gb / world, "frac": gb / world / pk["gbs"],
                          "frac_of_nominal_8TBs": gb / world / 8000.0,
                          "timed_as": "replayed from a CUDA graph of 10 steps"})
        return entry

    # ---------------- headline: config 2, split by (sequence x KV head) units over the ranks
    c = CFG2
    S = c["S"]
    w = workloads.dense_causal(c["B"], c["H"], S, c["D"], 1, dev, name="cfg2")     # same bits on every rank
    sm_scale = w.scale * LOG2E
    cu_host = [int(x) for x in w.cu_seqlens.cpu()]
    pieces = sharding.prefill_unit_pieces(c["B"], c["H"], world, rank)
    calls = []
    for piece in pieces:
        qs, ks, vs, cu_p = sharding.slice_prefill_piece(w.q, w.k, w.v, cu_host, piece)     # strided views, no copy
        calls.append((qs, ks, vs, torch.tensor(cu_p, dtype=torch.int32, device=dev)))

    def step():
        return [flash_attn_triton_fwd(qs, ks, vs, cu_p, sm_scale, max_seqlen=S) for qs, ks, vs, cu_p in calls]

    l0 = ops.launch_counter
    step()
    launches = (ops.launch_counter - l0) * args.steps     # kernels of ours per timed region on this rank
    for _ in range(args.warmup):
        step()
    regions = []
    for _ in range(5):
        ms_r, win = region(step, args.steps, warmup=0)
        regions.append({"ms_per_step": ms_r, "tflops": w.flops / ms_r / 1e9, "clocks": sampler.window(*win), "window": win})
    order = sorted(range(len(regions)), key=lambda i: regions[i]["ms_per_step"])
    med = regions[order[len(order) // 2]]
    ms = med["ms_per_step"]
    value = w.flops / ms / 1e9                            # whole job (one config-2 batch), TFLOP/s
    per_gpu = value / world
    # one long region: what the board sustains at its power cap
    n_long = int(min(40000, max(args.steps, 2200.0 / ms))) if args.steps >= 5 else args.steps
    ms_long, win_long = region(step, n_long, warmup=0)
    sustained = {"launches": n_long * len(calls), "seconds": ms_long * n_long / 1e3, "ms_per_step": ms_long,
                 "tflops_per_gpu": w.flops / ms_long / 1e9 / world,
                 "frac_of_sustained_peak": (w.flops / ms_long / 1e9 / world) / pk["tflops_sustained"] if pk["tflops_sustained"] else None,
                 "clocks": sampler.window(*win_long)}

    # ---------------- parity of the headline, and of the sharded run against one GPU
    parity, shard_check = {}, None
    outs = step()
    if rank == 0:
        o_full, lse_full = flash_attn_triton_fwd(w.q, w.k, w.v, w.cu_seqlens, sm_scale, max_seqlen=S)
        eo, el = err_dense_heads(w.q, w.k, w.v, o_full, lse_full, S, w.scale, [(0, 0), (1, 13), (3, 31)])
        parity["cfg2"] = {"max_abs_err_o": eo, "max_abs_err_lse": el, "tolerance_o": 2e-2,
                          "checked": "3 of 128 heads, every row, against fp32 softmax(QK^T scale)V on the device"}
    if world > 1:
        # unit-major copies of each rank's O / LSE, gathered; rank 0 compares with its own full run
        g = c["H"] // w.k.shape[2]
        mine_o = torch.cat([o.view(-1, S, o.shape[2] // g, g * c["D"]).permute(0, 2, 1, 3).reshape(-1, S, g * c["D"])
                            for o, _ in outs])
        mine_l = torch.cat([l.view(-1, S, l.shape[2] // g, g).permute(0, 2, 1, 3).reshape(-1, S, g) for _, l in outs])
        if (c["B"] * w.k.shape[2]) % world == 0:
            all_o = torch.empty(world * mine_o.shape[0], S, g * c["D"], device=dev, dtype=mine_o.dtype)
            all_l = torch.empty(world * mine_l.shape[0], S, g, device=dev, dtype=mine_l.dtype)
            dist.all_gather_into_tensor(all_o, mine_o.contiguous())
            dist.all_gather_into_tensor(all_l, mine_l.contiguous())
            if rank == 0:
                ref_o = o_full.view(c["B"], S, w.k.shape[2], g * c["D"]).permute(0, 2, 1, 3).reshape(-1, S, g * c["D"])
                ref_l = lse_full.view(c["B"], S, w.k.shape[2], g).permute(0, 2, 1, 3).reshape(-1, S, g)
                same = bool(torch.equal(all_o, ref_o)) and bool(torch.equal(all_l, ref_l))
                shard_check = {"cfg2": "bit-identical to the one-GPU result" if same else "MISMATCH",
                               "how": "O and LSE of all ranks gathered (NCCL all_gather, outside the timed region) "
                                      "and compared with rank 0's unsharded run"}
            del all_o, all_l
        del mine_o, mine_l
    del outs

    # ---------------- weak scaling beside it (N > 1): every rank its own full config 2
    weak = None
    if world > 1:
        full = lambda: flash_attn_triton_fwd(w.q, w.k, w.v, w.cu_seqlens, sm_scale, max_seqlen=S)
        ms_w, _ = region(full, args.steps)
        weak = {"value": w.flops * world / ms_w / 1e9, "unit": "TFLOP/s", "ms_per_step": ms_w,
                "what": "every rank runs its own full config 2 (global batch 4 x N)"}

    # ---------------- end to end: pinned host buffers in, O + LSE back out, every step
    host = []
    for qs, ks, vs, cu_p in calls:
        hq, hk, hv = (t.contiguous().cpu().pin_memory() for t in (qs, ks, vs))
        ho = torch.empty(hq.shape, dtype=hq.dtype).pin_memory()
        hl = torch.empty(hq.shape[:3], dtype=torch.float32).pin_memory()
        host.append((hq, hk, hv, ho, hl, [int(x) for x in cu_p.cpu()]))
    pipe = HostPrefill(dev)

    def e2e_step():
        for hq, hk, hv, ho, hl, cu_p in host:
            pipe.run(hq, hk, hv, cu_p, ho, hl, scale=sm_scale, scale_has_log2e=True, causal=True, lse_base2=True)

    e2e_steps = max(3, min(args.steps, 10))
    ms_e2e, _ = region(e2e_step, e2e_steps)
    h2d_rank = sum(sum(t.numel() * t.element_size() for t in (hq, hk, hv)) for hq, hk, hv, _, _, _ in host)
    d2h_rank = sum(ho.numel() * ho.element_size() + hl.numel() * 4 for _, _, _, ho, hl, _ in host)
    # the same copies on the same three streams with the same dependencies and no kernel between
    # them: what the box's PCIe / host memory alone allows
    def copy_floor_step():
        for hq, hk, hv, ho, hl, cu_p in host:
            pipe.run(hq, hk, hv, cu_p, ho, hl, scale=sm_scale, scale_has_log2e=True, causal=True, lse_base2=True,
                     copies_only=True)

    try:
        ms_floor, _ = region(copy_floor_step, e2e_steps)
    except Exception:
        ms_floor = None
    h2d = h2d_rank * world if world > 1 else h2d_rank
    d2h = d2h_rank * world if world > 1 else d2h_rank
    del host, pipe

    rl = {}      # per-kernel roofline entries beside the headline's
    other = {}

    def guard(name, fn):
        try:
            fn()
        except Exception as e:  # keep the headline even if a secondary config fails
            rl[name] = {"error": repr(e)[:300]}

    # ---------------- config 3: GQA decoding (HBM bound); N > 1: sequences dealt out by length
    def do_cfg3():
        w3 = workloads.cfg3(dev)
        lens = w3.seqlens.cpu().tolist()
        mine = sharding.balanced_shards(lens, world)[rank] if world > 1 else list(range(len(lens)))
        idx = torch.tensor(mine, device=dev)
        q3, k3, v3, sl3 = (w3.q[idx], w3.k_cache[idx], w3.v_cache[idx], w3.seqlens[idx]) if world > 1 else \
            (w3.q, w3.k_cache, w3.v_cache, w3.seqlens)
        f3 = lambda: ops.decode(q3, k3, v3, seqlens=sl3, max_seqlen=w3.max_seqlen)
        ms3, _ = region(f3, max(args.steps, 10))
        gbs = w3.kv_bytes / ms3 / 1e6                     # whole job
        entry = {"value": gbs, "unit": "GB/s", "ms_per_step": ms3, "bound": "hbm", "achieved": gbs / world,
                 "peak": pk["gbs"], "frac": gbs / world / pk["gbs"], "frac_of_nominal_8TBs": gbs / world / 8000.0,
                 "algorithmic_bytes": w3.kv_bytes, **traffic("cfg3"),
                 "workload": "cfg3: GQA decode bf16 B=64 Hq=32 Hkv=8 D=128, cache 8192, len U[1024,8192] seed 2, "
                             "split chunks chosen by the library; 2.6 GB of KV per step, far larger than L2"}
        with_graph(entry, f3, max(args.steps, 10), w3.kv_bytes)
        if world == 1:
            ms512, _ = region(lambda: ops.decode(q3, k3, v3, seqlens=sl3, max_seqlen=w3.max_seqlen, chunk=512),
                              max(args.steps, 10))
            entry["with_512_key_chunks_GBs"] = w3.kv_bytes / ms512 / 1e6
            entry["max_abs_err"] = err_decode_rows(w3, f3(), [0, 17, 41, 63])
            entry["checked"] = "4 of 64 sequences, all heads, against fp32 math on the device"
            parity["cfg3"] = entry["max_abs_err"]
        else:
            o_full = ops.decode(w3.q, w3.k_cache, w3.v_cache, seqlens=w3.seqlens, max_seqlen=w3.max_seqlen)
            entry["sharding"] = f"{len(mine)} sequences on this rank (greedy longest-first by length)"
            entry["shard_max_abs_diff_vs_one_gpu"] = reduce_max((f3().float() - o_full[idx].float()).abs().max().item())
        rl["decode_cfg3"] = entry

    guard("decode_cfg3", do_cfg3)

    # ---------------- config 4: block-sparse causal prefill (tensor bound, gathered KV blocks)
    def do_cfg4():
        w4 = workloads.cfg4(dev)
        S4, B4, H4 = 16384, 2, 16
        cu4 = [int(x) for x in w4.cu_seqlens.cpu()]
        calls4 = []
        for piece in sharding.prefill_unit_pieces(B4, H4, world, rank):
            qs, ks, vs, cu_p = sharding.slice_prefill_piece(w4.q, w4.k, w4.v, cu4, piece)
            b0, b1, h0, h1 = piece
            calls4.append((qs, ks, vs, torch.tensor(cu_p, dtype=torch.int32, device=dev),
                           w4.block_idx[b0:b1, h0:h1].contiguous(), w4.block_cnt[b0:b1, h0:h1].contiguous()))
        f4 = lambda: [ops.prefill(qs, ks, vs, cu_seqlens=cu_p, max_seqlen=S4, sparsity=ops.BLOCK_LIST, block_idx=bi,
                                  block_cnt=bc) for qs, ks, vs, cu_p, bi, bc in calls4]
        ms4, _ = region(f4, max(args.steps, 10))
        tf4 = w4.flops / ms4 / 1e9
        entry = {"value": tf4, "unit": "TFLOP/s", "ms_per_step": ms4, "bound": "tensor", "achieved": tf4 / world,
                 "peak": pk["tflops"], "frac": tf4 / world / pk["tflops"], "frac_of_nominal_2250": tf4 / world / 2250.0,
                 "algorithmic_flops": w4.flops, **traffic("cfg4"),
                 "workload": "cfg4: block-sparse causal prefill bf16 B=2 H=16 S=16384 D=128, 64x64 blocks, 8-block "
                             "window + Bernoulli(0.1) earlier blocks seed 3; FLOPs = 4*D per visible (query, key) pair "
                             "of the listed blocks only"}
        if world == 1:
            o4 = f4()[0][0]
            entry["max_abs_err"] = err_block_prefill(w4, o4, S4, [(0, 0, 0), (0, 7, 100), (1, 15, 255), (1, 3, 37)])
            entry["checked"] = "4 query blocks (64 rows each) against dense masked fp32 math on the device"
            parity["cfg4"] = entry["max_abs_err"]
        rl["prefill_cfg4"] = entry

    guard("prefill_cfg4", do_cfg4)

    # ---------------- config 5: top-k block decoding (HBM bound, gathered blocks); N > 1: by batch
    def do_cfg5():
        w5 = workloads.cfg5(dev)
        b0, b1 = sharding.contiguous_shard(w5.q.shape[0], world, rank)
        q5, k5, v5, sl5, bi5 = w5.q[b0:b1], w5.k_cache[b0:b1], w5.v_cache[b0:b1], w5.seqlens[b0:b1], w5.block_idx[b0:b1]
        f5 = lambda: ops.decode(q5, k5, v5, seqlens=sl5, sparsity=ops.BLOCK_LIST, block_idx=bi5, block_size=64)
        ms5, _ = region(f5, max(args.steps, 10))
        gbs5 = w5.kv_bytes / ms5 / 1e6
        entry = {"value": gbs5, "unit": "GB/s", "ms_per_step": ms5, "bound": "hbm", "achieved": gbs5 / world,
                 "peak": pk["gbs"], "frac": gbs5 / world / pk["gbs"], "frac_of_nominal_8TBs": gbs5 / world / 8000.0,
                 "algorithmic_bytes": w5.kv_bytes, **traffic("cfg5"),
                 "workload": "cfg5: block-sparse decode bf16 B=32 H=32 D=128, KV 32768 = 512 blocks of 64, 64 blocks per "
                             "(b,h) seed 4"}
        with_graph(entry, f5, max(args.steps, 10), w5.kv_bytes)
        if world == 1:
            entry["max_abs_err"] = err_block_decode(w5, f5(), [(0, 0), (5, 17), (13, 2), (31, 31), (20, 9), (8, 30)])
            entry["checked"] = "6 of 1024 (b, h) against fp32 math over the 64 gathered blocks on the device"
            parity["cfg5"] = entry["max_abs_err"]
        rl["decode_cfg5"] = entry

    guard("decode_cfg5", do_cfg5)

    if world == 1:
        # ---------------- config 2 backward (dQ, dK, dV; 2.5x the forward FLOPs)
        def do_bwd():
            o2, lse2 = flash_attn_triton_fwd(w.q, w.k, w.v, w.cu_seqlens, sm_scale, max_seqlen=S)
            do2 = torch.randn(w.q.shape, device=dev, dtype=torch.float32).to(w.q.dtype)
            fb = lambda: ops.prefill_bwd(w.q, w.k, w.v, o2, do2, lse2, cu_seqlens=w.cu_seqlens, max_seqlen=S,
                                         scale=sm_scale, scale_has_log2e=True, lse_base2=True)
            msb, _ = region(fb, max(args.steps // 2, 5))
            tfb = 2.5 * w.flops / msb / 1e9
            errs = err_backward(w, do2, fb(), S, [(0, 0), (3, 31)])
            rl["backward_cfg2"] = {
                "value": tfb, "unit": "TFLOP/s", "ms_per_step": msb, "bound": "tensor", "achieved": tfb,
                "peak": pk["tflops"], "frac": tfb / pk["tflops"], "algorithmic_flops": 2.5 * w.flops,
                **traffic("cfg2_backward"), "max_abs_err": errs,
                "checked": "2 of 128 heads, every row, against fp32 autograd on the device",
                "workload": "backward of cfg2 (dQ, dK, dV); FLOPs = 2.5 x the causal forward count (five products "
                            "instead of two)"}
            parity["cfg2_backward"] = errs

        guard("backward_cfg2", do_bwd)

        # ---------------- rows either side of the hot path: paged decoding and RMSNorm (HBM bound)
        def do_paged():
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
            msp, _ = region(fpg, max(args.steps, 10))
            gbp = w3.kv_bytes / msp / 1e6
            rl["paged_decode_cfg3"] = {
                "value": gbp, "unit": "GB/s", "ms_per_step": msp, "bound": "hbm", "achieved": gbp, "peak": pk["gbs"],
                "frac": gbp / pk["gbs"], "algorithmic_bytes": w3.kv_bytes, **traffic("paged_cfg3"),
                "bit_identical_to_padded_decode": same,
                "workload": "config 3's sequences in 64-key pages scattered at random over a pool, found through a "
                            "page table"}
            with_graph(rl["paged_decode_cfg3"], fpg, max(args.steps, 10), w3.kv_bytes)

        guard("paged_decode_cfg3", do_paged)

        def do_rms():
            rows_n, dim_n = 65536, 4096
            xn = torch.randn(rows_n, dim_n, device=dev, dtype=torch.bfloat16)
            wn = (1 + 0.1 * torch.randn(dim_n, device=dev)).to(torch.bfloat16)
            dyn = torch.randn_like(xn)
            y, rstd_n = ops.rmsnorm_fwd(xn, wn, 1e-6)
            nbytes = xn.numel() * 2
            msf, _ = region(lambda: ops.rmsnorm_fwd(xn, wn, 1e-6), max(args.steps, 10))
            msb, _ = region(lambda: ops.rmsnorm_bwd(dyn, xn, wn, rstd_n), max(args.steps, 10))
            xs = xn[:1024].float()
            ref = xs * torch.rsqrt(xs.pow(2).mean(-1, keepdim=True) + 1e-6) * wn.float()
            rl["rmsnorm_fwd"] = {
                "value": 2 * nbytes / msf / 1e6, "unit": "GB/s", "ms_per_step": msf, "bound": "hbm",
                "achieved": 2 * nbytes / msf / 1e6, "peak": pk["gbs"], "frac": 2 * nbytes / msf / 1e6 / pk["gbs"],
                "algorithmic_bytes": 2 * nbytes, **traffic("rmsnorm_fwd"),
                "max_abs_err": (y[:1024].float() - ref).abs().max().item(),
                "workload": "RMSNorm forward (x in, y out) over 65536 rows of 4096 bf16"}
            rl["rmsnorm_bwd"] = {
                "value": 3 * nbytes / msb / 1e6, "unit": "GB/s", "ms_per_step": msb, "bound": "hbm",
                "achieved": 3 * nbytes / msb / 1e6, "peak": pk["gbs"], "frac": 3 * nbytes / msb / 1e6 / pk["gbs"],
                "algorithmic_bytes": 3 * nbytes, **traffic("rmsnorm_bwd"),
                "workload": "RMSNorm backward (dy, x in, dx out; dw reduced) over 65536 rows of 4096 bf16"}

        guard("rmsnorm_fwd", do_rms)

        # ---------------- config 1: the reference's own small case (latency bound), in microseconds
        def do_cfg1():
            w1 = workloads.cfg1(dev)
            f1 = lambda: ops.prefill(w1.q, w1.k, w1.v, cu_seqlens=w1.cu_seqlens, max_seqlen=w1.max_seqlen,
                                     causal=False, scale=w1.scale)
            us_call = time_steps(f1, 200, 20, sync, barrier) * 1e3     # call rate incl. the Python host path
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
                graph_us = time_steps(g1.replay, 50, 5, sync, barrier) * 1e3 / 20
                del g1
            except Exception:
                graph_us = None
            o1, _ = f1()
            ref = _tutorial_full_attention(w1.q.float(), w1.k.float(), w1.v.float()).permute(0, 2, 1, 3)
            other["cfg1_small_noncausal"] = {
                "value": graph_us if graph_us is not None else us_call, "unit": "us per call",
                "per_call_with_python_host_path_us": us_call, "per_launch_replayed_from_a_cuda_graph_us": graph_us,
                "max_abs_err": (o1.float() - ref).abs().max().item(),
                "config": {"workload": "cfg1: non-causal fp16 B=1 H=2 S=128 D=64 (8.4 MFLOP, 128 KiB): launch-latency "
                                       "bound, one CTA"}}
            parity["cfg1"] = other["cfg1_small_noncausal"]["max_abs_err"]

        guard("cfg1", do_cfg1)

    sampler.stop()
    # `clocks` describes the headline's timed regions; the long region and the rest have their own record
    head = [s for s in sampler.samples if any(r["window"][0] <= s[0] <= r["window"][1] for r in regions)]
    clocks = dict(med["clocks"])
    if head:
        mhz = sorted(s[1] for s in head)
        bits = 0
        for s in head:
            bits |= s[2]
        clocks.update(sm_mhz=mhz[len(mhz) // 2], samples=len(head), power_w_max=max(s[3] for s in head),
                      reasons=[n for n, b in ClockSampler.REASONS if bits & b])
    clocks["what"] = "NVML samples inside the five headline regions; the sustained region has its own record"
    busy = [s for s in sampler.samples if any(a <= s[0] <= b for a, b in windows)]
    if busy:
        mhz = sorted(s[1] for s in busy)
        bits = 0
        for s in busy:
            bits |= s[2]
        clocks["all_timed_regions"] = {"sm_mhz": mhz[len(mhz) // 2], "sm_mhz_min": mhz[0], "samples": len(busy),
                                       "power_w_max": max(s[3] for s in busy),
                                       "reasons": [n for n, b in ClockSampler.REASONS if bits & b]}
    for r in regions:
        r.pop("window", None)
    torch.cuda.empty_cache()

    # ---------------- the reference's Triton kernels on this GPU (one GPU only; own process)
    if world == 1 and rank == 0 and not os.environ.get("B200ATTN_BENCH_SKIP_TRITON"):
        ref_gpu = reference_triton_on_gpu()
        if "cfg2_kernel_ms" in ref_gpu:
            ref_gpu["cfg2_speedup_kernel"] = ref_gpu["cfg2_kernel_ms"] / ms
            ref_gpu["cfg2_speedup_wrapper"] = ref_gpu["cfg2_wrapper_ms"] / ms
        if "cfg2_backward_wrapper_ms" in ref_gpu and "ms_per_step" in rl.get("backward_cfg2", {}):
            ref_gpu["cfg2_backward_speedup"] = ref_gpu["cfg2_backward_wrapper_ms"] / rl["backward_cfg2"]["ms_per_step"]
        if "cfg3_wrapper_ms" in ref_gpu and "ms_per_step" in rl.get("decode_cfg3", {}):
            # (eager against eager: the reference wrapper is timed through its own Python launch path)
            ref_gpu["cfg3_speedup_wrapper"] = ref_gpu["cfg3_wrapper_ms"] / rl["decode_cfg3"].get(
                "ms_per_step_eager", rl["decode_cfg3"]["ms_per_step"])
        rl["reference_triton_gpu"] = ref_gpu

    if rank != 0:
        return
    tr, tr_src = TRAFFIC["cfg2"]
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic N(0,1), seeded",
        "config": static_config(),
        "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": pk["tflops"],
                     "unit": "TFLOP/s", "frac": per_gpu / pk["tflops"],
                     "peak_source": pk["source"] + " cuBLAS bf16 burst (per GPU)",
                     "frac_of_sustained_peak": per_gpu / pk["tflops_sustained"] if pk["tflops_sustained"] else None,
                     "frac_of_nominal_2250": per_gpu / 2250.0,
                     "traffic": tr / world if tr else None, "traffic_source": tr_src,
                     "traffic_unit": "bytes per launch (ncu)",
                     "algorithmic_bytes": (4 * w.q.numel() * 2 + w.q.numel() // 128 * 4) / world,
                     "regions": {"what": f"5 regions of {args.steps} steps; the median one is the headline",
                                 "ms_per_step": [r["ms_per_step"] for r in regions],
                                 "tflops": [r["tflops"] for r in regions],
                                 "sm_mhz": [r["clocks"]["sm_mhz"] for r in regions],
                                 "min": min(r["tflops"] for r in regions), "max": max(r["tflops"] for r in regions)},
                     "sustained": sustained,
                     "max_abs_err": parity.get("cfg2"),
                     "shard_check": shard_check,
                     "weak_scaling": weak,
                     **rl},
        "cpu_baseline": cpu_base if cpu_base else {"value": None, "unit": "TFLOP/s", "cores": 0, "kind": "port",
                                                   "sample": "timed at N=1 only"},
        "e2e": {"value": w.flops / ms_e2e / 1e9, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "copy_floor_ms": ms_floor,
                "copy_floor_what": "the same host<->device copies on the same streams with the kernels left out",
                "api": "tritonops_b200.host.HostPrefill.run(pinned q, k, v -> pinned o, lse2): every sequence streamed "
                       "in 2048-row chunks through copy-in / kernel (b200attn_prefill_fwd_rows) / copy-out on three "
                       "streams; at N>1 every rank moves its own shard"},
        "gpu_launches": launches,
        "clocks": clocks,
        "parity": parity,
        "other": other,
    }
    print(json.dumps(line))


def reference_triton_on_gpu():
    """Time the reference's own Triton kernels (staged under oracle/_ref) on this GPU in a child
    process: a failure of that code cannot take the benchmark down with it."""
    try:
        out = subprocess.run([sys.executable, "-m", "oracle.ref_triton", "--bench"], cwd=ROOT, capture_output=True,
                             text=True, timeout=600)
        for ln in reversed(out.stdout.strip().splitlines()):
            if ln.startswith("{"):
                return json.loads(ln)
        return {"unavailable": (out.stderr or out.stdout)[-300:]}
    except Exception as e:
        return {"unavailable": repr(e)[:300]}


def run_single(args, dev, sync, barrier, pk):
    """One kernel's loop only (used for ncu captures; prints a short JSON line)."""
    from tritonops_b200 import ops, workloads
    if args.only == "prefill":
        w = workloads.dense_causal(4, 32, 4096, 128, 1, dev, name="cfg2")
        fn = lambda: ops.prefill(w.q, w.k, w.v, cu_seqlens=w.cu_seqlens, max_seqlen=w.max_seqlen)
        work, unit, peak = w.flops / 1e9, "TFLOP/s", pk["tflops"]
    elif args.only in ("decode", "paged_decode"):
        w = workloads.cfg3(dev)
        fn = lambda: ops.decode(w.q, w.k_cache, w.v_cache, cu_seqlens=w.cu_seqlens, max_seqlen=w.max_seqlen)
        if args.only == "paged_decode":
            page, B3, cap = 64, w.k_cache.shape[0], w.k_cache.shape[1]
            n_pages = B3 * cap // page
            table = torch.randperm(n_pages, generator=torch.Generator().manual_seed(7)).to(torch.int32).view(B3, -1).to(dev)
            kp = torch.empty(n_pages, page, *w.k_cache.shape[2:], device=dev, dtype=w.k_cache.dtype)
            vp = torch.empty_like(kp)
            kp[table.view(-1).long()] = w.k_cache.view(n_pages, page, *w.k_cache.shape[2:])
            vp[table.view(-1).long()] = w.v_cache.view(n_pages, page, *w.v_cache.shape[2:])
            fn = lambda: ops.paged_decode(w.q, kp, vp, table, w.seqlens, max_seqlen=w.max_seqlen)
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
    elif args.only in ("rmsnorm_fwd", "rmsnorm_bwd"):
        x = torch.randn(65536, 4096, device=dev, dtype=torch.bfloat16)
        wn = torch.ones(4096, device=dev, dtype=torch.bfloat16)
        dy = torch.randn_like(x)
        _, rstd = ops.rmsnorm_fwd(x, wn, 1e-6)
        fn = (lambda: ops.rmsnorm_fwd(x, wn, 1e-6)) if args.only == "rmsnorm_fwd" else (lambda: ops.rmsnorm_bwd(dy, x, wn, rstd))
        work, unit, peak = (2 if args.only == "rmsnorm_fwd" else 3) * x.numel() * 2 / 1e6, "GB/s", pk["gbs"]
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
                    choices=["all", "prefill", "decode", "paged_decode", "backward", "sparse_prefill", "sparse_decode",
                             "sparse_decode_small", "rmsnorm_fwd", "rmsnorm_bwd"],
                    help="profiling aid: run one kernel's timed loop and print a short line")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    # The CPU baselines run first, on one GPU only and before any GPU work or process group
    # exists: no rank waits in a collective (spinning its GPU) while rank 0 computes on the host.
    cpu_base = None
    if world == 1 and args.only == "all":
        budget = float(os.environ.get("B200ATTN_BENCH_CPU_SECONDS", "12"))
        cpu = cpu_prefill_sample(budget)
        cpu_base = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
        try:
            cpu_base["other_configs"] = cpu_other_configs(min(4.0, budget))
        except Exception as e:
            cpu_base["other_configs"] = {"error": repr(e)[:300]}
        try:
            cpu_base["other_configs"]["cfg1_triton_interpreter"] = cfg1_interpreter_sample()
        except Exception as e:
            cpu_base["other_configs"]["cfg1_triton_interpreter"] = {"unavailable": repr(e)[:300]}
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_ours(args, rank, world, local_rank, cpu_base)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
            dist.destroy_process_group()


def cfg1_interpreter_sample():
    """Config 1 through the reference's dense Triton kernel under TRITON_INTERPRET=1 (fp16; the
    kernel is causal), in a child process because the switch must be set before triton loads."""
    env = dict(os.environ, TRITON_INTERPRET="1", CUDA_VISIBLE_DEVICES="")
    out = subprocess.run([sys.executable, "-m", "oracle.ref_triton", "--interpret-cfg1"], cwd=ROOT, env=env,
                         capture_output=True, text=True, timeout=300)
    for ln in reversed(out.stdout.strip().splitlines()):
        if ln.startswith("{"):
            return json.loads(ln)
    return {"unavailable": (out.stderr or out.stdout)[-300:]}


if __name__ == "__main__":
    main()
