"""Prefill for callers whose Q, K and V live in pinned HOST memory.

The reference's entry points take device tensors; a caller that starts from host
buffers pays the PCIe copies around them.  `HostPrefill` hides most of that cost:
it walks the packed sequences one by one on three CUDA streams (copy in, attend,
copy out) with double-buffered device staging, so the transfers of neighbouring
sequences overlap the kernels and, PCIe being full duplex, each other.  The
arithmetic is `ops.prefill` on each sequence, i.e. exactly what
`flash_attn_triton_fwd` (flash_attn_triton/flash_attn_triton.py:595-658) computes for
that sequence inside a packed batch."""
from typing import List, Sequence

import torch

from . import ops


class _Slot:
    def __init__(self):
        self.q = self.k = self.v = None
        self.inputs_free = None    # the kernel that read q, k, v has finished
        self.cap = 0


class HostPrefill:
    def __init__(self, device, n_slots: int = 2):
        self.dev = torch.device(device)
        if self.dev.type != "cuda":
            raise RuntimeError("b200attn host pipeline needs a CUDA device (there is no CPU path)")
        self.s_in = torch.cuda.Stream(self.dev)
        self.s_run = torch.cuda.Stream(self.dev)
        self.s_out = torch.cuda.Stream(self.dev)
        self.slots: List[_Slot] = [_Slot() for _ in range(n_slots)]

    def _stage(self, slot: _Slot, n: int, hq, hk, hv):
        """Make the slot's staging tensors hold n tokens.  Called once per slot at the start of
        run(), sized for the longest sequence of that call, so nothing is reallocated while the
        pipeline is running.  Old tensors may still be read by a kernel of an earlier run() on
        s_run: s_in waits for that kernel before they are dropped (their memory goes back to
        s_in's pool and could otherwise be handed out and overwritten at once)."""
        if slot.cap < n or slot.q is None or slot.q.shape[2:] != hq.shape[2:] or slot.k.shape[2:] != hk.shape[2:] \
                or slot.q.dtype != hq.dtype:
            with torch.cuda.stream(self.s_in):
                if slot.inputs_free is not None:
                    self.s_in.wait_event(slot.inputs_free)
                slot.q = torch.empty(1, n, *hq.shape[2:], device=self.dev, dtype=hq.dtype)
                slot.k = torch.empty(1, n, *hk.shape[2:], device=self.dev, dtype=hk.dtype)
                slot.v = torch.empty(1, n, *hv.shape[2:], device=self.dev, dtype=hv.dtype)
            slot.cap = n

    def run(self, hq, hk, hv, cu_seqlens: Sequence[int], ho, hl, *, scale: float, scale_has_log2e: bool = False,
            causal: bool = True, lse_base2: bool = False) -> None:
        """hq [1, T, Hq, D], hk / hv [1, T, Hkv, D], ho like hq, hl fp32 [1, T, Hq]: pinned host
        tensors; cu_seqlens: host integers [B + 1].  Returns when the work is queued; the
        current stream is made to wait for all of it (synchronise it before reading ho / hl)."""
        for t in (hq, hk, hv, ho, hl):
            if t.is_cuda or not t.is_pinned():
                raise ValueError("b200attn host pipeline takes pinned host tensors")
        cur = torch.cuda.current_stream(self.dev)
        start = torch.cuda.Event()
        start.record(cur)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_event(start)
        cu = [int(x) for x in cu_seqlens]
        longest = max([cu[b + 1] - cu[b] for b in range(len(cu) - 1)] + [0])
        if longest > 0:
            for slot in self.slots:
                self._stage(slot, max(longest, slot.cap), hq, hk, hv)
        for b in range(len(cu) - 1):
            s0, s1 = cu[b], cu[b + 1]
            n = s1 - s0
            if n <= 0:
                continue
            slot = self.slots[b % len(self.slots)]
            with torch.cuda.stream(self.s_in):
                if slot.inputs_free is not None:
                    self.s_in.wait_event(slot.inputs_free)
                slot.q[:, :n].copy_(hq[:, s0:s1], non_blocking=True)
                slot.k[:, :n].copy_(hk[:, s0:s1], non_blocking=True)
                slot.v[:, :n].copy_(hv[:, s0:s1], non_blocking=True)
                landed = torch.cuda.Event()
                landed.record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(landed)
                o, lse = ops.prefill(slot.q[:, :n], slot.k[:, :n], slot.v[:, :n], scale=scale,
                                     scale_has_log2e=scale_has_log2e, causal=causal, lse_base2=lse_base2)
                done = torch.cuda.Event()
                done.record(self.s_run)
                slot.inputs_free = done
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done)
                o.record_stream(self.s_out)
                lse.record_stream(self.s_out)
                ho[:, s0:s1].copy_(o, non_blocking=True)
                hl[:, s0:s1].copy_(lse, non_blocking=True)
        end = torch.cuda.Event()
        end.record(self.s_out)
        cur.wait_event(end)
        # the staging buffers are written on s_in and read on s_run: both are ordered before `end`
        # through the events above, so the caller's stream also covers them
