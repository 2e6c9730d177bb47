"""Prefill for callers whose Q, K and V live in pinned HOST memory.

The reference's entry points take device tensors; a caller that starts from host
buffers pays the PCIe copies around them.  `HostPrefill` hides most of that cost:
it walks the packed sequences on three CUDA streams (copy in, attend, copy out)
with double-buffered device staging, so the transfers overlap the kernels and,
PCIe being full duplex, each other.  A causal sequence is streamed in chunks of
rows: rows [t0, t1) of Q, K and V are copied in, `ops.prefill_rows` attends
queries [t0, t1) to keys [0, t1) (a causal query needs no later key), and rows
[t0, t1) of O and LSE are copied out, so what is left after the last byte has
arrived is one chunk's kernel and copy-out instead of a whole sequence's.  The
arithmetic is that of `ops.prefill` on each sequence, bit for bit, i.e. exactly what
`flash_attn_triton_fwd` (flash_attn_triton/flash_attn_triton.py:595-658) computes for
that sequence inside a packed batch."""
from typing import List, Sequence

import torch

from . import ops

_ROW_ALIGN = 256      # b200attn_prefill_fwd_rows takes row ranges that start on a multiple of 256


def chunk_ranges(n: int, chunk_tokens: int, causal: bool):
    """Row ranges [t0, t1) in which a sequence of n tokens is streamed: every range starts on a
    multiple of 256 and ends on one or at n, as b200attn_prefill_fwd_rows asks; a non-causal
    sequence, whose queries need every key, is one range."""
    step = chunk_tokens if causal else max(n, 1)
    return [(t0, min(t0 + step, n)) for t0 in range(0, n, step)]


class _Slot:
    def __init__(self):
        self.q = self.k = self.v = self.o = self.lse = None
        self.inputs_free = None    # the last kernel that read q, k, v has finished
        self.outputs_free = None   # the last copy out of o, lse has finished
        self.cap = 0


class HostPrefill:
    def __init__(self, device, n_slots: int = 2, chunk_tokens: int = 2048):
        self.dev = torch.device(device)
        if self.dev.type != "cuda":
            raise RuntimeError("b200attn host pipeline needs a CUDA device (there is no CPU path)")
        if chunk_tokens <= 0 or chunk_tokens % _ROW_ALIGN:
            raise ValueError(f"chunk_tokens must be a positive multiple of {_ROW_ALIGN}")
        self.chunk = chunk_tokens
        self.s_in = torch.cuda.Stream(self.dev)
        self.s_run = torch.cuda.Stream(self.dev)
        self.s_out = torch.cuda.Stream(self.dev)
        self.slots: List[_Slot] = [_Slot() for _ in range(n_slots)]

    def _stage(self, slot: _Slot, n: int, hq, hk, hv):
        """Make the slot's staging tensors hold n tokens.  Called once per slot at the start of
        run(), sized for the longest sequence of that call, so nothing is reallocated while the
        pipeline is running.  Old tensors may still be in use by a kernel or a copy of an earlier
        run(): s_in waits for both before they are dropped (their memory goes back to s_in's pool
        and could otherwise be handed out and overwritten at once)."""
        if slot.cap < n or slot.q is None or slot.q.shape[2:] != hq.shape[2:] or slot.k.shape[2:] != hk.shape[2:] \
                or slot.q.dtype != hq.dtype:
            with torch.cuda.stream(self.s_in):
                if slot.inputs_free is not None:
                    self.s_in.wait_event(slot.inputs_free)
                if slot.outputs_free is not None:
                    self.s_in.wait_event(slot.outputs_free)
                slot.q = torch.empty(1, n, *hq.shape[2:], device=self.dev, dtype=hq.dtype)
                slot.k = torch.empty(1, n, *hk.shape[2:], device=self.dev, dtype=hk.dtype)
                slot.v = torch.empty(1, n, *hv.shape[2:], device=self.dev, dtype=hv.dtype)
                slot.o = torch.empty(1, n, *hq.shape[2:], device=self.dev, dtype=hq.dtype)
                slot.lse = torch.empty(1, n, hq.shape[2], device=self.dev, dtype=torch.float32)
                made = torch.cuda.Event()
                made.record(self.s_in)
            # o and lse are first written on s_run and first read on s_out
            self.s_run.wait_event(made)
            self.s_out.wait_event(made)
            slot.cap = n

    def run(self, hq, hk, hv, cu_seqlens: Sequence[int], ho, hl, *, scale: float, scale_has_log2e: bool = False,
            causal: bool = True, lse_base2: bool = False, copies_only: bool = False) -> None:
        """hq [1, T, Hq, D], hk / hv [1, T, Hkv, D], ho like hq, hl fp32 [1, T, Hq]: pinned host
        tensors; cu_seqlens: host integers [B + 1].  Returns when the work is queued; the
        current stream is made to wait for all of it (synchronise it before reading ho / hl).
        copies_only leaves the kernels out (the same copies on the same streams with the same
        dependencies: what the host link alone allows; ho / hl then receive unspecified bytes)."""
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
            q, k, v, o, lse = slot.q[:, :n], slot.k[:, :n], slot.v[:, :n], slot.o[:, :n], slot.lse[:, :n]
            for t0, t1 in chunk_ranges(n, self.chunk, causal):
                with torch.cuda.stream(self.s_in):
                    if t0 == 0 and slot.inputs_free is not None:
                        self.s_in.wait_event(slot.inputs_free)     # the slot's previous sequence has been attended to
                    q[:, t0:t1].copy_(hq[:, s0 + t0:s0 + t1], non_blocking=True)
                    k[:, t0:t1].copy_(hk[:, s0 + t0:s0 + t1], non_blocking=True)
                    v[:, t0:t1].copy_(hv[:, s0 + t0:s0 + t1], non_blocking=True)
                    landed = torch.cuda.Event()
                    landed.record(self.s_in)
                with torch.cuda.stream(self.s_run):
                    self.s_run.wait_event(landed)
                    if t0 == 0 and slot.outputs_free is not None:
                        self.s_run.wait_event(slot.outputs_free)   # ... and its results have been copied out
                    if not copies_only:
                        ops.prefill_rows(q, k, v, o, lse, t0, t1, scale=scale, scale_has_log2e=scale_has_log2e,
                                         causal=causal, lse_base2=lse_base2)
                    done = torch.cuda.Event()
                    done.record(self.s_run)
                    slot.inputs_free = done
                with torch.cuda.stream(self.s_out):
                    self.s_out.wait_event(done)
                    ho[:, s0 + t0:s0 + t1].copy_(o[:, t0:t1], non_blocking=True)
                    hl[:, s0 + t0:s0 + t1].copy_(lse[:, t0:t1], non_blocking=True)
                    out = torch.cuda.Event()
                    out.record(self.s_out)
                    slot.outputs_free = out
        end = torch.cuda.Event()
        end.record(self.s_out)
        cur.wait_event(end)
        # the staging buffers are written on s_in and s_run and read on s_run and s_out: all of it is
        # ordered before `end` through the events above, so the caller's stream also covers them
