"""Fused attention for callers whose Q/K/V and output live in HOST memory (one GPU).

The reference's ops take device tensors; a caller with host data pays three host->device copies,
the kernel and one device->host copy back to back.  Here the row windows are cut into a few chunks
(by edge count, on 16-row boundaries) that are preprocessed separately once per graph, and every
call runs a three-stream pipeline:

    copy-in stream :  K, V | Q chunk 0 | Q chunk 1 | ...
    compute stream :          (wait K, V, Q0) kernel 0 | kernel 1 | ...
    copy-out stream:                                 out 0 | out 1 | ...

so the copy of the output (the largest transfer: fp32) and of the later Q chunks overlaps the kernel.
K and V must be complete before a window can be finished because every window gathers arbitrary rows --
but not before it can be started: with ``kv_halves`` (head dim 64, fp32 output) K and V travel in two
halves and every chunk runs as the two-launch forward (``f3s_forward_phase``): launch 1 works on the
columns of the half that has arrived while the other half is still on the bus, launch 2 continues from
the state launch 1 left and writes the output:

    copy-in stream :  K,V upper half | Q chunks | K,V lower half
    compute stream :                  (upper, Q0) launch 1 of chunk 0 | ... | (lower) launch 2 of chunk 0 | ...
    copy-out stream:                                                                           out 0 | ...

Host buffers should be pinned; pageable ones work but serialise.
"""
from __future__ import annotations

import numpy as np

from . import cabi, sharding


class HostPipelinedAttention:
    def __init__(self, rowptr: np.ndarray, colidx: np.ndarray, num_nodes: int, heads: int, dim: int, device="cuda",
                 chunks: int = 4, block_w: int = 16, out_dtype=None, kv_halves=None):
        """``kv_halves``: None = on when the two-launch forward applies (head dim 64, fp32 output) and the
        graph is large enough for the saved copy time to exceed the second launch's overhead."""
        import torch

        self.n, self.heads, self.dim = num_nodes, heads, dim
        self.device = torch.device(device)
        self.out_dtype = torch.float32 if out_dtype is None else out_dtype
        can_split = dim == 64 and self.out_dtype == torch.float32 and num_nodes >= 32
        self.kv_halves = (can_split and num_nodes * heads >= 100_000) if kv_halves is None else (bool(kv_halves) and can_split)
        self.col_split = (num_nodes // 2) // 16 * 16  # columns >= this id are the half that is copied first
        chunks = max(1, min(chunks, (num_nodes + 15) // 16))
        self.cuts = sharding.partition_rows(rowptr, num_nodes, chunks)
        shape = (num_nodes, dim) if heads == 1 else (num_nodes, heads, dim)
        with torch.cuda.device(self.device):
            self.q_dev = torch.empty(shape, dtype=torch.float16, device=self.device)
            self.k_dev = torch.empty_like(self.q_dev)
            self.v_dev = torch.empty_like(self.q_dev)
            self.out_dev = torch.empty(shape, dtype=self.out_dtype, device=self.device)
            self.plans = []
            for c in range(chunks):
                r0, r1 = int(self.cuts[c]), int(self.cuts[c + 1])
                if r1 == r0:
                    continue
                e0, e1 = int(rowptr[r0]), int(rowptr[r1])
                rp = torch.from_numpy((rowptr[r0:r1 + 1].astype(np.int64) - e0).astype(np.int32)).to(self.device)
                ci = torch.from_numpy(np.ascontiguousarray(colidx[e0:e1])).to(self.device)
                tcb = cabi.preprocess(ci, rp, r1 - r0, block_w, num_cols=num_nodes)
                self.plans.append((r0, r1, tcb))
            self.s_in = torch.cuda.Stream(device=self.device)
            self.s_out = torch.cuda.Stream(device=self.device)
        self._fwd = {}

    def _plan(self, idx: int, scale_divisor: float):
        key = (idx, float(scale_divisor))
        p = self._fwd.get(key)
        if p is None:
            r0, r1, tcb = self.plans[idx]
            p = cabi.ForwardPlan(tcb, r1 - r0, self.q_dev[r0:r1], self.k_dev, self.v_dev, scale_divisor,
                                 out=self.out_dev[r0:r1])
            self._fwd[key] = p
        return p

    def _phased(self, idx: int, scale_divisor: float):
        key = ("phased", idx, float(scale_divisor))
        p = self._fwd.get(key)
        if p is None:
            r0, r1, tcb = self.plans[idx]
            p = cabi.PhasedForwardPlan(tcb, r1 - r0, self.q_dev[r0:r1], self.k_dev, self.v_dev, scale_divisor,
                                       self.col_split, out=self.out_dev[r0:r1])
            self._fwd[key] = p
        return p

    def _forward_kv_halves(self, q_host, k_host, v_host, out_host, scale_divisor: float):
        import torch

        sp = self.col_split
        with torch.cuda.device(self.device):
            cur = torch.cuda.current_stream()
            start = torch.cuda.Event()
            start.record(cur)
            self.s_in.wait_event(start)
            self.s_out.wait_event(start)
            q_ready = []
            with torch.cuda.stream(self.s_in):
                self.k_dev[sp:].copy_(k_host[sp:], non_blocking=True)
                self.v_dev[sp:].copy_(v_host[sp:], non_blocking=True)
                for r0, r1, _ in self.plans:
                    self.q_dev[r0:r1].copy_(q_host[r0:r1], non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(self.s_in)
                    q_ready.append(ev)
                self.k_dev[:sp].copy_(k_host[:sp], non_blocking=True)
                self.v_dev[:sp].copy_(v_host[:sp], non_blocking=True)
                kv_all = torch.cuda.Event()
                kv_all.record(self.s_in)
            for idx in range(len(self.plans)):  # the upper halves precede every Q chunk on the copy stream
                cur.wait_event(q_ready[idx])
                self._phased(idx, scale_divisor).launch_phase(1)
            cur.wait_event(kv_all)
            last = None
            for idx, (r0, r1, _) in enumerate(self.plans):
                self._phased(idx, scale_divisor).launch_phase(2)
                done = torch.cuda.Event()
                done.record(cur)
                with torch.cuda.stream(self.s_out):
                    self.s_out.wait_event(done)
                    out_host[r0:r1].copy_(self.out_dev[r0:r1], non_blocking=True)
                    last = torch.cuda.Event()
                    last.record(self.s_out)
            if last is not None:
                cur.wait_event(last)
            end = torch.cuda.Event()
            end.record(cur)
        return end

    def forward(self, q_host, k_host, v_host, out_host, scale_divisor: float = 1.0):
        """q/k/v_host: fp16 host tensors of shape [N, d] or [N, H, d]; out_host: host tensor of the
        output dtype and the same shape.  Returns after everything is enqueued; the event returned is
        recorded after the last device->host copy (``event.synchronize()`` before reading out_host)."""
        import torch

        if self.kv_halves:
            return self._forward_kv_halves(q_host, k_host, v_host, out_host, scale_divisor)

        with torch.cuda.device(self.device):
            cur = torch.cuda.current_stream()
            start = torch.cuda.Event()
            start.record(cur)
            self.s_in.wait_event(start)
            self.s_out.wait_event(start)
            with torch.cuda.stream(self.s_in):
                self.k_dev.copy_(k_host, non_blocking=True)
                self.v_dev.copy_(v_host, non_blocking=True)
                kv_ready = torch.cuda.Event()
                kv_ready.record(self.s_in)
            cur.wait_event(kv_ready)
            last = None
            for idx, (r0, r1, _) in enumerate(self.plans):
                with torch.cuda.stream(self.s_in):
                    self.q_dev[r0:r1].copy_(q_host[r0:r1], non_blocking=True)
                    q_ready = torch.cuda.Event()
                    q_ready.record(self.s_in)
                cur.wait_event(q_ready)
                self._plan(idx, scale_divisor).launch()  # on the current stream
                done = torch.cuda.Event()
                done.record(cur)
                with torch.cuda.stream(self.s_out):
                    self.s_out.wait_event(done)
                    out_host[r0:r1].copy_(self.out_dev[r0:r1], non_blocking=True)
                    last = torch.cuda.Event()
                    last.record(self.s_out)
            if last is not None:
                cur.wait_event(last)  # later work on the caller's stream is ordered after the copies
            end = torch.cuda.Event()
            end.record(cur)
        return end
