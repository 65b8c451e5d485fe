"""Sharding of one graph's fused attention over the GPUs of a node (one process per GPU).

The reference is single-GPU.  Two schemes, both without any collective after the kernel
except where the caller asks for the output to be moved back:

**Row-window sharding** (``ShardedAttention``; any head count).  Row windows (16 query
rows) are independent units of the fused kernel: each needs its own Q rows and TC-block
arrays plus read access to every K/V row, and writes a disjoint block of output rows.

1. ``partition_rows`` cuts the windows into ``world`` contiguous ranges with near-equal
   edge counts (host-side, from the CSR row pointer);
2. every rank preprocesses only its own block of CSR rows.  Column ids are renumbered into
   the *padded gather layout*: rank r's rows occupy ids ``[r*max_rows, r*max_rows+rows_r)``
   with ``max_rows`` the largest block, so that
3. per call, K and V -- row-sharded like Q -- are all-gathered with one equal-size NCCL
   ``all_gather_into_tensor`` each, straight into the buffer the kernel indexes (no
   unpacking copy), into each GPU's own HBM; then the local fused kernel runs on local
   memory only;
4. the output stays row-sharded.

**Head sharding** (``HeadShardedAttention``; H a multiple of the GPU count).  Every rank
runs all row windows for its own heads.  If Q/K/V are produced head-sharded (the layout a
column-parallel projection leaves them in) there is no communication at all; if they
arrive row-sharded, one all-to-all per tensor brings each rank its heads of all rows and
one all-to-all returns the output to row-sharded form -- 3.2x fewer bytes than
all-gathering K and V at 8 GPUs.

No kernel of this package reads peer memory, and nothing here waits on a flag written by
another rank: the only inter-rank synchronisation is the NCCL collective itself.
"""
from __future__ import annotations

import os

from dataclasses import dataclass

import numpy as np

from . import cabi


def partition_rows(rowptr: np.ndarray, num_nodes: int, n_parts: int, window_weight: np.ndarray | None = None) -> np.ndarray:
    """Row cut points (multiples of 16, last = num_nodes) of a contiguous partition of the row windows
    with near-equal total weight.  ``window_weight[w]`` is the cost of window w -- its TC-block count is
    what the fused kernel's time follows (``cabi.window_tcb_counts``); without it the edge count from
    ``rowptr`` stands in.  Returns int64[n_parts + 1]."""
    n_rw = (num_nodes + 15) // 16
    if window_weight is None:
        win_rows = np.minimum(np.arange(n_rw + 1, dtype=np.int64) * 16, num_nodes)
        prefix = np.ascontiguousarray(rowptr[win_rows], dtype=np.int32)  # edges before each window
    else:
        assert window_weight.shape[0] == n_rw
        prefix = np.zeros(n_rw + 1, dtype=np.int64)
        np.cumsum(window_weight.astype(np.int64), out=prefix[1:])
        assert prefix[-1] < 2**31
        prefix = prefix.astype(np.int32)
    cuts_w = cabi.partition_row_windows(prefix, n_parts)
    return np.minimum(cuts_w.astype(np.int64) * 16, num_nodes)


@dataclass
class RowShard:
    rank: int
    world: int
    row_begin: int
    row_end: int
    num_cols: int       # columns of the whole graph
    rowptr: np.ndarray  # int32, local, starts at 0
    colidx: np.ndarray  # int32, GLOBAL column ids
    row_cuts: np.ndarray
    max_rows: int       # largest row block of any rank
    local_last: bool = False  # number the rank's own columns after everybody else's (see padded_colidx)

    @property
    def num_rows(self) -> int:
        return self.row_end - self.row_begin

    @property
    def nnz(self) -> int:
        return int(self.colidx.shape[0])

    @property
    def gathered_rows(self) -> int:
        """Rows of the all-gather's output: ``world`` blocks of ``max_rows``."""
        return self.world * self.max_rows

    @property
    def col_split(self) -> int:
        """With ``local_last``: column ids at or above this value are the rank's own rows."""
        return self.world * self.max_rows

    @property
    def padded_cols(self) -> int:
        """Rows of the buffer the kernel gathers from: the ``world`` gathered blocks and, with
        ``local_last``, one more block that holds the rank's own rows (it doubles as the send buffer of
        the all-gather)."""
        return (self.world + (1 if self.local_last and self.world > 1 else 0)) * self.max_rows

    def padded_colidx(self) -> np.ndarray:
        """Column ids in the padded gather layout: a row of rank s sits at ``s*max_rows + i``, where the
        all-gather puts it (monotone in the global id, so sortedness and the TC-block structure are
        unchanged).  With ``local_last`` the rank's own rows are numbered ``world*max_rows + i`` instead
        -- the send buffer itself, which follows the gathered blocks -- so a window's own columns are the
        tail of its column list: what the fused kernel can work on before the all-gather has finished."""
        if self.world == 1:
            return self.colidx
        owner = np.searchsorted(self.row_cuts, self.colidx, side="right") - 1
        local = self.colidx.astype(np.int64) - self.row_cuts[owner]
        block = owner.astype(np.int64)
        if self.local_last:
            block = np.where(owner == self.rank, self.world, block)
        return (block * self.max_rows + local).astype(np.int32)


def make_shard(rowptr: np.ndarray, colidx: np.ndarray, num_nodes: int, rank: int, world: int,
               window_weight: np.ndarray | None = None, local_last: bool = False) -> RowShard:
    cuts = partition_rows(rowptr, num_nodes, world, window_weight)
    r0, r1 = int(cuts[rank]), int(cuts[rank + 1])
    e0, e1 = int(rowptr[r0]), int(rowptr[r1])
    local_ptr = (rowptr[r0 : r1 + 1].astype(np.int64) - e0).astype(np.int32)
    return RowShard(rank, world, r0, r1, num_nodes, local_ptr, np.ascontiguousarray(colidx[e0:e1]), cuts,
                    int(np.max(np.diff(cuts))), local_last)


class CollectiveError(RuntimeError):
    """A collective of the sharded path did not complete (a peer never joined, or the backend reported an
    error).  The reference has no counterpart (it is single-GPU); this is the host-side failure report of
    the multi-GPU layer: nothing on a GPU waits without a limit, the host learns of the failure."""


_collective_timeout_s: float | None = (
    float(os.environ["F3S_COLLECTIVE_TIMEOUT_S"]) if os.environ.get("F3S_COLLECTIVE_TIMEOUT_S") else None
)


def set_collective_timeout(seconds: float | None) -> float | None:
    """Guarded mode for every NCCL / gloo collective of this module: ``seconds`` = host-side limit per
    collective (``None`` = off, the default: collectives are enqueued and never polled).  Returns the previous
    value.  In guarded mode a collective is issued asynchronously, the host polls its completion and raises
    ``CollectiveError`` naming the collective and the rank when the limit passes or the backend reports an
    error -- at the price of one host synchronisation per collective, so it is a diagnosis mode, not the
    timed path.  (The multicast all-gather of torch symmetric memory returns no work handle and is not
    covered; its set-up is checked once, see ``ShardedAttention``.)"""
    global _collective_timeout_s
    prev = _collective_timeout_s
    _collective_timeout_s = None if seconds is None else float(seconds)
    return prev


def _run_collective(name, issue, group=None):
    """``issue(async_op)`` enqueues one collective and returns its work handle (or None)."""
    import time

    import torch.distributed as dist

    limit = _collective_timeout_s
    if limit is None:
        issue(False)
        return
    where = f"{name} on rank {dist.get_rank(group)} of {dist.get_world_size(group)}"
    try:
        work = issue(True)
        deadline = time.monotonic() + limit
        while work is not None and not work.is_completed():
            if time.monotonic() > deadline:
                raise CollectiveError(f"{where}: not complete after {limit:g} s (a peer that never joined?)")
            time.sleep(0.0005)
        if work is not None:
            work.wait()  # orders the current stream after the collective; raises what the backend recorded
    except CollectiveError:
        raise
    except Exception as exc:  # noqa: BLE001 -- whatever the backend raises is reported with its context
        raise CollectiveError(f"{where}: {exc}") from exc


def all_gather_padded(local_padded, full_padded, group=None):
    """``full_padded`` ([world*max_rows, ...]) <- every rank's ``local_padded`` ([max_rows, ...])."""
    import torch.distributed as dist

    world = full_padded.shape[0] // local_padded.shape[0]
    if world == 1 or not dist.is_initialized():
        full_padded.copy_(local_padded)
        return full_padded
    if dist.get_backend(group) == "nccl":
        _run_collective("all_gather_into_tensor",
                        lambda a: dist.all_gather_into_tensor(full_padded, local_padded, group=group, async_op=a),
                        group)
    else:  # gloo (CPU tests)
        chunks = list(full_padded.view((world,) + tuple(local_padded.shape)).unbind(0))
        _run_collective("all_gather",
                        lambda a: dist.all_gather(chunks, local_padded.contiguous(), group=group, async_op=a), group)
    return full_padded


def all_gather_rows(local, row_cuts, full=None, group=None):
    """Gather row blocks of unequal height into a dense ``full`` ([N, ...]) on every rank (used to
    assemble results for checking; the attention path itself uses ``all_gather_padded``)."""
    import torch
    import torch.distributed as dist

    n = int(row_cuts[-1])
    world = len(row_cuts) - 1
    if full is None:
        full = torch.empty((n,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    if world == 1 or not dist.is_initialized():
        full.copy_(local)
        return full
    max_rows = int(np.max(np.diff(row_cuts)))
    pad = torch.zeros((max_rows,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    pad[: local.shape[0]] = local
    gathered = [torch.empty_like(pad) for _ in range(world)]
    _run_collective("all_gather", lambda a: dist.all_gather(gathered, pad, group=group, async_op=a), group)
    for r in range(world):
        a, b = int(row_cuts[r]), int(row_cuts[r + 1])
        full[a:b].copy_(gathered[r][: b - a])
    return full


class ShardedAttention:
    """Fused sparse attention on this rank's block of rows (row-window sharding).

    K and V rows of a node are kept side by side in ONE buffer (``[rows, 2, H, d]``: the kernel takes a
    row stride, so the interleaving costs nothing), which makes the exchange one collective instead of
    two.  ``send_buffers`` hands out the views a producer writes its K / V rows into.

    With ``two_phase=True``, a ``local_last`` shard and more than one rank, ``forward`` overlaps the
    all-gather with compute: the collective runs on a side stream while the first kernel launch works on the columns the rank
    already holds (its own rows); the second launch waits for the collective's event and does the rest.
    No kernel reads another GPU's memory and nothing spins on a flag: two launches and one event.

    ``forward_fn(tcb, num_rows, q_local, k_full, v_full, scale_divisor) -> out_local`` replaces the CUDA
    path in the CPU tests, so that the partition / gather logic can run under gloo without a GPU."""

    def __init__(self, shard: RowShard, device, block_w: int = 16, forward_fn=None, preprocess_fn=None, tcb=None,
                 two_phase: bool = False, reserve_sms: int = 16, collective: str = "auto"):
        """``two_phase``: overlap the all-gather with a first kernel launch on the rank's own columns (needs
        a ``local_last`` shard).  Off by default: on B200 / NVLink 5 the collective is short (about 0.1 ms for
        60 MB) and cutting every window's work in two launches costs more than the overlap returns; it
        pays when the exchange is long compared with the kernel.
        ``reserve_sms``: SMs the two-phase forward leaves free for the collective's own kernels (the
        fused kernel is persistent and would otherwise hold every SM until its launch is finished).
        ``collective``: "nccl" = ``all_gather_into_tensor``; "multimem" = torch symmetric memory's one-shot
        all-gather through NVSwitch multicast (``symm_mem.multimem_all_gather_out``: every rank stores its
        block once to the multicast address; measured 0.102 ms against 0.140 ms for 60 MB on 8 B200);
        every rank's egress is one block, so it wins when the blocks are small -- at 2 GPUs (30 MB blocks) it
        measured 0.133 ms against NCCL's 0.095 ms); "auto" = multimem from 8 ranks on when the buffers can be
        set up on this machine, else NCCL.  ``collective_used`` says which one runs."""
        import torch

        self.reserve_sms = int(reserve_sms)
        self.shard = shard
        self.device = torch.device(device)
        self.block_w = block_w
        self.forward_fn = forward_fn
        if tcb is not None:
            self.tcb = tcb
        elif preprocess_fn is None:
            rp = torch.from_numpy(shard.rowptr).to(self.device)
            ci = torch.from_numpy(shard.padded_colidx()).to(self.device)
            self.tcb = cabi.preprocess(ci, rp, shard.num_rows, block_w, num_cols=shard.padded_cols)
        else:
            self.tcb = preprocess_fn(shard)
        self._kv = None       # [padded_cols, 2, ...]: gathered blocks (+ the own block when local_last)
        self._send = None     # [max_rows, 2, ...]: what this rank contributes to the all-gather
        self._plan = None
        self._phased = None
        self._comm_stream = None
        self.two_phase = bool(two_phase and shard.local_last and shard.world > 1 and forward_fn is None)
        if collective not in ("auto", "nccl", "multimem"):
            raise ValueError(f"collective must be auto, nccl or multimem, got {collective!r}")
        self.collective = collective
        self.collective_used = "nccl"
        self._mm_group = None

    # views of the interleaved buffers
    @property
    def _k_full(self):
        return self._kv[:, 0]

    @property
    def _v_full(self):
        return self._kv[:, 1]

    def _symmetric_buffers(self, tail, dtype, device):
        """(send, gathered) in torch symmetric memory, registered with the default group; raises if that
        cannot be set up here."""
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        s = self.shard
        gname = dist.group.WORLD.group_name
        send = symm.empty((s.max_rows, 2) + tail, dtype=dtype, device=device)
        full = symm.empty((s.gathered_rows, 2) + tail, dtype=dtype, device=device)
        symm.rendezvous(send, gname)
        symm.rendezvous(full, gname)
        # trust but verify, once: every rank's block must arrive where the kernel will look for it
        import torch

        full.zero_()
        send.fill_(float(s.rank + 1))
        torch.ops.symm_mem.multimem_all_gather_out(send, gname, full)
        torch.cuda.synchronize(device)
        firsts = full.view(s.world, -1)[:, 0].float().cpu()
        lasts = full.view(s.world, -1)[:, -1].float().cpu()
        want = torch.arange(1, s.world + 1, dtype=torch.float32)
        if not (torch.equal(firsts, want) and torch.equal(lasts, want)):
            raise RuntimeError("the multicast all-gather did not deliver every rank's block")
        send.zero_()
        full.zero_()
        return send, full, gname

    def _buffers(self, like):
        import torch

        s = self.shard
        tail = tuple(like.shape[1:])
        if self._kv is None or tuple(self._kv.shape[2:]) != tail or self._kv.dtype != like.dtype:
            self._plan = self._phased = None
            self._mm_group = None
            self.collective_used = "nccl"
            want_mm = (self.collective != "nccl" and s.world > 1 and like.device.type == "cuda"
                       and not s.local_last and self.forward_fn is None
                       and (self.collective == "multimem" or s.world >= 8))
            if want_mm:
                import torch.distributed as dist

                err, bufs = None, None
                try:
                    bufs = self._symmetric_buffers(tail, like.dtype, like.device)
                except Exception as e:  # not available here: every rank has to learn of it
                    err = e
                agreed = torch.tensor([0 if bufs is None else 1], device=like.device)
                dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
                if int(agreed) == 1:
                    self._send, self._kv, self._mm_group = bufs
                    self.collective_used = "multimem"
                    return
                if self.collective == "multimem":
                    raise err if err is not None else RuntimeError("another rank could not set up the multicast all-gather")
            self._kv = torch.zeros((s.padded_cols, 2) + tail, dtype=like.dtype, device=like.device)
            if s.local_last and s.world > 1:  # the own block follows the gathered ones and is the send buffer
                self._send = self._kv[s.gathered_rows:]
            else:
                self._send = torch.zeros((s.max_rows, 2) + tail, dtype=like.dtype, device=like.device)

    def send_buffers(self, like):
        """Persistent ``[max_rows, ...]`` views (K, V) a caller may write its K / V rows into directly
        (rows beyond its block stay zero); passing them to ``forward`` skips one local copy."""
        self._buffers(like)
        return self._send[:, 0], self._send[:, 1]

    def _stage(self, k_local, v_local):
        self._buffers(k_local)
        n = self.shard.num_rows
        if k_local.data_ptr() != self._send[:, 0].data_ptr():
            self._send[:n, 0].copy_(k_local[:n])
        if v_local.data_ptr() != self._send[:, 1].data_ptr():
            self._send[:n, 1].copy_(v_local[:n])

    def _all_gather(self):
        s = self.shard
        if self._mm_group is not None:
            import torch

            torch.ops.symm_mem.multimem_all_gather_out(self._send, self._mm_group, self._kv)
            return
        all_gather_padded(self._send, self._kv[: s.gathered_rows])

    def gather_kv(self, k_local, v_local):
        """All-gather (one collective for K and V); returns the K and V views the kernel indexes."""
        self._stage(k_local, v_local)
        self._all_gather()
        return self._k_full, self._v_full

    def forward_local(self, q_local, k_full, v_full, scale_divisor: float = 1.0):
        """Kernel only: K and V (padded gather layout) are already complete on this GPU."""
        if self.forward_fn is not None:
            return self.forward_fn(self.tcb, self.shard.num_rows, q_local, k_full, v_full, scale_divisor)
        p = self._plan
        if p is None or p.q is not q_local or p.k.data_ptr() != k_full.data_ptr() or \
                p.v.data_ptr() != v_full.data_ptr() or p.scale_divisor != scale_divisor:
            p = cabi.ForwardPlan(self.tcb, self.shard.num_rows, q_local, k_full, v_full, scale_divisor)
            self._plan = p
        p.launch()
        return p.out

    def forward(self, q_local, k_local, v_local, scale_divisor: float = 1.0):
        """All-gather K/V rows and run the fused kernel on the local rows; with a ``local_last`` shard
        the kernel's first launch (own columns) runs while the collective is in flight."""
        if not self.two_phase:
            k_full, v_full = self.gather_kv(k_local, v_local)
            return self.forward_local(q_local, k_full, v_full, scale_divisor)
        import torch

        self._stage(k_local, v_local)
        p = self._phased
        if p is None or p.q is not q_local or p.scale_divisor != float(scale_divisor):
            p = cabi.PhasedForwardPlan(self.tcb, self.shard.num_rows, q_local, self._k_full, self._v_full,
                                       scale_divisor, self.shard.col_split)
            self._phased = p
        if self._comm_stream is None:
            self._comm_stream = torch.cuda.Stream(device=self.device)
        cur = torch.cuda.current_stream(self.device)
        self._comm_stream.wait_stream(cur)  # the K / V rows of this step have been written
        with torch.cuda.stream(self._comm_stream):
            self._all_gather()
            arrived = torch.cuda.Event()
            arrived.record(self._comm_stream)
        previous = None
        if self.reserve_sms > 0:   # room for the collective's kernels beside the persistent fused kernel
            sms = torch.cuda.get_device_properties(self.device).multi_processor_count
            previous = cabi.lib().f3s_set_max_ctas(max(1, sms - self.reserve_sms))
        try:
            p.launch_phase(1)      # columns this rank owns: reads only the send block
        finally:
            if previous is not None:
                cabi.lib().f3s_set_max_ctas(previous)
        cur.wait_event(arrived)
        p.launch_phase(2)          # everybody else's columns, continuing from phase 1's state
        # the next step's K / V may overwrite the send block only after the collective has read it; the
        # wait above already orders every later operation of this stream behind the collective
        return p.out


class HeadShardedAttention:
    """Fused sparse attention with the heads divided over the ranks; every rank holds the whole
    graph's TC-block arrays and processes all row windows for ``heads/world`` heads.

    * ``forward_resident(q, k, v)``: inputs already head-sharded ``[N, heads/world, d]`` -- no
      communication.
    * ``forward_from_rows(q_rows, k_rows, v_rows)``: inputs row-sharded ``[N/world, heads, d]``
      (N divisible by world); all-to-all in, kernel, all-to-all out; returns ``[N/world, heads, d]``.
    """

    def __init__(self, rowptr: np.ndarray, colidx: np.ndarray, num_nodes: int, heads: int, rank: int, world: int,
                 device, block_w: int = 16, forward_fn=None, tcb=None):
        import torch

        assert heads % world == 0, "head sharding needs heads divisible by the number of ranks"
        self.n, self.heads, self.rank, self.world = num_nodes, heads, rank, world
        self.local_heads = heads // world
        self.device = torch.device(device)
        self.forward_fn = forward_fn
        if tcb is not None:
            self.tcb = tcb
        elif forward_fn is None:
            rp = torch.from_numpy(rowptr).to(self.device)
            ci = torch.from_numpy(colidx).to(self.device)
            self.tcb = cabi.preprocess(ci, rp, num_nodes, block_w)
        else:
            self.tcb = (rowptr, colidx)
        self._plan = None

    def forward_resident(self, q, k, v, scale_divisor: float = 1.0):
        if self.forward_fn is not None:
            return self.forward_fn(self.tcb, self.n, q, k, v, scale_divisor)
        p = self._plan
        if p is None or p.q is not q or p.k is not k or p.v is not v or p.scale_divisor != scale_divisor:
            p = cabi.ForwardPlan(self.tcb, self.n, q, k, v, scale_divisor)
            self._plan = p
        p.launch()
        return p.out

    def _rows_to_heads(self, x_rows):
        """[N/W, H, d] on every rank -> [N, H/W, d] (this rank's heads of all rows)."""
        import torch
        import torch.distributed as dist

        w, hl = self.world, self.local_heads
        rows, _, d = x_rows.shape
        send = x_rows.view(rows, w, hl, d).permute(1, 0, 2, 3).contiguous()  # [W(dest), rows, hl, d]
        recv = torch.empty_like(send)  # [W(src), rows, hl, d] == [N, hl, d]
        _all_to_all(recv, send)
        return recv.view(w * rows, hl, d)

    def _heads_to_rows(self, x_heads):
        """[N, H/W, d] -> [N/W, H, d] (all heads of this rank's rows)."""
        import torch
        import torch.distributed as dist

        w, hl = self.world, self.local_heads
        n, _, d = x_heads.shape
        rows = n // w
        send = x_heads.view(w, rows, hl, d)  # chunk j = rows of rank j, contiguous
        recv = torch.empty_like(send)  # [W(src = head group), rows, hl, d]
        _all_to_all(recv, send.contiguous())
        return recv.permute(1, 0, 2, 3).reshape(rows, w * hl, d)

    def forward_from_rows(self, q_rows, k_rows, v_rows, scale_divisor: float = 1.0):
        assert self.n % self.world == 0, "row-sharded input needs N divisible by the number of ranks"
        q = self._rows_to_heads(q_rows)
        k = self._rows_to_heads(k_rows)
        v = self._rows_to_heads(v_rows)
        out = self.forward_resident(q, k, v, scale_divisor)
        return self._heads_to_rows(out)


def _all_to_all(recv, send, group=None):
    """``recv[j]`` <- rank j's ``send[this rank]`` (equal blocks along dim 0); a copy without a process group."""
    import torch.distributed as dist

    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        recv.copy_(send)
    else:
        _run_collective("all_to_all_single",
                        lambda a: dist.all_to_all_single(recv, send, group=group, async_op=a), group)


class HeadShardedPipeline:
    """Heads over the ranks with row-sharded producers and consumers, pipelined.

    Every rank owns a block of rows (cut on 16-row boundaries) of Q, K, V and of the output, all heads;
    it computes all rows for ``heads/world`` heads.  Per call:

        exchange stream:  K+V all-to-all | Q chunk 0 | Q chunk 1 | ... | out chunk 0 | out chunk 1 | ...
        compute stream :                  (K+V, Q0) kernel 0 | kernel 1 | ...

    The rows are cut into ``chunks`` pieces that each hold the same share of EVERY rank's block (so each
    piece's all-to-all loads all links evenly); piece c has its own TC-block plan.  The kernel of piece c
    needs K and V complete but only its own Q rows, and its output leaves while piece c+1 is computed.
    K and V travel in one collective; the buffers on both sides of every collective are laid out so that
    neither the kernel nor the collective needs a transposing copy ("exchange layout"):

        q_x   [chunks, world(dest head group), seg, heads/world, d]     rows of piece c of this rank
        kv_x  [world(dest head group), 2 (K, V), chunks*seg, heads/world, d]
        out_x [chunks, world(source head group), seg, heads/world, d]   fp32

    ``to_exchange_layout`` / ``kv_to_exchange_layout`` / ``from_exchange_layout`` convert from and to
    ``[rows, heads, d]`` for callers that do not produce these layouts directly (a projection GEMM can:
    they are strided-batched outputs).  The reference is single-GPU; no counterpart there."""

    def __init__(self, rowptr: np.ndarray, colidx: np.ndarray, num_nodes: int, heads: int, rank: int, world: int,
                 device, chunks: int = 4, block_w: int = 16, forward_fn=None, reserve_sms: int = 32, group=None,
                 kv_group=None):
        """``reserve_sms``: SMs left to the collectives' kernels while the fused kernels run (the fused kernel
        is persistent and would otherwise hold every SM until its launch is finished); ``group``: the process
        group of the all-to-alls that run beside the kernels (Q and output pieces) -- one whose NCCL
        communicator is capped at about as many CTAs as SMs are reserved; ``kv_group``: the group of the K+V
        all-to-all, which precedes every kernel of the call and so may be the default, uncapped one (``ProcessGroupNCCL.Options().config.max_ctas``) overlaps best (measured on 8 B200:
        1.83 ms per step with 32 / 32 against 2.12 ms with neither)."""
        import torch

        assert heads % world == 0, "head sharding needs heads divisible by the number of ranks"
        self.reserve_sms = int(reserve_sms)
        self.group = group
        # the K+V exchange runs before any kernel of the call, so it may use an uncapped communicator
        self.kv_group = kv_group
        self.n, self.heads, self.rank, self.world = num_nodes, heads, rank, world
        self.hl = heads // world
        self.device = torch.device(device)
        self.forward_fn = forward_fn
        self.block_w = block_w
        n_rw = (num_nodes + 15) // 16
        self.cuts = np.minimum(np.round(np.arange(world + 1) * n_rw / world).astype(np.int64) * 16, num_nodes)
        self.row_begin, self.row_end = int(self.cuts[rank]), int(self.cuts[rank + 1])
        max_rows = int(np.max(np.diff(self.cuts)))
        self.chunks = max(1, min(chunks, (max_rows + 15) // 16))
        self.seg = ((max_rows + self.chunks - 1) // self.chunks + 15) // 16 * 16
        self.rows_p = self.seg * self.chunks            # padded rows per rank
        self.num_cols = world * 2 * self.rows_p          # K of rank s at s*2*rows_p + i, V rows_p further on
        self._build_plans(rowptr, colidx)
        self._bufs = None
        self._comm = None
        self._fwd = {}

    def _build_plans(self, rowptr, colidx):
        import torch

        w, seg, cuts = self.world, self.seg, self.cuts
        ptr = rowptr.astype(np.int64)
        self.plans, self.n_tcb, self.preprocess_ms = [], 0, 0.0
        for c in range(self.chunks):
            deg = np.zeros(w * seg, dtype=np.int64)
            pieces = []
            for j in range(w):
                a = min(int(cuts[j]) + c * seg, int(cuts[j + 1]))
                b = min(a + seg, int(cuts[j + 1]))
                deg[j * seg:j * seg + (b - a)] = np.diff(ptr[a:b + 1])
                pieces.append(colidx[ptr[a]:ptr[b]])
            cols = np.concatenate(pieces).astype(np.int64) if pieces else np.zeros(0, np.int64)
            owner = np.searchsorted(cuts, cols, side="right") - 1
            cols = (owner * 2 * self.rows_p + (cols - cuts[owner])).astype(np.int32)
            rp = np.zeros(w * seg + 1, dtype=np.int64)
            np.cumsum(deg, out=rp[1:])
            rp = rp.astype(np.int32)
            if self.forward_fn is not None:
                self.plans.append((rp, cols))
                continue
            with torch.cuda.device(self.device):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                tcb = cabi.preprocess(torch.from_numpy(cols).to(self.device), torch.from_numpy(rp).to(self.device),
                                      w * seg, self.block_w, num_cols=self.num_cols)
                e1.record()
                e1.synchronize()
                self.preprocess_ms += e0.elapsed_time(e1)
            self.n_tcb += tcb["nTCB"]
            self.plans.append(tcb)

    # ---- layouts
    def _pad_rows(self, x_rows):
        import torch

        rows = self.row_end - self.row_begin
        assert x_rows.shape[0] == rows
        if rows == self.rows_p:
            return x_rows
        pad = torch.zeros((self.rows_p,) + tuple(x_rows.shape[1:]), dtype=x_rows.dtype, device=x_rows.device)
        pad[:rows] = x_rows
        return pad

    def to_exchange_layout(self, q_rows):
        """``[rows, heads, d]`` of this rank -> ``q_x`` ``[chunks, world, seg, heads/world, d]``."""
        d = q_rows.shape[-1]
        x = self._pad_rows(q_rows).view(self.chunks, self.seg, self.world, self.hl, d)
        return x.permute(0, 2, 1, 3, 4).contiguous()

    def kv_to_exchange_layout(self, k_rows, v_rows):
        """Two ``[rows, heads, d]`` -> ``kv_x`` ``[world, 2, chunks*seg, heads/world, d]``."""
        import torch

        d = k_rows.shape[-1]
        kv = torch.stack([self._pad_rows(k_rows), self._pad_rows(v_rows)], dim=0)  # [2, rows_p, H, d]
        return kv.view(2, self.rows_p, self.world, self.hl, d).permute(2, 0, 1, 3, 4).contiguous()

    def from_exchange_layout(self, out_x):
        """``out_x`` ``[chunks, world, seg, heads/world, d]`` -> ``[rows, heads, d]`` of this rank."""
        d = out_x.shape[-1]
        y = out_x.permute(0, 2, 1, 3, 4).reshape(self.rows_p, self.heads, d)
        return y[: self.row_end - self.row_begin]

    def describe(self) -> str:
        return (f"{self.hl} of {self.heads} heads per GPU; row-sharded producers/consumers in exchange layout; per step: "
                f"one all-to-all for K+V, {self.chunks} for Q pieces, {self.chunks} kernel launches, {self.chunks} "
                "all-to-alls for output pieces; the exchange of a piece overlaps the kernel of its neighbours")

    def _buffers(self, q_x):
        import torch

        if self._bufs is None or self._bufs["q"].dtype != q_x.dtype or self._bufs["q"].shape != q_x.shape:
            d = q_x.shape[-1]
            dev = q_x.device
            self._bufs = {
                "q": torch.empty_like(q_x),  # [chunks, world(src), seg, hl, d]: piece c = rows of every rank
                "kv": torch.empty((self.world, 2, self.rows_p, self.hl, d), dtype=q_x.dtype, device=dev),
                "out_send": torch.empty((self.chunks, self.world, self.seg, self.hl, d), dtype=torch.float32, device=dev),
                "out": torch.empty((self.chunks, self.world, self.seg, self.hl, d), dtype=torch.float32, device=dev),
            }
            self._fwd = {}
        return self._bufs

    def _kernel(self, c: int, scale_divisor: float):
        """Launch the fused kernel of piece c on the current stream (inputs as the exchange left them)."""
        b = self._bufs
        d = b["q"].shape[-1]
        q = b["q"][c].view(self.world * self.seg, self.hl, d)
        kv = b["kv"].view(self.world * 2 * self.rows_p, self.hl, d)
        k, v = kv, kv[self.rows_p:]  # a V row sits rows_p rows behind its K row
        out = b["out_send"][c].view(self.world * self.seg, self.hl, d)
        if self.forward_fn is not None:
            out.copy_(self.forward_fn(self.plans[c], self.world * self.seg, q, k, v, scale_divisor))
            return
        key = (c, float(scale_divisor))
        p = self._fwd.get(key)
        if p is None:
            p = cabi.ForwardPlan(self.plans[c], self.world * self.seg, q, k, v, scale_divisor, out=out)
            self._fwd[key] = p
        p.launch()

    def kernel_only(self, scale_divisor: float = 8.0):
        """The kernels of all pieces back to back, no exchange (inputs as the last ``forward`` left them)."""
        for c in range(self.chunks):
            self._kernel(c, scale_divisor)

    def forward(self, q_x, kv_x, scale_divisor: float = 1.0):
        """``q_x``, ``kv_x`` in exchange layout (fp16) -> ``out_x`` in exchange layout (fp32, a buffer that
        the next call overwrites)."""
        import torch

        b = self._buffers(q_x)
        if self.device.type != "cuda":  # CPU tests: same data movement, no streams
            _all_to_all(b["kv"], kv_x, self.kv_group)
            for c in range(self.chunks):
                _all_to_all(b["q"][c], q_x[c], self.group)
                self._kernel(c, scale_divisor)
                _all_to_all(b["out"][c], b["out_send"][c], self.group)
            return b["out"]
        if self._comm is None:
            self._comm = torch.cuda.Stream(device=self.device)
        cur, comm = torch.cuda.current_stream(self.device), self._comm
        comm.wait_stream(cur)  # inputs written, previous call's kernels done with the buffers
        previous = None
        if self.reserve_sms > 0 and self.world > 1:
            sms = torch.cuda.get_device_properties(self.device).multi_processor_count
            previous = cabi.lib().f3s_set_max_ctas(max(1, sms - self.reserve_sms))
        try:
            self._enqueue(b, q_x, kv_x, scale_divisor, cur, comm)
        finally:
            if previous is not None:
                cabi.lib().f3s_set_max_ctas(previous)
        cur.wait_stream(comm)
        return b["out"]

    def _enqueue(self, b, q_x, kv_x, scale_divisor, cur, comm):
        """The collectives and kernels of one call, in issue order (see the class docstring)."""
        import torch

        q_ready = []
        with torch.cuda.stream(comm):
            _all_to_all(b["kv"], kv_x, self.kv_group)
            for c in range(self.chunks):
                _all_to_all(b["q"][c], q_x[c], self.group)
                ev = torch.cuda.Event()
                ev.record(comm)
                q_ready.append(ev)
        for c in range(self.chunks):
            cur.wait_event(q_ready[c])  # K+V were exchanged before any Q piece on the same stream
            self._kernel(c, scale_divisor)
            done = torch.cuda.Event()
            done.record(cur)
            with torch.cuda.stream(comm):
                comm.wait_event(done)
                _all_to_all(b["out"][c], b["out_send"][c], self.group)


# ---------------------------------------------------------------------------------------------------
# Row-sharded training (forward with log-sum-exp + backward)
# ---------------------------------------------------------------------------------------------------
def transpose_csr_host(rowptr: np.ndarray, colidx: np.ndarray, num_nodes: int):
    """CSR of the transposed pattern on the host (int32): row j lists, ascending, the rows i of the input
    that hold column j; repeated entries are kept once."""
    deg = np.diff(rowptr.astype(np.int64))
    rows = np.repeat(np.arange(num_nodes, dtype=np.int64), deg)
    keys = np.unique(colidx.astype(np.int64) * num_nodes + rows)
    rp = np.zeros(num_nodes + 1, dtype=np.int64)
    np.cumsum(np.bincount(keys // num_nodes, minlength=num_nodes), out=rp[1:])
    return rp.astype(np.int32), (keys % num_nodes).astype(np.int32)


def make_shard_from_cuts(rowptr: np.ndarray, colidx: np.ndarray, num_nodes: int, rank: int, world: int,
                         cuts: np.ndarray) -> RowShard:
    """``make_shard`` with given row cut points (the transposed graph must be cut where the graph is)."""
    r0, r1 = int(cuts[rank]), int(cuts[rank + 1])
    e0, e1 = int(rowptr[r0]), int(rowptr[r1])
    local_ptr = (rowptr[r0 : r1 + 1].astype(np.int64) - e0).astype(np.int32)
    return RowShard(rank, world, r0, r1, num_nodes, local_ptr, np.ascontiguousarray(colidx[e0:e1]), cuts,
                    int(np.max(np.diff(cuts))))


class ShardedTrainingAttention:
    """Forward and backward of the fused attention with the rows divided over the ranks.

    A rank owns a block of rows: its queries and the same block of keys and values, and produces the
    output rows and the gradients dq, dk, dv of that block.  Forward: K and V are all-gathered (as in
    ``ShardedAttention``).  Backward: dq needs only local data plus the gathered K/V; dk and dv of the
    block need the queries, the upstream gradients and the softmax statistics of every row that
    attends to the block, so Q, dO (fp16) and the {lse, delta} pairs are all-gathered once each and the
    rank runs the dK/dV launch on the TC blocks of ITS rows of the transposed graph.  No reduction
    across ranks, no atomics; the collectives are the only inter-rank synchronisation."""

    def __init__(self, rowptr: np.ndarray, colidx: np.ndarray, num_nodes: int, rank: int, world: int, device,
                 block_w: int = 16):
        import torch

        self.device = torch.device(device)
        self.shard = make_shard(rowptr, colidx, num_nodes, rank, world)
        self.fwd = ShardedAttention(self.shard, self.device, block_w)
        rp_t, ci_t = transpose_csr_host(rowptr, colidx, num_nodes)
        self.shard_t = make_shard_from_cuts(rp_t, ci_t, num_nodes, rank, world, self.shard.row_cuts)
        with torch.cuda.device(self.device):
            self.tcb_t = cabi.preprocess(torch.from_numpy(self.shard_t.padded_colidx()).to(self.device),
                                         torch.from_numpy(self.shard_t.rowptr).to(self.device), self.shard_t.num_rows,
                                         block_w, num_cols=self.shard_t.padded_cols)
        self._saved = None

    def _gather(self, local):
        """[rows, ...] of this rank -> padded gather layout [world * max_rows, ...] on every rank."""
        import torch

        s = self.shard
        send = torch.zeros((s.max_rows,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
        send[: s.num_rows].copy_(local)
        full = torch.empty((s.padded_cols,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
        return all_gather_padded(send, full)

    def forward_save(self, q_local, k_local, v_local, scale_divisor: float = 1.0):
        """Forward pass that returns ``(out, saved)``; ``saved`` owns everything ``backward_from`` needs
        (its gathered K/V are buffers of their own), so any number of forwards may be outstanding --
        several layers sharing one graph, gradient accumulation, an inference call in between."""
        k_full, v_full = self._gather(k_local), self._gather(v_local)
        out, lse = cabi.forward_lse(self.fwd.tcb, self.shard.num_rows, q_local, k_full, v_full, scale_divisor)
        return out, (q_local, k_local, v_local, k_full, v_full, out, lse, float(scale_divisor))

    def backward_from(self, saved, d_out_local, grad_dtype=None):
        """(dq, dk, dv) of this rank's rows for the upstream gradient of its output rows."""
        q_local, k_local, v_local, k_full, v_full, out, lse, scale = saved
        n = self.shard.num_rows
        do_h, stats = cabi.backward_prepare(out, lse, d_out_local)
        dq = cabi.backward_dq(self.fwd.tcb, n, q_local, k_full, v_full, do_h, stats, scale, grad_dtype)
        q_full, do_full, stats_full = self._gather(q_local), self._gather(do_h), self._gather(stats)
        dk, dv = cabi.backward_dkv(self.tcb_t, n, k_local, v_local, q_full, do_full, stats_full, scale, grad_dtype)
        return dq, dk, dv

    def forward(self, q_local, k_local, v_local, scale_divisor: float = 1.0):
        """One-slot convenience form: keeps what ``backward`` needs inside this object.  A second
        ``forward`` before the matching ``backward`` is refused (it would replace the saved tensors and
        the backward would silently use the wrong ones); use ``forward_save`` / ``backward_from`` for that."""
        if self._saved is not None:
            raise RuntimeError("ShardedTrainingAttention.forward called again before backward; use forward_save / "
                               "backward_from to keep several forward passes outstanding")
        out, self._saved = self.forward_save(q_local, k_local, v_local, scale_divisor)
        return out

    def backward(self, d_out_local, grad_dtype=None):
        if self._saved is None:
            raise RuntimeError("ShardedTrainingAttention.backward without a preceding forward")
        saved, self._saved = self._saved, None
        return self.backward_from(saved, d_out_local, grad_dtype)
