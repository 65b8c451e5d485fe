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

from dataclasses import dataclass

import numpy as np

from . import cabi


def partition_rows(rowptr: np.ndarray, num_nodes: int, n_parts: int) -> np.ndarray:
    """Row cut points (multiples of 16, last = num_nodes) of a contiguous partition of the
    row windows with near-equal edge counts.  Returns int64[n_parts + 1]."""
    n_rw = (num_nodes + 15) // 16
    win_rows = np.minimum(np.arange(n_rw + 1, dtype=np.int64) * 16, num_nodes)
    prefix = np.ascontiguousarray(rowptr[win_rows], dtype=np.int32)  # edges before each window
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

    @property
    def num_rows(self) -> int:
        return self.row_end - self.row_begin

    @property
    def nnz(self) -> int:
        return int(self.colidx.shape[0])

    @property
    def padded_cols(self) -> int:
        return self.world * self.max_rows

    def padded_colidx(self) -> np.ndarray:
        """Column ids in the padded gather layout (monotone in the global id, so sortedness and
        the TC-block structure are unchanged)."""
        if self.world == 1:
            return self.colidx
        owner = np.searchsorted(self.row_cuts, self.colidx, side="right") - 1
        local = self.colidx.astype(np.int64) - self.row_cuts[owner]
        return (owner.astype(np.int64) * self.max_rows + local).astype(np.int32)


def make_shard(rowptr: np.ndarray, colidx: np.ndarray, num_nodes: int, rank: int, world: int) -> RowShard:
    cuts = partition_rows(rowptr, num_nodes, world)
    r0, r1 = int(cuts[rank]), int(cuts[rank + 1])
    e0, e1 = int(rowptr[r0]), int(rowptr[r1])
    local_ptr = (rowptr[r0 : r1 + 1].astype(np.int64) - e0).astype(np.int32)
    return RowShard(rank, world, r0, r1, num_nodes, local_ptr, np.ascontiguousarray(colidx[e0:e1]), cuts,
                    int(np.max(np.diff(cuts))))


def all_gather_padded(local_padded, full_padded, group=None):
    """``full_padded`` ([world*max_rows, ...]) <- every rank's ``local_padded`` ([max_rows, ...])."""
    import torch.distributed as dist

    world = full_padded.shape[0] // local_padded.shape[0]
    if world == 1 or not dist.is_initialized():
        full_padded.copy_(local_padded)
        return full_padded
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(full_padded, local_padded, group=group)
    else:  # gloo (CPU tests)
        chunks = list(full_padded.view((world,) + tuple(local_padded.shape)).unbind(0))
        dist.all_gather(chunks, local_padded.contiguous(), group=group)
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
    dist.all_gather(gathered, pad, group=group)
    for r in range(world):
        a, b = int(row_cuts[r]), int(row_cuts[r + 1])
        full[a:b].copy_(gathered[r][: b - a])
    return full


class ShardedAttention:
    """Fused sparse attention on this rank's block of rows (row-window sharding).

    ``forward_fn(tcb, num_rows, q_local, k_full, v_full, scale_divisor) -> out_local`` defaults
    to the CUDA path; the CPU tests substitute a checker so that the partition / gather logic
    can run under gloo without a GPU.  ``k_full``/``v_full`` are in the padded gather layout and
    the column ids the kernel sees are renumbered accordingly."""

    def __init__(self, shard: RowShard, device, block_w: int = 16, forward_fn=None, preprocess_fn=None, tcb=None):
        import torch

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
        self._k_full = None
        self._v_full = None
        self._k_send = None
        self._v_send = None
        self._plan = None

    def _buffers(self, like):
        import torch

        s = self.shard
        tail = tuple(like.shape[1:])
        if self._k_full is None or tuple(self._k_full.shape[1:]) != tail or self._k_full.dtype != like.dtype:
            mk = lambda rows: torch.zeros((rows,) + tail, dtype=like.dtype, device=like.device)
            self._k_full, self._v_full = mk(s.padded_cols), mk(s.padded_cols)
            self._k_send, self._v_send = mk(s.max_rows), mk(s.max_rows)
            self._plan = None

    def send_buffers(self, like):
        """Persistent ``[max_rows, ...]`` buffers a caller may write its K/V rows into directly
        (rows beyond its block stay zero); passing them to ``forward`` skips one local copy."""
        self._buffers(like)
        return self._k_send, self._v_send

    def gather_kv(self, k_local, v_local):
        self._buffers(k_local)
        n = self.shard.num_rows
        if k_local.data_ptr() != self._k_send.data_ptr():
            self._k_send[:n].copy_(k_local[:n])
        if v_local.data_ptr() != self._v_send.data_ptr():
            self._v_send[:n].copy_(v_local[:n])
        all_gather_padded(self._k_send, self._k_full)
        all_gather_padded(self._v_send, self._v_full)
        return self._k_full, self._v_full

    def forward_local(self, q_local, k_full, v_full, scale_divisor: float = 1.0):
        """Kernel only: K and V (padded gather layout) are already complete on this GPU."""
        if self.forward_fn is not None:
            return self.forward_fn(self.tcb, self.shard.num_rows, q_local, k_full, v_full, scale_divisor)
        p = self._plan
        if p is None or p.q is not q_local or p.k is not k_full or p.v is not v_full or p.scale_divisor != scale_divisor:
            p = cabi.ForwardPlan(self.tcb, self.shard.num_rows, q_local, k_full, v_full, scale_divisor)
            self._plan = p
        p.launch()
        return p.out

    def forward(self, q_local, k_local, v_local, scale_divisor: float = 1.0):
        """All-gather K/V rows, then run the fused kernel on the local rows."""
        k_full, v_full = self.gather_kv(k_local, v_local)
        return self.forward_local(q_local, k_full, v_full, scale_divisor)


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
        if w == 1 or not dist.is_initialized():
            recv.copy_(send)
        else:
            dist.all_to_all_single(recv, send)
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
        if w == 1 or not dist.is_initialized():
            recv.copy_(send)
        else:
            dist.all_to_all_single(recv, send.contiguous())
        return recv.permute(1, 0, 2, 3).reshape(rows, w * hl, d)

    def forward_from_rows(self, q_rows, k_rows, v_rows, scale_divisor: float = 1.0):
        assert self.n % self.world == 0, "row-sharded input needs N divisible by the number of ranks"
        q = self._rows_to_heads(q_rows)
        k = self._rows_to_heads(k_rows)
        v = self._rows_to_heads(v_rows)
        out = self.forward_resident(q, k, v, scale_divisor)
        return self._heads_to_rows(out)


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
