"""CPU tests of the multi-GPU host logic with world_size-2 gloo ranks: the edge-balanced
row-window partition, per-rank CSR slices, the uneven all-gather of K/V rows, and that the
sharded outputs concatenate to the single-rank result.  The compute step is a checker
(the CPU oracle) injected through ``forward_fn``; the product's CUDA path is covered by the
GPU tests."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import random_csr
from fused3s_b200 import sharding
from oracle import attention_oracle as ao


def test_partition_balances_edges_and_cuts_on_windows():
    rowptr, colidx = random_csr(1000, 20, 0)
    for parts in (1, 2, 3, 8):
        cuts = sharding.partition_rows(rowptr, 1000, parts)
        assert cuts[0] == 0 and cuts[-1] == 1000 and np.all(np.diff(cuts) >= 0)
        assert all(int(c) % 16 == 0 for c in cuts[:-1])
        per = np.diff(rowptr[cuts])
        assert per.sum() == len(colidx)
        if parts > 1:
            assert per.max() <= len(colidx) / parts + 2 * 16 * 40  # within two windows of the ideal


def test_shards_cover_the_graph():
    rowptr, colidx = random_csr(333, 9, 1)
    got_cols, got_rows = [], 0
    for r in range(4):
        s = sharding.make_shard(rowptr, colidx, 333, r, 4)
        assert s.rowptr[0] == 0 and s.rowptr[-1] == s.nnz and s.num_cols == 333
        got_cols.append(s.colidx)
        got_rows += s.num_rows
    assert got_rows == 333 and np.array_equal(np.concatenate(got_cols), colidx)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_forward(shard, num_rows, q_local, k_full, v_full, scale):
    # `shard` stands in for the TC-block arrays (see preprocess_fn below); K/V arrive in the padded
    # gather layout, so the columns are looked up through the shard's renumbered ids
    return ao.edge_attention(shard.rowptr, shard.padded_colidx(), q_local, k_full, v_full, scale,
                             row_begin=0, row_end=num_rows)


def _worker(rank, world, port, rowptr, colidx, n, heads, out_file):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        gen = torch.Generator().manual_seed(7)
        shape = (n, 16) if heads == 1 else (n, heads, 16)
        q, k, v = (torch.randn(shape, generator=gen).half() for _ in range(3))
        shard = sharding.make_shard(rowptr, colidx, n, rank, world)
        attn = sharding.ShardedAttention(shard, "cpu", forward_fn=_oracle_forward, preprocess_fn=lambda s: s)
        r0, r1 = shard.row_begin, shard.row_end
        out = attn.forward(q[r0:r1], k[r0:r1], v[r0:r1], 4.0)
        # K/V were really exchanged: every rank's block sits at its padded position
        for r in range(world):
            a, b = int(shard.row_cuts[r]), int(shard.row_cuts[r + 1])
            assert torch.equal(attn._k_full[r * shard.max_rows : r * shard.max_rows + (b - a)], k[a:b])
            assert torch.equal(attn._v_full[r * shard.max_rows : r * shard.max_rows + (b - a)], v[a:b])
        full = ao.edge_attention(rowptr, colidx, q, k, v, 4.0)
        assert torch.allclose(out, full[r0:r1], rtol=1e-6, atol=1e-6)
        gathered = sharding.all_gather_rows(out, shard.row_cuts)
        assert torch.allclose(gathered, full, rtol=1e-6, atol=1e-6)
        if rank == 0:
            torch.save({"ok": True, "rows": [int(c) for c in shard.row_cuts]}, out_file)
    finally:
        dist.destroy_process_group()


def _head_worker(rank, world, port, rowptr, colidx, n, heads, out_file):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        gen = torch.Generator().manual_seed(9)
        q, k, v = (torch.randn((n, heads, 16), generator=gen).half() for _ in range(3))
        full = ao.edge_attention(rowptr, colidx, q, k, v, 4.0)
        fn = lambda tcb, nn, qq, kk, vv, sc: ao.edge_attention(tcb[0], tcb[1], qq, kk, vv, sc)
        attn = sharding.HeadShardedAttention(rowptr, colidx, n, heads, rank, world, "cpu", forward_fn=fn)
        hl = heads // world
        # inputs already head-sharded: no communication
        out_h = attn.forward_resident(q[:, rank * hl:(rank + 1) * hl].contiguous(),
                                      k[:, rank * hl:(rank + 1) * hl].contiguous(),
                                      v[:, rank * hl:(rank + 1) * hl].contiguous(), 4.0)
        assert torch.allclose(out_h, full[:, rank * hl:(rank + 1) * hl], rtol=1e-6, atol=1e-6)
        # inputs row-sharded: all-to-all in and out
        rows = n // world
        sl = slice(rank * rows, (rank + 1) * rows)
        out_r = attn.forward_from_rows(q[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous(), 4.0)
        assert out_r.shape == (rows, heads, 16)
        assert torch.allclose(out_r, full[sl], rtol=1e-6, atol=1e-6)
        if rank == 0:
            torch.save({"ok": True}, out_file)
    finally:
        dist.destroy_process_group()


def test_two_rank_head_sharded_forward_equals_single(tmp_path):
    n = 256
    rowptr, colidx = random_csr(n, 9, 6)
    out_file = str(tmp_path / "res.pt")
    mp.spawn(_head_worker, args=(2, _free_port(), rowptr, colidx, n, 4, out_file), nprocs=2, join=True)
    assert torch.load(out_file)["ok"]


def _pipeline_worker(rank, world, port, rowptr, colidx, n, heads, chunks, out_file):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        gen = torch.Generator().manual_seed(11)
        q, k, v = (torch.randn((n, heads, 16), generator=gen).half() for _ in range(3))
        full = ao.edge_attention(rowptr, colidx, q, k, v, 4.0)
        fn = lambda plan, rows, qq, kk, vv, sc: ao.edge_attention(plan[0], plan[1], qq, kk, vv, sc)
        hp = sharding.HeadShardedPipeline(rowptr, colidx, n, heads, rank, world, "cpu", chunks=chunks, forward_fn=fn)
        assert hp.row_begin % 16 == 0 and hp.seg % 16 == 0
        rb, re_ = hp.row_begin, hp.row_end
        q_x = hp.to_exchange_layout(q[rb:re_])
        kv_x = hp.kv_to_exchange_layout(k[rb:re_], v[rb:re_])
        # the layouts round-trip
        assert torch.equal(hp.from_exchange_layout(q_x.float()), q[rb:re_].float())
        for _ in range(2):
            out = hp.from_exchange_layout(hp.forward(q_x, kv_x, 4.0))
            assert out.shape == (re_ - rb, heads, 16)
            assert torch.allclose(out, full[rb:re_], rtol=1e-6, atol=1e-6)
        if rank == 0:
            torch.save({"ok": True}, out_file)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n,heads,chunks", [(256, 4, 2), (301, 2, 3)])
def test_two_rank_head_sharded_pipeline_equals_single(tmp_path, n, heads, chunks):
    rowptr, colidx = random_csr(n, 9, 16)
    out_file = str(tmp_path / "res.pt")
    mp.spawn(_pipeline_worker, args=(2, _free_port(), rowptr, colidx, n, heads, chunks, out_file), nprocs=2, join=True)
    assert torch.load(out_file)["ok"]


def test_local_last_numbering_splits_own_and_other_columns():
    rowptr, colidx = random_csr(500, 12, 3)
    for r in range(3):
        s = sharding.make_shard(rowptr, colidx, 500, r, 3, local_last=True)
        pc = s.padded_colidx().astype(np.int64)
        own = (s.colidx >= s.row_begin) & (s.colidx < s.row_end)
        assert pc.max() < s.padded_cols == 4 * s.max_rows
        assert np.all(pc[own] >= s.col_split) and np.all(pc[~own] < s.col_split)
        # other ranks' columns keep their order; own columns keep theirs
        assert np.array_equal(np.argsort(pc[~own], kind="stable"), np.argsort(s.colidx[~own], kind="stable"))
        assert np.array_equal(np.argsort(pc[own], kind="stable"), np.argsort(s.colidx[own], kind="stable"))
    w = np.ones((500 + 15) // 16, dtype=np.int64)
    w[:4] = 50  # heavy first windows: the cut moves forward
    cuts = sharding.partition_rows(rowptr, 500, 2, window_weight=w)
    assert cuts[1] < sharding.partition_rows(rowptr, 500, 2)[1]


def test_padded_column_ids_are_monotone():
    rowptr, colidx = random_csr(500, 12, 3)
    for r in range(3):
        s = sharding.make_shard(rowptr, colidx, 500, r, 3)
        pc = s.padded_colidx().astype(np.int64)
        assert pc.max() < s.padded_cols
        # order-preserving renumbering: sorting by padded id == sorting by global id
        assert np.array_equal(np.argsort(pc, kind="stable"), np.argsort(s.colidx, kind="stable"))


@pytest.mark.parametrize("heads", [1, 2])
def test_two_rank_sharded_forward_equals_single(tmp_path, heads):
    n = 300
    rowptr, colidx = random_csr(n, 11, 5)
    out_file = str(tmp_path / "res.pt")
    mp.spawn(_worker, args=(2, _free_port(), rowptr, colidx, n, heads, out_file), nprocs=2, join=True)
    res = torch.load(out_file)
    assert res["ok"] and res["rows"][0] == 0 and res["rows"][-1] == n


def test_phase_split_array_names_the_only_block_with_columns_of_both_kinds():
    """The two-launch forward's ``phase_split[w]``: first TC block of window w whose FIRST column id is at or
    above the split; every block before the one preceding it holds only lower ids, every block from it on only
    higher ones (checked by brute force on the oracle's TC-block arrays, CPU tensors)."""
    from fused3s_b200 import cabi
    from oracle import preprocess_oracle as po

    n = 400
    rowptr, colidx = random_csr(n, 30, 21)
    tcb_np = po.preprocess(colidx, rowptr, n, 16, 16)
    tcb = {"block_w": 16, "rowWindowOffset": torch.from_numpy(tcb_np["rowWindowOffset"]),
           "sparseAToXidx": torch.from_numpy(tcb_np["sparseAToXidx"])}
    rwo, atox = tcb_np["rowWindowOffset"], tcb_np["sparseAToXidx"].reshape(-1, 16)
    for split in (0, 1, 137, 250, n, n + 5):
        ps = cabi.phase_split_array(tcb, split).numpy()
        for w in range(len(rwo) - 1):
            a, z, lb = int(rwo[w]), int(rwo[w + 1]), int(ps[w])
            assert a <= lb <= z
            for t in range(a, z):
                first = int(atox[t, 0])
                assert (first >= split) == (t >= lb), (w, t, first, split, lb)
            # blocks before lb - 1 hold nothing at or above the split (padding slots of a last block are 0)
            for t in range(a, max(a, lb - 1)):
                assert int(atox[t].max()) < split


def _guard_worker(rank, world, port, out_file):
    """Host-made failure: rank 1 joins the first collective and then never calls the second one."""
    import time

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    assert sharding.set_collective_timeout(1.5) is None
    local = torch.full((4, 3), float(rank + 1))
    full = torch.zeros(world * 4, 3)
    sharding.all_gather_padded(local, full)  # guarded, every rank joins: completes, result as without the guard
    ok = bool(torch.equal(full[:4], torch.full((4, 3), 1.0)) and torch.equal(full[4:], torch.full((4, 3), 2.0)))
    recv = torch.zeros(world, 2)
    sharding._all_to_all(recv, torch.full((world, 2), float(rank)))
    ok = ok and bool(torch.equal(recv[:, 0], torch.arange(world, dtype=torch.float32)))
    if rank == 1:
        time.sleep(4.0)  # never joins the next collective; leaves between steps, nothing of its own in flight
        os._exit(0)
    t0 = time.monotonic()
    try:
        sharding.all_gather_padded(local, full)
        outcome = "completed"
    except sharding.CollectiveError as e:
        outcome = "raised" if ("rank 0 of 2" in str(e) and "all_gather" in str(e)) else f"wrong message: {e}"
    torch.save({"ok": ok, "outcome": outcome, "seconds": time.monotonic() - t0}, out_file)
    os._exit(0)  # the abandoned collective would block an orderly shutdown of the process group


def test_guarded_collective_reports_a_rank_that_never_joins(tmp_path):
    out_file = str(tmp_path / "res.pt")
    mp.spawn(_guard_worker, args=(2, _free_port(), out_file), nprocs=2, join=True)
    res = torch.load(out_file)
    assert res["ok"] and res["outcome"] == "raised", res
    assert 1.4 <= res["seconds"] <= 3.5, res
