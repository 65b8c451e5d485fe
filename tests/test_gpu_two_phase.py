"""GPU tests of the two-phase forward (own columns first, the rest after the all-gather) and of the
plan-once launches.  Several ranks are emulated on one GPU by building each rank's shard, filling the
buffer the all-gather would leave, and running that rank's two launches; the outputs of all ranks are
compared with the oracle of the whole graph."""
import numpy as np
import pytest
import torch

from fused3s_b200 import graphs, sharding
from oracle import attention_oracle as ao

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _gathered_kv(shard, k, v):
    """The interleaved K/V buffer of one rank after the all-gather (own rows also in the last block)."""
    w, mr = shard.world, shard.max_rows
    kv = torch.zeros((shard.padded_cols, 2) + tuple(k.shape[1:]), dtype=k.dtype, device=DEV)
    for r in range(w):
        a, b = int(shard.row_cuts[r]), int(shard.row_cuts[r + 1])
        kv[r * mr:r * mr + (b - a), 0] = k[a:b].to(DEV)
        kv[r * mr:r * mr + (b - a), 1] = v[a:b].to(DEV)
    a, b = shard.row_begin, shard.row_end
    kv[w * mr:w * mr + (b - a), 0] = k[a:b].to(DEV)
    kv[w * mr:w * mr + (b - a), 1] = v[a:b].to(DEV)
    return kv


def _hub_graph(n, seed, hubs):
    rng = np.random.default_rng(seed)
    deg = rng.integers(1, 24, size=n)
    for row, d in hubs:
        deg[row:row + 16] = d
    cols = [np.sort(rng.choice(n, size=int(x), replace=False)) for x in deg]
    rowptr = np.zeros(n + 1, np.int32)
    rowptr[1:] = np.cumsum(deg)
    return rowptr, np.concatenate(cols).astype(np.int32)


@pytest.mark.parametrize("world,heads", [(2, 1), (4, 2), (8, 1)])
def test_two_phase_forward_of_every_rank_matches_oracle(world, heads):
    from fused3s_b200 import cabi

    n, d = 12000, 64
    # heavy windows (cut into chunks in both launches), one window whose columns are all its rank's own
    rowptr, colidx = _hub_graph(n, 3 + world, [(0, 5000), (6000, 7000), (11000, 3000)])
    e0, e1 = int(rowptr[32]), int(rowptr[33])
    colidx[e0:e1] = np.sort(np.random.default_rng(1).choice(200, size=e1 - e0, replace=False))  # row 32: local only
    gen = torch.Generator().manual_seed(world)
    shape = (n, d) if heads == 1 else (n, heads, d)
    q, k, v = (torch.randn(shape, generator=gen).half() for _ in range(3))
    want = ao.edge_attention(rowptr, colidx, q, k, v, 8.0)
    for rank in range(world):
        sh = sharding.make_shard(rowptr, colidx, n, rank, world, local_last=True)
        ci = sh.padded_colidx()
        own = (sh.colidx >= sh.row_begin) & (sh.colidx < sh.row_end)
        assert np.all(ci[own] >= sh.col_split) and np.all(ci[~own] < sh.col_split) and ci.max() < sh.padded_cols
        tcb = cabi.preprocess(torch.from_numpy(ci).to(DEV), torch.from_numpy(sh.rowptr).to(DEV), sh.num_rows, 16,
                              num_cols=sh.padded_cols)
        kv = _gathered_kv(sh, k, v)
        ql = q[sh.row_begin:sh.row_end].to(DEV)
        plan = cabi.PhasedForwardPlan(tcb, sh.num_rows, ql, kv[:, 0], kv[:, 1], 8.0, sh.col_split)
        for call in range(2):  # the scratch is left ready for the next pair of launches
            plan.out.fill_(float("nan"))
            plan.launch_phase(1)
            plan.launch_phase(2)
            torch.cuda.synchronize()
            m = ao.compare(plan.out.cpu(), want[sh.row_begin:sh.row_end])
            assert m["max_abs"] <= ao.MAX_ABS_TOL and m["mean_rel"] <= ao.MEAN_REL_TOL, (rank, call, m)
        one = cabi.forward(tcb, sh.num_rows, ql, kv[:, 0], kv[:, 1], 8.0)  # the same plan in one launch
        assert torch.allclose(plan.out, one, rtol=2e-3, atol=5e-4)


def test_phase_one_reads_only_the_own_block():
    """Phase 1 must not depend on anything the all-gather delivers: poison the gathered blocks while it
    runs (NaN would spread through any row that touched them), restore them for phase 2."""
    from fused3s_b200 import cabi

    g = graphs.make_config(2)
    n = g.num_nodes
    q, k, v = graphs.make_features(g)
    want = ao.edge_attention(g.rowptr, g.colidx, q, k, v, 8.0)
    sh = sharding.make_shard(g.rowptr, g.colidx, n, 1, 3, local_last=True)
    tcb = cabi.preprocess(torch.from_numpy(sh.padded_colidx()).to(DEV), torch.from_numpy(sh.rowptr).to(DEV),
                          sh.num_rows, 16, num_cols=sh.padded_cols)
    kv = _gathered_kv(sh, k, v)
    good = kv[:sh.gathered_rows].clone()
    plan = cabi.PhasedForwardPlan(tcb, sh.num_rows, q[sh.row_begin:sh.row_end].to(DEV), kv[:, 0], kv[:, 1], 8.0,
                                  sh.col_split)
    kv[:sh.gathered_rows] = float("nan")
    plan.launch_phase(1)
    torch.cuda.synchronize()
    kv[:sh.gathered_rows] = good
    plan.launch_phase(2)
    torch.cuda.synchronize()
    assert torch.isfinite(plan.out).all()
    m = ao.compare(plan.out.cpu(), want[sh.row_begin:sh.row_end])
    assert m["max_abs"] <= ao.MAX_ABS_TOL and m["mean_rel"] <= ao.MEAN_REL_TOL, m


@pytest.mark.parametrize("cfg,scale", [(3, 0.05), (4, 0.03)])
def test_plan_once_launches_repeat_bit_for_bit(cfg, scale):
    """ForwardPlan schedules on its first launch only; every later launch is the fused kernel alone on
    the scratch the previous launch left behind (counters back at zero), also with interleaved K / V."""
    from fused3s_b200 import cabi

    g = graphs.make_config(cfg, scale=scale)
    n = g.num_nodes
    q, k, v = graphs.make_features(g)
    tcb = cabi.preprocess(torch.from_numpy(g.colidx).to(DEV), torch.from_numpy(g.rowptr).to(DEV), n, 16)
    kv = torch.stack([k, v], dim=1).to(DEV)  # [N, 2, d]: one buffer, row stride 2 d
    plan = cabi.ForwardPlan(tcb, n, q.to(DEV), kv[:, 0], kv[:, 1], 8.0)
    assert plan.ld_kv == 2 * plan.ld
    lib = cabi.lib()
    outs = []
    for call in range(4):
        before = lib.f3s_kernel_launch_count()
        plan.out.fill_(float("nan"))
        plan.launch()
        torch.cuda.synchronize()
        launches = lib.f3s_kernel_launch_count() - before
        assert launches == (2 if call == 0 and plan.ws_bytes > 256 else 1), (call, launches)
        outs.append(plan.out.clone())
        plan.status()
    assert all(torch.equal(outs[0], o) for o in outs[1:])
    m = ao.compare(outs[0].cpu(), ao.edge_attention(g.rowptr, g.colidx, q, k, v, 8.0))
    assert m["max_abs"] <= ao.MAX_ABS_TOL and m["mean_rel"] <= ao.MEAN_REL_TOL, m
    assert torch.equal(outs[0], cabi.forward(tcb, n, q.to(DEV), k.to(DEV), v.to(DEV), 8.0))
