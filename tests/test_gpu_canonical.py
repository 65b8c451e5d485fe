"""GPU tests of the canonical schedule (``f3s_set_canonical_chunk_tiles``): with it, a row window is
computed by the same sequence of operations whether it is part of the whole graph on one GPU, of a row
shard (ranks emulated on one GPU here), of a one-head or a multi-head call, or runs on the built-in scratch
of ``f3s_forward_static`` -- the outputs are equal bit for bit."""
import numpy as np
import pytest
import torch

from fused3s_b200 import graphs, sharding
from oracle import attention_oracle as ao

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture()
def canonical():
    from fused3s_b200 import cabi

    cabi.lib().f3s_set_canonical_chunk_tiles(128)
    yield
    cabi.lib().f3s_set_canonical_chunk_tiles(0)


@pytest.mark.parametrize("cfg,scale,world", [(4, 0.05, 2), (4, 0.05, 8), (5, 0.02, 4), (3, 0.05, 2), (2, 1.0, 3)])
def test_row_shards_equal_single_gpu_bit_for_bit(canonical, cfg, scale, world):
    from fused3s_b200 import cabi

    g = graphs.make_config(cfg, scale=scale)
    n = g.num_nodes
    q, k, v = graphs.make_features(g)
    tcb = cabi.preprocess(torch.from_numpy(g.colidx).to(DEV), torch.from_numpy(g.rowptr).to(DEV), n, 16)
    whole = cabi.forward(tcb, n, q.to(DEV), k.to(DEV), v.to(DEV), 8.0)
    want = ao.edge_attention(g.rowptr, g.colidx, q, k, v, 8.0)
    m = ao.compare(whole.cpu(), want)
    assert m["max_abs"] <= ao.MAX_ABS_TOL and m["mean_rel"] <= ao.MEAN_REL_TOL, m
    if g.heads > 1:  # a head of the multi-head call equals the one-head call on that head
        one = cabi.forward(tcb, n, q[:, 1].to(DEV), k[:, 1].to(DEV), v[:, 1].to(DEV), 8.0)
        assert torch.equal(one, whole[:, 1])
    for rank in range(world):
        sh = sharding.make_shard(g.rowptr, g.colidx, n, rank, world)  # padded layout that keeps the column order
        if sh.num_rows == 0:
            continue
        t = cabi.preprocess(torch.from_numpy(sh.padded_colidx()).to(DEV), torch.from_numpy(sh.rowptr).to(DEV),
                            sh.num_rows, 16, num_cols=sh.padded_cols)
        kf = torch.zeros((sh.padded_cols,) + tuple(k.shape[1:]), dtype=k.dtype, device=DEV)
        vf = torch.zeros_like(kf)
        for r in range(world):
            a, b = int(sh.row_cuts[r]), int(sh.row_cuts[r + 1])
            kf[r * sh.max_rows:r * sh.max_rows + (b - a)] = k[a:b].to(DEV)
            vf[r * sh.max_rows:r * sh.max_rows + (b - a)] = v[a:b].to(DEV)
        part = cabi.forward(t, sh.num_rows, q[sh.row_begin:sh.row_end].to(DEV), kf, vf, 8.0)
        assert torch.equal(part, whole[sh.row_begin:sh.row_end]), f"rank {rank} of {world}"


def test_static_scratch_equals_workspace_forward_bit_for_bit(canonical):
    from fused3s_b200 import cabi

    n, d = 8192, 64
    rng = np.random.default_rng(4)
    deg = np.full(n, 64, np.int64)
    deg[:16] = 4000
    deg[4096:4112] = 2500
    cols = [np.sort(rng.choice(n, size=x, replace=False)) for x in deg]
    rowptr = np.zeros(n + 1, np.int32)
    rowptr[1:] = np.cumsum(deg)
    colidx = np.concatenate(cols).astype(np.int32)
    gen = torch.Generator().manual_seed(13)
    q, k, v = (torch.randn(n, d, generator=gen).half().to(DEV) for _ in range(3))
    tcb = cabi.preprocess(torch.from_numpy(colidx).to(DEV), torch.from_numpy(rowptr).to(DEV), n, 16)
    want = cabi.forward(tcb, n, q, k, v, 8.0)
    out = torch.empty_like(want)
    for _ in range(2):
        out.fill_(float("nan"))
        cabi.forward_static(tcb, n, q, k, v, out, 8.0)
        torch.cuda.synchronize()
        assert torch.equal(out, want)
