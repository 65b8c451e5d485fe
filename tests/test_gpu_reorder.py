"""GPU test of the node-reordering row: the CUDA path run on a relabelled graph (TC blocks built from
``reorder.permute_csr``, features moved with ``reorder.apply``) and brought back with
``reorder.restore`` must meet the same bar against the oracle of the ORIGINAL graph, and the relabelled
graph's TC-block arrays must equal the CPU restatement's bit for bit."""
import numpy as np
import pytest
import torch

from fused3s_b200 import graphs, reorder
from oracle import attention_oracle as ao
from oracle import preprocess_oracle as po

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("cfg,scale", [(2, 1.0), (4, 0.05)])
@pytest.mark.parametrize("order", ["degree", "random"])
def test_forward_on_relabelled_graph_matches_oracle_of_original(cfg, scale, order):
    from fused3s_b200 import cabi

    g = graphs.make_config(cfg, scale=scale)
    n = g.num_nodes
    q, k, v = graphs.make_features(g)
    perm = reorder.degree_order(g.rowptr) if order == "degree" else np.random.default_rng(cfg).permutation(n)
    rp, ci = reorder.permute_csr(g.rowptr, g.colidx, perm, device=DEV)
    assert np.array_equal(rp, reorder.permute_csr(g.rowptr, g.colidx, perm)[0])  # device and host sort agree
    tcb = cabi.preprocess(torch.from_numpy(ci).to(DEV), torch.from_numpy(rp).to(DEV), n, 16)
    want_tcb = po.preprocess(ci, rp, n, 16, 16)
    assert tcb["nTCB"] == want_tcb["nTCB"] == reorder.tcb_count(rp, ci)
    for name in ("rowWindowOffset", "sortedRowWindows", "sparseAToXidx", "tcblock_offset", "tcblocktile_id"):
        assert np.array_equal(tcb[name].cpu().numpy(), want_tcb[name]), name
    assert np.array_equal(tcb["tcbBitMap"].cpu().numpy().view(np.uint64), want_tcb["tcbBitMap"])
    if order == "degree":
        assert tcb["nTCB"] < graphs.tcb_stats(g.rowptr, g.colidx)["nTCB"]  # the point of the relabelling
    qn, kn, vn = (reorder.apply(perm, x).to(DEV) for x in (q, k, v))
    out = reorder.restore(perm, cabi.forward(tcb, n, qn, kn, vn, 8.0)).cpu()
    want = ao.edge_attention(g.rowptr, g.colidx, q, k, v, 8.0)
    m = ao.compare(out, want)
    assert m["max_abs"] <= ao.MAX_ABS_TOL and m["mean_rel"] <= ao.MEAN_REL_TOL, m
