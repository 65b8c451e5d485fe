"""GPU test of the host-buffer pipeline (fused3s_b200/host_pipeline.py): chunked preprocessing plus
overlapped copies must give what one plain call gives."""
import pytest
import torch

from fused3s_b200 import graphs
from oracle import attention_oracle as ao

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("kv_halves", [False, True])
@pytest.mark.parametrize("cfg,scale,chunks", [(4, 0.02, 4), (5, 0.01, 3), (1, 1.0, 8)])
def test_host_pipeline_matches_single_call(cfg, scale, chunks, kv_halves):
    from fused3s_b200 import cabi
    from fused3s_b200.host_pipeline import HostPipelinedAttention

    g = graphs.make_config(cfg, scale=scale)
    q, k, v = (x.pin_memory() for x in graphs.make_features(g))
    pipe = HostPipelinedAttention(g.rowptr, g.colidx, g.num_nodes, g.heads, g.dim, DEV, chunks=chunks,
                                  kv_halves=kv_halves)
    assert pipe.kv_halves == kv_halves  # K and V in two halves, every chunk as the two-launch forward
    out_host = torch.empty(q.shape, dtype=torch.float32).pin_memory()
    for _ in range(2):  # buffers and plans are reused from the second call on
        out_host.fill_(float("nan"))
        pipe.forward(q, k, v, out_host, 8.0).synchronize()
        assert torch.isfinite(out_host).all()
    tcb = cabi.preprocess(torch.from_numpy(g.colidx).to(DEV), torch.from_numpy(g.rowptr).to(DEV), g.num_nodes, 16)
    single = cabi.forward(tcb, g.num_nodes, q.to(DEV), k.to(DEV), v.to(DEV), 8.0).cpu()
    m = ao.compare(out_host, single)
    assert m["max_abs"] <= 5e-3 and m["mean_rel"] <= 5e-4, m  # chunk boundaries move the split points
    want = ao.edge_attention(g.rowptr, g.colidx, q, k, v, 8.0)
    m = ao.compare(out_host, want)
    assert m["max_abs"] <= ao.MAX_ABS_TOL and m["mean_rel"] <= ao.MEAN_REL_TOL, m
