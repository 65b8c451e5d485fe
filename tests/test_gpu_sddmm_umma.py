"""GPU tests of the tcgen05 / tensor-memory score kernel (``f3s_sddmm_umma``): its score tiles against
the oracle's (the layout of the reference's ``process_matrix``) and against the score dump of the
mma.sync kernel on the same arrays."""
import numpy as np
import pytest
import torch

from conftest import random_csr
from fused3s_b200 import graphs
from oracle import attention_oracle as ao
from oracle import preprocess_oracle as po

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("bw", [16, 8])
@pytest.mark.parametrize("n,deg,seed", [(40, 5, 0), (257, 12, 1), (1000, 40, 2), (300, 150, 3)])
def test_score_tiles_match_oracle_and_mma_sync_dump(n, deg, seed, bw):
    from fused3s_b200 import cabi

    rowptr, colidx = random_csr(n, deg, seed)
    gen = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(n, 64, generator=gen).half() for _ in range(3))
    tcb = cabi.preprocess(torch.from_numpy(colidx).to(DEV), torch.from_numpy(rowptr).to(DEV), n, bw)
    got = cabi.sddmm_umma(tcb, n, q.to(DEV), k.to(DEV))
    torch.cuda.synchronize()
    want = ao.sddmm_tiles(po.preprocess(colidx, rowptr, n, 16, bw), n, q, k, bw).reshape(-1)
    assert got.numel() == want.numel()
    assert torch.allclose(got.cpu(), want, rtol=1e-3, atol=1e-3)
    dump = torch.zeros_like(got)
    cabi.forward(tcb, n, q.to(DEV), k.to(DEV), v.to(DEV), 1.0, sddmm_out=dump)
    torch.cuda.synchronize()
    assert torch.allclose(got, dump, rtol=1e-4, atol=1e-4)  # both accumulate fp16 products in fp32
    assert torch.equal(got == 0, dump == 0) or float(((got == 0) != (dump == 0)).float().mean()) < 1e-4


def test_score_tiles_on_a_graph_with_long_windows_and_strided_inputs():
    from fused3s_b200 import cabi

    g = graphs.make_config(4, scale=0.03)
    n = g.num_nodes
    q, k, v = graphs.make_features(g)
    tcb = cabi.preprocess(torch.from_numpy(g.colidx).to(DEV), torch.from_numpy(g.rowptr).to(DEV), n, 16)
    qkv = torch.stack([q, k, v], dim=1).to(DEV)  # [N, 3, 64]: row stride 192
    got = cabi.sddmm_umma(tcb, n, qkv[:, 0], qkv[:, 1])
    dump = torch.zeros_like(got)
    cabi.forward(tcb, n, q.to(DEV), k.to(DEV), v.to(DEV), 1.0, sddmm_out=dump)
    torch.cuda.synchronize()
    assert torch.allclose(got, dump, rtol=1e-4, atol=1e-4)
    # the number of non-zero scores is the number of edges (a score of exactly 0 has probability ~0)
    assert abs(int((got != 0).sum()) - g.nnz) <= 2
