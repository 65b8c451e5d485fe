"""GPU test of ``f3s_forward_static``, the forward entry point for hosts that cannot allocate
device memory (a server with a memory budget frozen at load time, a runtime calling from inside
its own callback).  It must give what ``f3s_forward`` gives, call after call, although its scratch
is one fixed array that every call reuses.

Collected last on purpose (file name), so a run that stops at the first failure has already run
every other test.  The test does not depend on what ran before it: it passes alone in a fresh
process and at the end of the full suite.
"""
import numpy as np
import pytest
import torch

from fused3s_b200 import graphs
from oracle import attention_oracle as ao

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
# Two schedules of one problem cut heavy row windows at different places; every probability is rounded to
# fp16 against the running maximum of its own chunk, so the two results differ by that rounding (a few
# 1e-4 absolute on outputs of size 0.1-1), far inside the acceptance bar against the oracle (2e-2 / 1e-3).


def _problem():
    # big enough to leave the one-launch mode, with a few row windows heavy enough to be cut into
    # chunks, so that the schedule, the arrival counters and the partial results all live in scratch
    n, d = 8192, 64
    rng = np.random.default_rng(4)
    deg = np.full(n, 64, np.int64)
    deg[:16] = 4000
    deg[4096:4112] = 2500
    cols = [np.sort(rng.choice(n, size=x, replace=False)) for x in deg]
    rowptr = np.zeros(n + 1, np.int32)
    rowptr[1:] = np.cumsum(deg)
    colidx = np.concatenate(cols).astype(np.int32)
    gen = torch.Generator().manual_seed(12)
    q, k, v = (torch.randn(n, d, generator=gen).half() for _ in range(3))
    return n, rowptr, colidx, q, k, v


def test_static_scratch_forward_matches_workspace_forward_twice():
    from fused3s_b200 import cabi

    n, rowptr, colidx, q, k, v = _problem()
    tcb = cabi.preprocess(torch.from_numpy(colidx).to(DEV), torch.from_numpy(rowptr).to(DEV), n, 16)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    ws_bytes = cabi.lib().f3s_forward_workspace_bytes(tcb["rowWindowOffset"].numel() - 1, tcb["nTCB"], 16, 1, 64)
    assert 256 < ws_bytes <= cabi.STATIC_SCRATCH_BYTES  # scheduled mode (schedule + partials in scratch), no growth
    want = cabi.forward(tcb, n, qd, kd, vd, 8.0)  # the existing entry point, caller-provided workspace
    oracle = ao.edge_attention(rowptr, colidx, q, k, v, scale_divisor=8.0)
    out = torch.empty_like(want)  # every buffer is allocated before the calls under test
    torch.cuda.synchronize()
    for call in range(2):  # the second call finds the first call's leftovers in the array
        out.fill_(float("nan"))
        cabi.forward_static(tcb, n, qd, kd, vd, out, 8.0)
        torch.cuda.synchronize()
        assert torch.isfinite(out).all(), f"call {call}"
        assert torch.allclose(out, want, rtol=2e-3, atol=5e-4), f"call {call} differs from f3s_forward"
        m = ao.compare(out.cpu(), oracle)
        assert m["max_abs"] <= ao.MAX_ABS_TOL and m["mean_rel"] <= ao.MEAN_REL_TOL, (call, m)
    # a different problem right after: leftovers of a larger schedule must not leak into a smaller one
    g = graphs.make_config(3, scale=0.05)
    q2, k2, v2 = graphs.make_features(g)
    tcb2 = cabi.preprocess(torch.from_numpy(g.colidx).to(DEV), torch.from_numpy(g.rowptr).to(DEV), g.num_nodes, 16)
    want2 = cabi.forward(tcb2, g.num_nodes, q2.to(DEV), k2.to(DEV), v2.to(DEV), 8.0)
    out2 = torch.empty_like(want2)
    cabi.forward_static(tcb2, g.num_nodes, q2.to(DEV), k2.to(DEV), v2.to(DEV), out2, 8.0)
    torch.cuda.synchronize()
    assert torch.allclose(out2, want2, rtol=2e-3, atol=5e-4)


def test_static_scratch_with_chunks_grown_to_fit_and_without_any_allocation():
    """A graph whose schedule would need 87 MB with the usual chunk size: the entry point has to grow
    the chunks of heavy row windows (twice) until the scratch fits its 32 MiB, a geometry that
    ``f3s_forward`` never uses for this problem.  Also checks what the entry point is for: the device's
    free memory is the same before and after a call."""
    from fused3s_b200 import cabi

    n, d = 32768, 64
    rowptr, colidx = graphs.chung_lu(n, 6_000_000, 2.1, 4000, seed=11, device=DEV)
    gen = torch.Generator().manual_seed(13)
    q, k, v = (torch.randn(n, d, generator=gen).half() for _ in range(3))
    tcb = cabi.preprocess(torch.from_numpy(colidx).to(DEV), torch.from_numpy(rowptr).to(DEV), n, 16)
    ws_bytes = cabi.lib().f3s_forward_workspace_bytes(tcb["rowWindowOffset"].numel() - 1, tcb["nTCB"], 16, 1, d)
    assert ws_bytes > cabi.STATIC_SCRATCH_BYTES, "the case must not fit without growing the chunks"
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    want = cabi.forward(tcb, n, qd, kd, vd, 8.0)
    oracle = ao.edge_attention(rowptr, colidx, q, k, v, scale_divisor=8.0)
    out = torch.empty_like(want)
    cabi.forward_static(tcb, n, qd, kd, vd, out, 8.0)  # first call on the device: looks up the array's address
    torch.cuda.synchronize()
    for call in range(2):
        out.fill_(float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(torch.device(DEV))[0]
        cabi.forward_static(tcb, n, qd, kd, vd, out, 8.0)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info(torch.device(DEV))[0] == free_before, "the call changed the free device memory"
        cabi.forward_static_status(DEV)
        assert torch.isfinite(out).all(), f"call {call}"
        assert torch.allclose(out, want, rtol=2e-3, atol=5e-4), f"call {call} differs from f3s_forward"
        m = ao.compare(out.cpu(), oracle)
        assert m["max_abs"] <= ao.MAX_ABS_TOL and m["mean_rel"] <= ao.MEAN_REL_TOL, (call, m)
    # strided views (the three slices of one fused projection buffer) are read with their real row stride
    qkv = torch.stack([qd, kd, vd], dim=1).contiguous()  # [N, 3, d]
    out.fill_(float("nan"))
    cabi.forward_static(tcb, n, qkv[:, 0], qkv[:, 1], qkv[:, 2], out, 8.0)
    torch.cuda.synchronize()
    assert torch.allclose(out, want, rtol=2e-3, atol=5e-4)
    with pytest.raises(cabi.F3SError):  # a wrong output buffer is refused before anything is launched
        cabi.forward_static(tcb, n, qd, kd, vd, torch.empty(n, d, dtype=torch.float16, device=DEV), 8.0)


def test_static_scratch_rejects_oversized_problem():
    from fused3s_b200 import cabi

    lib = cabi.lib()
    # 130 million TC blocks: even with the largest chunks the entry point allows, the partial
    # results of the heavy windows would not fit the 32 MiB array
    n_rw = 2_000_000
    rc = lib.f3s_forward_static(None, None, None, None, n_rw * 16, n_rw, 130_000_000, 16, 1, 64, 64, None, None, None,
                                8.0, 1, None, None)
    assert rc == cabi.ERR_WORKSPACE
    msg = lib.f3s_last_error_string().decode()
    assert "too large" in msg and "f3s_forward" in msg
