"""GPU tests of the error-reporting side of the C ABI: the device status word (a kernel that cannot
finish says so and the host can ask), and the plan check that stands in for a memory checker on plans
that did not come from the preprocessing calls.  Nothing here faults, traps or waits: the only
failure provoked is a pure bounds check in the schedule kernel."""
import ctypes as C

import numpy as np
import pytest
import torch

from fused3s_b200 import graphs
from oracle import attention_oracle as ao

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _heavy_problem():
    # several row windows far above the split threshold, enough work to leave the one-launch mode
    n, d = 8192, 64
    rng = np.random.default_rng(9)
    deg = np.full(n, 64, np.int64)
    deg[:16] = 4000
    deg[1024:1040] = 3000
    deg[4096:4112] = 2500
    cols = [np.sort(rng.choice(n, size=x, replace=False)) for x in deg]
    rowptr = np.zeros(n + 1, np.int32)
    rowptr[1:] = np.cumsum(deg)
    colidx = np.concatenate(cols).astype(np.int32)
    gen = torch.Generator().manual_seed(3)
    q, k, v = (torch.randn(n, d, generator=gen).half() for _ in range(3))
    return n, rowptr, colidx, q, k, v


def test_status_is_ok_after_normal_calls_and_reports_unit_list_overflow():
    from fused3s_b200 import cabi

    lib = cabi.lib()
    n, rowptr, colidx, q, k, v = _heavy_problem()
    tcb = cabi.preprocess(torch.from_numpy(colidx).to(DEV), torch.from_numpy(rowptr).to(DEV), n, 16)
    plan = cabi.ForwardPlan(tcb, n, q.to(DEV), k.to(DEV), v.to(DEV), 8.0)
    assert plan.ws_bytes > 256, "the problem must use the scheduled mode (unit list in scratch)"
    plan.launch()
    plan.status()  # no error
    good = plan.out.clone()
    m = ao.compare(good.cpu(), ao.edge_attention(rowptr, colidx, q, k, v, 8.0))
    assert m["max_abs"] <= ao.MAX_ABS_TOL and m["mean_rel"] <= ao.MEAN_REL_TOL, m
    try:
        lib.f3s_debug_set_unit_list_limit(1)  # three heavy windows want several chunks each: one slot is too few
        plan.planned = False  # the schedule is made again under the cap
        plan.out.fill_(float("nan"))
        plan.launch()
        with pytest.raises(cabi.F3SError) as e:
            plan.status()
        assert e.value.status == cabi.ERR_DEVICE and "overflow" in str(e.value)
        # the non-blocking form: raw word into host memory, decoded after a synchronise
        word = torch.zeros(1, dtype=torch.int32).pin_memory()
        stream = C.c_void_p(torch.cuda.current_stream(torch.device(DEV)).cuda_stream)
        cabi.check(lib.f3s_forward_status(C.c_void_p(plan.ws.data_ptr()), C.c_void_p(word.data_ptr()), stream))
        torch.cuda.synchronize()
        assert int(word[0]) != 0 and lib.f3s_status_word_to_code(int(word[0])) == cabi.ERR_DEVICE
        # every row is either right (its window was scheduled) or untouched (its window was dropped); the
        # three hub windows are certainly among the dropped ones
        untouched = torch.isnan(plan.out)
        assert bool(((plan.out == good) | untouched).all())
        for a in (0, 1024, 4096):
            assert bool(untouched[a:a + 16].all())
    finally:
        lib.f3s_debug_set_unit_list_limit(0)
    plan.planned = False
    plan.launch()
    plan.status()  # scheduling again clears the word
    assert torch.equal(plan.out, good)


def test_status_after_one_launch_mode_is_ok_even_on_dirty_scratch():
    from fused3s_b200 import cabi

    g = graphs.make_config(1)
    q, k, v = graphs.make_features(g)
    tcb = cabi.preprocess(torch.from_numpy(g.colidx).to(DEV), torch.from_numpy(g.rowptr).to(DEV), g.num_nodes, 16)
    plan = cabi.ForwardPlan(tcb, g.num_nodes, q.to(DEV), k.to(DEV), v.to(DEV), 8.0)
    plan.ws.fill_(0xFF)  # stale garbage where the status word lives
    plan.launch()
    plan.status()


def test_timed_torch_op_checks_the_status_word():
    from fused3s_b200 import cabi, import_f3s

    F3S = import_f3s()
    n, rowptr, colidx, q, k, v = _heavy_problem()
    tcb = cabi.preprocess(torch.from_numpy(colidx).to(DEV), torch.from_numpy(rowptr).to(DEV), n, 16)
    args = (tcb["rowWindowOffset"], tcb["sortedRowWindows"], tcb["sparseAToXidx"], tcb["tcbBitMap"], n, q.to(DEV),
            k.to(DEV), v.to(DEV), 8.0, 8)
    F3S.f3s_1tb1rw_scheduled_permuteV_scaleQK(*args)
    try:
        cabi.lib().f3s_debug_set_unit_list_limit(1)
        with pytest.raises(RuntimeError, match="overflow"):
            F3S.f3s_1tb1rw_scheduled_permuteV_scaleQK(*args)
    finally:
        cabi.lib().f3s_debug_set_unit_list_limit(0)
    F3S.f3s_1tb1rw_scheduled_permuteV_scaleQK(*args)


def test_validate_plan_accepts_preprocessed_plans_and_names_the_first_bad_index():
    from fused3s_b200 import cabi

    g = graphs.make_config(2)
    n = g.num_nodes
    tcb = cabi.preprocess(torch.from_numpy(g.colidx).to(DEV), torch.from_numpy(g.rowptr).to(DEV), n, 16)
    cabi.validate_plan(tcb, n)
    with pytest.raises(cabi.F3SError) as e:  # K/V with fewer rows than the largest column id
        cabi.validate_plan(tcb, n // 2)
    assert e.value.status == cabi.ERR_INVALID_ARG and "column id" in str(e.value)
    bad = dict(tcb)
    bad["sparseAToXidx"] = tcb["sparseAToXidx"].clone()
    bad["sparseAToXidx"][1234] = -7
    with pytest.raises(cabi.F3SError) as e:
        cabi.validate_plan(bad, n)
    assert "position 1234" in str(e.value) and "-7" in str(e.value)
    bad = dict(tcb)
    bad["rowWindowOffset"] = tcb["rowWindowOffset"].clone()
    bad["rowWindowOffset"][-1] += 3  # offsets that run past the TCB arrays (for instance a bad concatenation)
    with pytest.raises(cabi.F3SError, match="differs from n_tcb"):
        cabi.validate_plan(bad, n)
    bad = dict(tcb)
    bad["sortedRowWindows"] = tcb["sortedRowWindows"].clone()
    bad["sortedRowWindows"][5] = bad["rowWindowOffset"].numel() + 10
    with pytest.raises(cabi.F3SError, match="window id"):
        cabi.validate_plan(bad, n)
    cabi.validate_plan(bad, n, scheduled=False)  # natural order does not read the window order


def test_preprocess_refuses_block_partition_that_was_not_zeroed():
    from fused3s_b200 import cabi

    n = 64
    rowptr = np.zeros(n + 1, np.int32)
    rowptr[1:17] = np.arange(1, 17)  # window 0 has edges, windows 1-3 have none
    rowptr[17:] = 16
    colidx = np.arange(16, dtype=np.int32)
    dirty = torch.full((4,), 3, dtype=torch.int32, device=DEV)
    with pytest.raises(cabi.F3SError) as e:
        cabi.preprocess(torch.from_numpy(colidx).to(DEV), torch.from_numpy(rowptr).to(DEV), n, 16, block_partition=dirty)
    assert e.value.status == cabi.ERR_INVALID_ARG and "not zeroed" in str(e.value)
    cabi.preprocess(torch.from_numpy(colidx).to(DEV), torch.from_numpy(rowptr).to(DEV), n, 16)
