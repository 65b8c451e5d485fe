"""CPU tests of the C-ABI library: it loads, exports every function the header declares, and its
host-only entry points behave.  No kernel is launched here."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_functions():
    text = (ROOT / "include" / "f3s_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(f3s_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from fused3s_b200 import cabi

    lib = cabi.lib()
    names = declared_functions()
    assert len(names) >= 9
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/f3s_b200.h but not exported"
    assert set(names) == set(cabi.EXPORTS)
    assert lib.f3s_version() >= 100


def test_partition_row_windows_host_only():
    from fused3s_b200 import cabi

    # 10 windows with TCB (or edge) counts 1..10
    counts = np.arange(1, 11)
    prefix = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    cuts = cabi.partition_row_windows(prefix, 2)
    assert cuts[0] == 0 and cuts[-1] == 10
    left = prefix[cuts[1]]
    assert abs(left - prefix[-1] / 2) <= 5  # within one window of the ideal cut
    cuts = cabi.partition_row_windows(prefix, 4)
    assert list(cuts) == sorted(cuts) and cuts[0] == 0 and cuts[-1] == 10
    # more parts than windows: empty parts are allowed, cuts stay monotone
    cuts = cabi.partition_row_windows(np.array([0, 5, 9], np.int32), 8)
    assert cuts[0] == 0 and cuts[-1] == 2 and np.all(np.diff(cuts) >= 0)
    one = cabi.partition_row_windows(prefix, 1)
    assert list(one) == [0, 10]


def test_argument_errors_are_status_codes_not_exits():
    from fused3s_b200 import cabi

    lib = cabi.lib()
    assert lib.f3s_forward_workspace_bytes(10, 100, 12, 1, 64) == 0  # bad block width
    assert lib.f3s_forward_workspace_bytes(10, 100, 16, 1, 40) == 0  # head dim not a multiple of 16
    assert lib.f3s_forward_workspace_bytes(10, 100, 16, 1, 256) == 0  # head dim above 128
    assert lib.f3s_forward_workspace_bytes(10, 100, 16, 1, 48) > 0
    assert lib.f3s_preprocess_workspace_bytes(-1, 0, 16) == 0
    assert lib.f3s_forward_workspace_bytes(10, 100, 16, 1, 64) > 0
    rc = lib.f3s_partition_row_windows(None, 1, 1, None)
    assert rc == cabi.ERR_INVALID_ARG
    assert b"null" in lib.f3s_last_error_string()
    # forward with a bad block width is rejected before any CUDA call
    rc = lib.f3s_forward(None, None, None, None, 16, 1, 0, 12, 1, 64, 64, None, None, None, 1.0, 1, None, None,
                         None, 0, None)
    assert rc == cabi.ERR_UNSUPPORTED
    with pytest.raises(cabi.F3SError):
        cabi.check(rc)


def test_f3s_extension_module_surface():
    """Same op names as the reference's PYBIND11_MODULE (src/F3S.cpp:298-305)."""
    from fused3s_b200 import import_f3s

    F3S = import_f3s()
    for name in ("preprocess_gpu", "f3s_1tb1tcb", "f3s_1tb1rw", "f3s_1tb1rw_scheduled",
                 "f3s_1tb1rw_scheduled_permuteV", "f3s_1tb1rw_scheduled_permuteV_scaleQK"):
        assert hasattr(F3S, name)
    import torch

    with pytest.raises(RuntimeError):  # CPU tensors are rejected, as the reference's CHECK_CUDA does
        F3S.preprocess_gpu(torch.zeros(1, dtype=torch.int32), torch.zeros(2, dtype=torch.int32), 1, 16, 16,
                           torch.zeros(1, dtype=torch.int32), torch.zeros(1, dtype=torch.int32),
                           torch.zeros(1, dtype=torch.int32))


def test_newer_entry_points_reject_bad_arguments_before_any_cuda_call():
    from fused3s_b200 import cabi

    lib = cabi.lib()
    # two-launch forward: head_dim 64 only, phase 1 or 2
    assert lib.f3s_forward_phased_workspace_bytes(10, 100, 16, 1, 32) == 0
    assert lib.f3s_forward_phased_workspace_bytes(10, 100, 16, 2, 64) > lib.f3s_forward_workspace_bytes(10, 100, 16, 2, 64)
    rc = lib.f3s_forward_phase(3, None, None, None, None, None, 0, 16, 1, 0, 16, 1, 64, 64, None, 64, None, None, 8.0,
                               None, None, 0, None)
    assert rc == cabi.ERR_INVALID_ARG and b"phase" in lib.f3s_last_error_string()
    rc = lib.f3s_forward_phase(1, None, None, None, None, None, 0, 16, 1, 0, 16, 1, 32, 32, None, 32, None, None, 8.0,
                               None, None, 0, None)
    assert rc == cabi.ERR_UNSUPPORTED
    # score stage on tcgen05: head_dim 64 only
    rc = lib.f3s_sddmm_umma(None, None, None, 16, 1, 0, 16, 32, 32, None, 32, None, None, None, 0, None)
    assert rc == cabi.ERR_UNSUPPORTED and b"64" in lib.f3s_last_error_string()
    # plan validation needs its 16 bytes of scratch and real arrays
    rc = lib.f3s_validate_plan(None, None, None, 1, 0, 16, 16, None, 0, None)
    assert rc == cabi.ERR_INVALID_ARG
    # status decoding is pure host code
    assert lib.f3s_status_word_to_code(0) == cabi.OK
    assert lib.f3s_status_word_to_code(1) == cabi.ERR_DEVICE and b"overflow" in lib.f3s_last_error_string()
    assert lib.f3s_status_word_to_code(2) == cabi.ERR_DEVICE and b"wait" in lib.f3s_last_error_string()
    rc = lib.f3s_forward_status(None, None, None)
    assert rc == cabi.ERR_INVALID_ARG
    assert lib.f3s_kernel_launch_count() >= 0
    lib.f3s_set_max_ctas(0)
    lib.f3s_set_canonical_chunk_tiles(0)
    lib.f3s_debug_set_unit_list_limit(0)
