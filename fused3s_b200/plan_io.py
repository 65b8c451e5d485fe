"""Save / load the TC-block arrays of one graph ("plan") so that preprocessing is paid once.

The reference recomputes ``preprocess_gpu`` in every script run and has no stored form of its
tuple (src/F3S.cpp:83-86); its only on-disk graph format is the ``.npz`` edge list written by
``scripts/downloadDataset.py:5-11`` (``src_li``, ``dst_li``, ``num_nodes``).  This module stores the
preprocessed tuple itself as a versioned ``.npz`` bundle and can also read the reference's edge-list
files into CSR.

A plan is the dict returned by ``fused3s_b200.cabi.preprocess`` (tensors on any device) or by the
CPU checker (numpy arrays); loading returns numpy arrays, ``to_device`` turns them into the tensors
the forward entry points take.
"""
from __future__ import annotations

import numpy as np

FORMAT_VERSION = 1
ARRAYS = ("rowWindowOffset", "sortedRowWindows", "tcblock_rowid", "tcblocktile_id", "tcblock_offset",
          "sparseAToXidx", "tcbBitMap")
DTYPES = {"rowWindowOffset": np.int32, "sortedRowWindows": np.int32, "tcblock_rowid": np.int32,
          "tcblocktile_id": np.uint8, "tcblock_offset": np.int32, "sparseAToXidx": np.int32,
          "tcbBitMap": np.uint64}


def _to_numpy(x, name):
    if isinstance(x, np.ndarray):
        a = x
    else:  # torch tensor
        a = x.detach().cpu().numpy()
    if name == "tcbBitMap" and a.dtype != np.uint64:
        a = a.view(np.uint64)
    return np.ascontiguousarray(a, dtype=DTYPES[name])


def check_plan(plan: dict, num_nodes: int, block_w: int) -> None:
    """Structural checks that every consumer relies on; raises ValueError on a malformed plan."""
    rwo = plan["rowWindowOffset"]
    n_rw = (num_nodes + 15) // 16
    n_tcb = int(rwo[-1]) if len(rwo) else 0
    wpt = 16 * block_w // 64
    problems = []
    if len(rwo) != n_rw + 1 or (len(rwo) and rwo[0] != 0) or np.any(np.diff(rwo) < 0):
        problems.append("rowWindowOffset must be a non-decreasing int32[nRW+1] starting at 0")
    if len(plan["sortedRowWindows"]) != n_rw or not np.array_equal(np.sort(plan["sortedRowWindows"]), np.arange(n_rw)):
        problems.append("sortedRowWindows must be a permutation of the row windows")
    if len(plan["sparseAToXidx"]) != n_tcb * block_w:
        problems.append("sparseAToXidx must have nTCB*block_w entries")
    if len(plan["tcbBitMap"]) != n_tcb * wpt:
        problems.append("tcbBitMap must have nTCB*16*block_w/64 words")
    if len(plan["tcblock_rowid"]) != n_tcb or len(plan["tcblock_offset"]) != n_tcb + 1:
        problems.append("tcblock_rowid / tcblock_offset sizes do not match the TCB count")
    if len(plan["sparseAToXidx"]) and (plan["sparseAToXidx"].min() < 0):
        problems.append("negative column id in sparseAToXidx")
    if problems:
        raise ValueError("; ".join(problems))


def save_plan(path, plan: dict, num_nodes: int, block_w: int, num_cols: int | None = None) -> None:
    arrays = {k: _to_numpy(plan[k], k) for k in ARRAYS}
    check_plan(arrays, num_nodes, block_w)
    np.savez_compressed(path, format_version=np.int64(FORMAT_VERSION), num_nodes=np.int64(num_nodes),
                        num_cols=np.int64(num_nodes if num_cols is None else num_cols), block_w=np.int64(block_w),
                        nTCB=np.int64(arrays["rowWindowOffset"][-1] if len(arrays["rowWindowOffset"]) else 0),
                        **arrays)


def load_plan(path) -> dict:
    with np.load(path) as z:
        version = int(z["format_version"])
        if version != FORMAT_VERSION:
            raise ValueError(f"plan format version {version} is not supported (expected {FORMAT_VERSION})")
        plan = {k: np.ascontiguousarray(z[k], dtype=DTYPES[k]) for k in ARRAYS}
        plan["num_nodes"] = int(z["num_nodes"])
        plan["num_cols"] = int(z["num_cols"])
        plan["block_w"] = int(z["block_w"])
        plan["nTCB"] = int(z["nTCB"])
    check_plan(plan, plan["num_nodes"], plan["block_w"])
    if plan["nTCB"] and int(plan["sparseAToXidx"].max()) >= plan["num_cols"]:
        raise ValueError("column id beyond num_cols in sparseAToXidx")
    return plan


def to_device(plan: dict, device, validate: bool = True) -> dict:
    """numpy plan -> dict of torch tensors in the form ``cabi.forward`` / ``cabi.ForwardPlan`` take.
    On a CUDA device the plan is checked once with ``f3s_validate_plan`` (every offset and column id the
    kernels will dereference, against the ``num_cols`` the file records): a file is not a trusted source."""
    import torch

    out = dict(plan)
    for k in ARRAYS:
        a = plan[k]
        t = torch.from_numpy(a.view(np.int64) if k == "tcbBitMap" else a).to(device)
        out[k] = t.view(torch.uint64) if k == "tcbBitMap" else t
    if validate and torch.device(device).type == "cuda":
        from . import cabi

        cabi.validate_plan(out, int(plan.get("num_cols", plan.get("num_nodes", 0))))
    return out


def csr_from_edge_list_npz(path) -> tuple[np.ndarray, np.ndarray, int]:
    """Read the reference's dataset file (``src_li``, ``dst_li``, ``num_nodes``;
    scripts/downloadDataset.py:5-11) into a CSR pattern: row = source, column = destination, columns
    ascending, duplicates merged (the reference's loader goes through scipy ``coo_matrix(...).tocsr()``,
    which sums duplicates into one entry: scripts/baseline_comp/baseline_comp_kernel_only.py:731-741)."""
    with np.load(path) as z:
        src = np.asarray(z["src_li"], dtype=np.int64)
        dst = np.asarray(z["dst_li"], dtype=np.int64)
        n = int(z["num_nodes"])
    keys = np.unique(src * n + dst)
    rows = keys // n
    cols = (keys - rows * n).astype(np.int32)
    rowptr = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(np.bincount(rows, minlength=n), out=rowptr[1:])
    return rowptr.astype(np.int32), cols, n
