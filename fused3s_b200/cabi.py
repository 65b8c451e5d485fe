"""ctypes view of the C ABI declared in ``include/f3s_b200.h``.

The shared library is loaded from this directory (``libf3s_b200.so``, built in-tree by
``fused3s_b200.build``).  There is no fallback: if the library is missing, loading raises.
The helpers below take torch tensors only to obtain device pointers, the current stream
and scratch allocations; all computation happens inside the library.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "libf3s_b200.so"
_lib = None

OK = 0
ERR_INVALID_ARG = -1
ERR_UNSUPPORTED = -2
ERR_CUDA = -3
ERR_WORKSPACE = -4
ERR_DEVICE = -5

EXPORTS = (
    "f3s_version",
    "f3s_last_error_string",
    "f3s_kernel_launch_count",
    "f3s_preprocess_workspace_bytes",
    "f3s_preprocess_count",
    "f3s_preprocess_count_rect",
    "f3s_preprocess_fill",
    "f3s_forward_workspace_bytes",
    "f3s_forward",
    "f3s_forward_f16out",
    "f3s_forward_static",
    "f3s_forward_traced",
    "f3s_forward_lse",
    "f3s_forward_plan",
    "f3s_forward_planned",
    "f3s_forward_phased_workspace_bytes",
    "f3s_forward_phased_plan",
    "f3s_forward_phase",
    "f3s_set_max_ctas",
    "f3s_set_canonical_chunk_tiles",
    "f3s_sddmm_umma",
    "f3s_forward_status",
    "f3s_forward_static_status",
    "f3s_status_word_to_code",
    "f3s_debug_set_unit_list_limit",
    "f3s_validate_plan",
    "f3s_backward_workspace_bytes",
    "f3s_backward",
    "f3s_backward_prepare",
    "f3s_backward_stage_workspace_bytes",
    "f3s_backward_dq",
    "f3s_backward_dkv",
    "f3s_partition_row_windows",
    "f3s_probe_gather_rows",
)


class F3SError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"f3s_b200 status {status}: {message}")
        self.status = status


def lib() -> C.CDLL:
    """Load (once) and return the C-ABI library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise ImportError(
                f"{_LIB_PATH} is missing: build it with `python -m fused3s_b200.build` "
                "(there is no CPU or PyTorch fallback for this path)"
            )
        l = C.CDLL(str(_LIB_PATH))
        vp, i32, i64, sz, f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_size_t, C.c_float
        l.f3s_version.restype = C.c_int
        l.f3s_last_error_string.restype = C.c_char_p
        l.f3s_kernel_launch_count.restype = C.c_uint64
        l.f3s_preprocess_workspace_bytes.restype = sz
        l.f3s_preprocess_workspace_bytes.argtypes = [i64, i64, C.c_int]
        l.f3s_preprocess_count.restype = C.c_int
        l.f3s_preprocess_count.argtypes = [vp, vp, i32, i64, i32, i32, vp, vp, vp, vp, vp, sz,
                                           C.POINTER(i32), C.POINTER(i32), vp]
        l.f3s_preprocess_count_rect.restype = C.c_int
        l.f3s_preprocess_count_rect.argtypes = [vp, vp, i32, i32, i64, i32, i32, vp, vp, vp, vp, vp, sz,
                                                C.POINTER(i32), C.POINTER(i32), vp]
        l.f3s_preprocess_fill.restype = C.c_int
        l.f3s_preprocess_fill.argtypes = [vp, vp, i32, i64, i32, i32, vp, vp, vp, i32, vp, vp, vp, vp, vp, vp,
                                          vp, sz, vp]
        l.f3s_forward_workspace_bytes.restype = sz
        l.f3s_forward_workspace_bytes.argtypes = [i32, i64, i32, i32, i32]
        l.f3s_forward.restype = C.c_int
        l.f3s_forward.argtypes = [vp, vp, vp, vp, i32, i32, i64, i32, i32, i32, i64, vp, vp, vp, f32, i32, vp, vp,
                                  vp, sz, vp]
        l.f3s_forward_static.restype = C.c_int
        l.f3s_forward_static.argtypes = [vp, vp, vp, vp, i32, i32, i64, i32, i32, i32, i64, vp, vp, vp, f32, i32, vp,
                                         vp]
        l.f3s_forward_f16out.restype = C.c_int
        l.f3s_forward_f16out.argtypes = [vp, vp, vp, vp, i32, i32, i64, i32, i32, i32, i64, vp, vp, vp, f32, i32, vp,
                                         vp, sz, vp]
        l.f3s_forward_traced.restype = C.c_int
        l.f3s_forward_traced.argtypes = [vp, vp, vp, vp, i32, i32, i64, i32, i32, i32, i64, vp, vp, vp, f32, i32, vp,
                                         vp, sz, vp, vp]
        l.f3s_forward_lse.restype = C.c_int
        l.f3s_forward_lse.argtypes = [vp, vp, vp, vp, i32, i32, i64, i32, i32, i32, i64, vp, vp, vp, f32, vp, vp, vp,
                                      sz, vp]
        l.f3s_forward_plan.restype = C.c_int
        l.f3s_forward_plan.argtypes = [vp, vp, i32, i32, i64, i32, i32, i32, vp, sz, vp]
        l.f3s_forward_planned.restype = C.c_int
        l.f3s_forward_planned.argtypes = [vp, vp, vp, vp, i32, i32, i64, i32, i32, i32, i64, vp, i64, vp, vp, f32, i32,
                                          vp, i32, vp, sz, vp]
        l.f3s_forward_phased_workspace_bytes.restype = sz
        l.f3s_forward_phased_workspace_bytes.argtypes = [i32, i64, i32, i32, i32]
        l.f3s_forward_phased_plan.restype = C.c_int
        l.f3s_forward_phased_plan.argtypes = [vp, vp, vp, i32, i32, i64, i32, i32, i32, vp, sz, vp]
        l.f3s_forward_phase.restype = C.c_int
        l.f3s_forward_phase.argtypes = [i32, vp, vp, vp, vp, vp, i32, i32, i32, i64, i32, i32, i32, i64, vp, i64, vp,
                                        vp, f32, vp, vp, sz, vp]
        l.f3s_sddmm_umma.restype = C.c_int
        l.f3s_sddmm_umma.argtypes = [vp, vp, vp, i32, i32, i64, i32, i32, i64, vp, i64, vp, vp, vp, sz, vp]
        l.f3s_set_canonical_chunk_tiles.restype = None
        l.f3s_set_canonical_chunk_tiles.argtypes = [i32]
        l.f3s_set_max_ctas.restype = C.c_int32
        l.f3s_set_max_ctas.argtypes = [i32]
        l.f3s_forward_status.restype = C.c_int
        l.f3s_forward_status.argtypes = [vp, vp, vp]
        l.f3s_forward_static_status.restype = C.c_int
        l.f3s_forward_static_status.argtypes = [vp, vp]
        l.f3s_status_word_to_code.restype = C.c_int
        l.f3s_status_word_to_code.argtypes = [i32]
        l.f3s_debug_set_unit_list_limit.restype = None
        l.f3s_debug_set_unit_list_limit.argtypes = [i32]
        l.f3s_validate_plan.restype = C.c_int
        l.f3s_validate_plan.argtypes = [vp, vp, vp, i32, i64, i32, i32, vp, sz, vp]
        l.f3s_backward_workspace_bytes.restype = sz
        l.f3s_backward_workspace_bytes.argtypes = [i32, i64, i64, i32, i32, i32]
        l.f3s_backward.restype = C.c_int
        l.f3s_backward.argtypes = [vp, vp, vp, vp, i64, vp, vp, vp, vp, i64, i32, i32, i32, i32, i32, i64, vp, vp, vp,
                                   f32, vp, vp, vp, vp, vp, vp, i32, vp, sz, vp]
        l.f3s_backward_prepare.restype = C.c_int
        l.f3s_backward_prepare.argtypes = [vp, vp, vp, i32, i32, i32, vp, vp, vp]
        l.f3s_backward_stage_workspace_bytes.restype = sz
        l.f3s_backward_stage_workspace_bytes.argtypes = [i64, i32, i32, i32, i32]
        l.f3s_backward_dq.restype = C.c_int
        l.f3s_backward_dq.argtypes = [vp, vp, vp, vp, i64, i32, i32, i32, i32, i32, i64, vp, i64, vp, vp, f32, vp, vp,
                                      vp, i32, vp, sz, vp]
        l.f3s_backward_dkv.restype = C.c_int
        l.f3s_backward_dkv.argtypes = [vp, vp, vp, vp, i64, i32, i32, i32, i32, i32, i64, vp, vp, i64, vp, vp, vp, f32,
                                       vp, vp, i32, vp, sz, vp]
        l.f3s_probe_gather_rows.restype = C.c_int
        l.f3s_probe_gather_rows.argtypes = [vp, i64, vp, i64, vp, vp]
        l.f3s_partition_row_windows.restype = C.c_int
        l.f3s_partition_row_windows.argtypes = [vp, i32, i32, vp]
        _lib = l
    return _lib


def check(status: int) -> None:
    if status != OK:
        raise F3SError(status, lib().f3s_last_error_string().decode())


def _ptr(t):
    return C.c_void_p(0 if t is None else t.data_ptr())


def _stream(device):
    import torch

    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def preprocess(colidx, rowptr, num_nodes: int, block_w: int = 16, block_h: int = 16,
               block_partition=None, edge_to_column=None, edge_to_row=None, num_cols: int | None = None) -> dict:
    """CSR -> TC-block arrays through ``f3s_preprocess_count`` + ``f3s_preprocess_fill``.

    ``colidx`` / ``rowptr`` are int32 CUDA tensors.  Returns a dict with the names of the
    reference's tuple (src/F3S.cpp:83-86) plus the three in-place outputs."""
    import torch

    l = lib()
    dev = colidx.device
    nnz = int(colidx.numel())
    n_rw = (num_nodes + 15) // 16
    i32 = dict(dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        bp = torch.zeros(n_rw, **i32) if block_partition is None else block_partition
        e2c = torch.empty(nnz, **i32) if edge_to_column is None else edge_to_column
        e2r = torch.empty(nnz, **i32) if edge_to_row is None else edge_to_row
        rwo = torch.empty(n_rw + 1, **i32)
        ws_bytes = l.f3s_preprocess_workspace_bytes(num_nodes, nnz, block_w)
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
        n_tcb, max_tcb = C.c_int32(0), C.c_int32(0)
        if num_cols is None:
            check(l.f3s_preprocess_count(_ptr(colidx), _ptr(rowptr), num_nodes, nnz, block_h, block_w, _ptr(bp),
                                         _ptr(e2c), _ptr(e2r), _ptr(rwo), _ptr(ws), ws_bytes, C.byref(n_tcb),
                                         C.byref(max_tcb), _stream(dev)))
        else:  # rows of a shard, columns of the whole graph
            check(l.f3s_preprocess_count_rect(_ptr(colidx), _ptr(rowptr), num_nodes, num_cols, nnz, block_h, block_w,
                                              _ptr(bp), _ptr(e2c), _ptr(e2r), _ptr(rwo), _ptr(ws), ws_bytes,
                                              C.byref(n_tcb), C.byref(max_tcb), _stream(dev)))
        nt = n_tcb.value
        wpt = 16 * block_w // 64
        sorted_rw = torch.empty(n_rw, **i32)
        rowid = torch.empty(nt, **i32)
        tile_id = torch.empty(nnz, dtype=torch.uint8, device=dev)
        tcb_off = torch.empty(nt + 1, **i32)
        atox = torch.empty(nt * block_w, **i32)
        bitmap = torch.empty(nt * wpt, dtype=torch.uint64, device=dev)
        check(l.f3s_preprocess_fill(_ptr(colidx), _ptr(rowptr), num_nodes, nnz, block_h, block_w, _ptr(e2c),
                                    _ptr(e2r), _ptr(rwo), nt, _ptr(sorted_rw), _ptr(rowid), _ptr(tile_id),
                                    _ptr(tcb_off), _ptr(atox), _ptr(bitmap), _ptr(ws), ws_bytes, _stream(dev)))
    return {
        "rowWindowOffset": rwo, "sortedRowWindows": sorted_rw, "tcblock_rowid": rowid, "tcblocktile_id": tile_id,
        "tcblock_offset": tcb_off, "sparseAToXidx": atox, "tcbBitMap": bitmap, "nTCB": nt,
        "maxTCBPerWindow": max_tcb.value, "blockPartition": bp, "edgeToColumn": e2c, "edgeToRow": e2r,
        "block_w": block_w,
    }


class ForwardPlan:
    """Device pointers and scratch of one forward problem, so repeated launches (benchmark
    loops, CUDA-graph capture) cost one C call each."""

    def __init__(self, tcb: dict, num_nodes: int, q, k, v, scale_divisor: float = 1.0, apply_softmax: bool = True,
                 scheduled: bool = True, out=None, sddmm_out=None, out_dtype=None):
        import torch

        self.l = lib()
        self.dev = q.device
        self.heads = q.shape[1] if q.dim() == 3 else 1
        self.dim = q.shape[-1]
        self.num_nodes = num_nodes
        self.tcb = tcb
        self.q, self.k, self.v = q, k, v
        # Row strides in elements.  Q, K and V may be views into larger buffers (the three slices of a fused
        # QKV projection output, or K and V rows interleaved in one gathered buffer) as long as each row's
        # heads*d values are contiguous; K and V share one row stride, Q has its own.
        def row_stride(t):
            return int(t.stride(0)) if t.shape[0] > 1 else self.heads * self.dim

        self.ld, self.ld_kv = row_stride(q), row_stride(k)
        for name, t, ld in (("q", q, self.ld), ("k", k, self.ld_kv), ("v", v, self.ld_kv)):
            inner_ok = t.stride(-1) == 1 and (t.dim() == 2 or t.stride(1) == self.dim)
            row_ok = t.shape[0] <= 1 or t.stride(0) == ld
            if not (inner_ok and row_ok and ld >= self.heads * self.dim):
                raise F3SError(ERR_INVALID_ARG, f"{name}: rows must be contiguous; k and v must share one row stride")
        self.block_w = tcb["block_w"]
        self.n_rw = tcb["rowWindowOffset"].numel() - 1
        self.n_tcb = tcb["sparseAToXidx"].numel() // self.block_w
        self.scale_divisor = float(scale_divisor)
        self.apply_softmax = 1 if apply_softmax else 0
        self.sorted = tcb["sortedRowWindows"] if scheduled else None
        shape = (num_nodes, self.heads, self.dim) if q.dim() == 3 else (num_nodes, self.dim)
        if out is None:
            out = torch.empty(shape, dtype=torch.float32 if out_dtype is None else out_dtype, device=self.dev)
        if out.dtype not in (torch.float32, torch.float16):
            raise F3SError(ERR_UNSUPPORTED, f"output dtype {out.dtype} (fp32 or fp16)")
        self.out = out
        self.out_half = out.dtype == torch.float16
        self.sddmm = sddmm_out
        self.ws_bytes = self.l.f3s_forward_workspace_bytes(self.n_rw, self.n_tcb, self.block_w, self.heads, self.dim)
        if self.ws_bytes == 0:
            raise F3SError(ERR_UNSUPPORTED, f"unsupported head_dim {self.dim} / block_w {self.block_w}")
        self.ws = torch.empty(self.ws_bytes, dtype=torch.uint8, device=self.dev)
        self.planned = False  # the schedule is written into the scratch by the first launch

    def launch(self, stream=None) -> None:
        s = _stream(self.dev) if stream is None else C.c_void_p(stream)
        t = self.tcb
        if self.sddmm is None:
            # schedule once (first launch, same stream), then one kernel per call
            if not self.planned:
                check(self.l.f3s_forward_plan(_ptr(t["rowWindowOffset"]), _ptr(self.sorted), self.num_nodes, self.n_rw,
                                              self.n_tcb, self.block_w, self.heads, self.dim, _ptr(self.ws),
                                              self.ws_bytes, s))
                self.planned = True
            check(self.l.f3s_forward_planned(_ptr(t["rowWindowOffset"]), _ptr(self.sorted), _ptr(t["sparseAToXidx"]),
                                             _ptr(t["tcbBitMap"]), self.num_nodes, self.n_rw, self.n_tcb,
                                             self.block_w, self.heads, self.dim, self.ld, _ptr(self.q), self.ld_kv,
                                             _ptr(self.k), _ptr(self.v), self.scale_divisor, self.apply_softmax,
                                             _ptr(self.out), 1 if self.out_half else 0, _ptr(self.ws), self.ws_bytes,
                                             s))
            return
        if self.ld_kv != self.ld:
            raise F3SError(ERR_INVALID_ARG, "the score dump needs q, k and v with one common row stride")
        if self.out_half:  # fp16 output entry point (no score dump)
            check(self.l.f3s_forward_f16out(_ptr(t["rowWindowOffset"]), _ptr(self.sorted), _ptr(t["sparseAToXidx"]),
                                            _ptr(t["tcbBitMap"]), self.num_nodes, self.n_rw, self.n_tcb, self.block_w,
                                            self.heads, self.dim, self.ld, _ptr(self.q), _ptr(self.k),
                                            _ptr(self.v), self.scale_divisor, self.apply_softmax, _ptr(self.out),
                                            _ptr(self.ws), self.ws_bytes, s))
            return
        check(self.l.f3s_forward(_ptr(t["rowWindowOffset"]), _ptr(self.sorted), _ptr(t["sparseAToXidx"]),
                                 _ptr(t["tcbBitMap"]), self.num_nodes, self.n_rw, self.n_tcb, self.block_w,
                                 self.heads, self.dim, self.ld, _ptr(self.q), _ptr(self.k),
                                 _ptr(self.v), self.scale_divisor, self.apply_softmax, _ptr(self.out),
                                 _ptr(self.sddmm), _ptr(self.ws), self.ws_bytes, s))


    def status(self, stream=None) -> None:
        """Blocks until the plan's stream has drained and raises ``F3SError`` (``ERR_DEVICE``) if a
        kernel of the last launch reported that it could not finish (``f3s_forward_status``)."""
        s = _stream(self.dev) if stream is None else C.c_void_p(stream)
        try:
            check(self.l.f3s_forward_status(_ptr(self.ws), None, s))
        except F3SError:
            self.planned = False  # a failed launch may leave counters behind: schedule again before the next one
            raise


def phase_split_array(tcb: dict, col_split: int):
    """For every row window the index of its first TC block whose first column id is >= ``col_split``
    (``rowWindowOffset[w+1]`` if none): the ``phase_split`` argument of the two-phase entry points.
    Integer bookkeeping on the plan's device, once per graph."""
    import torch

    bw = tcb["block_w"]
    rwo = tcb["rowWindowOffset"].long()
    first = tcb["sparseAToXidx"][::bw]  # a block's first slot is never padding
    low = torch.zeros(first.numel() + 1, dtype=torch.int64, device=first.device)
    low[1:] = torch.cumsum((first < col_split).to(torch.int64), 0)
    # inside a window the blocks' first columns ascend, so the blocks below the split are a prefix
    return (rwo[:-1] + (low[rwo[1:]] - low[rwo[:-1]])).to(torch.int32)


class PhasedForwardPlan:
    """Two-phase forward (``f3s_forward_phase``) of one problem: ``launch_phase(1)`` works on the columns
    with id >= ``col_split`` and may run before the other K / V rows have arrived, ``launch_phase(2)`` does
    the rest and writes ``out``.  head_dim 64, softmax always."""

    def __init__(self, tcb: dict, num_nodes: int, q, k, v, scale_divisor: float, col_split: int, scheduled: bool = True,
                 out=None):
        import torch

        self.l = lib()
        self.dev = q.device
        self.heads = q.shape[1] if q.dim() == 3 else 1
        self.dim = q.shape[-1]
        self.num_nodes, self.tcb, self.q, self.k, self.v = num_nodes, tcb, q, k, v
        self.ld = _ld(q, self.heads, self.dim)
        self.ld_kv = _ld(k, self.heads, self.dim)
        if _ld(v, self.heads, self.dim) != self.ld_kv:
            raise F3SError(ERR_INVALID_ARG, "k and v must share one row stride")
        self.block_w = tcb["block_w"]
        self.n_rw = tcb["rowWindowOffset"].numel() - 1
        self.n_tcb = tcb["sparseAToXidx"].numel() // self.block_w
        self.scale_divisor = float(scale_divisor)
        self.col_split = int(col_split)
        self.sorted = tcb["sortedRowWindows"] if scheduled else None
        with torch.cuda.device(self.dev):
            self.split = phase_split_array(tcb, self.col_split)
            shape = (num_nodes,) + tuple(q.shape[1:])
            self.out = torch.empty(shape, dtype=torch.float32, device=self.dev) if out is None else out
            self.ws_bytes = self.l.f3s_forward_phased_workspace_bytes(self.n_rw, self.n_tcb, self.block_w, self.heads,
                                                                      self.dim)
            if self.ws_bytes == 0:
                raise F3SError(ERR_UNSUPPORTED, f"two-phase calls need head_dim 64, got {self.dim}")
            self.ws = torch.empty(self.ws_bytes, dtype=torch.uint8, device=self.dev)
            check(self.l.f3s_forward_phased_plan(_ptr(tcb["rowWindowOffset"]), _ptr(self.sorted), _ptr(self.split),
                                                 num_nodes, self.n_rw, self.n_tcb, self.block_w, self.heads, self.dim,
                                                 _ptr(self.ws), self.ws_bytes, _stream(self.dev)))

    def launch_phase(self, phase: int, stream=None) -> None:
        s = _stream(self.dev) if stream is None else C.c_void_p(stream)
        t = self.tcb
        check(self.l.f3s_forward_phase(phase, _ptr(t["rowWindowOffset"]), _ptr(self.sorted), _ptr(t["sparseAToXidx"]),
                                       _ptr(t["tcbBitMap"]), _ptr(self.split), self.col_split, self.num_nodes,
                                       self.n_rw, self.n_tcb, self.block_w, self.heads, self.dim, self.ld,
                                       _ptr(self.q), self.ld_kv, _ptr(self.k), _ptr(self.v), self.scale_divisor,
                                       _ptr(self.out), _ptr(self.ws), self.ws_bytes, s))


def window_tcb_counts(colidx, rowptr, num_nodes: int, block_w: int = 16):
    """TC blocks per row window (int32 device tensor) without building the plan: the counting half of the
    preprocessing (``f3s_preprocess_count``).  What a TCB-balanced partition of the windows is cut from."""
    import torch

    l = lib()
    dev = colidx.device
    nnz = int(colidx.numel())
    n_rw = (num_nodes + 15) // 16
    with torch.cuda.device(dev):
        bp = torch.zeros(n_rw, dtype=torch.int32, device=dev)
        e2c = torch.empty(nnz, dtype=torch.int32, device=dev)
        e2r = torch.empty(nnz, dtype=torch.int32, device=dev)
        rwo = torch.empty(n_rw + 1, dtype=torch.int32, device=dev)
        ws_bytes = l.f3s_preprocess_workspace_bytes(num_nodes, nnz, block_w)
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
        n_tcb, max_tcb = C.c_int32(0), C.c_int32(0)
        check(l.f3s_preprocess_count(_ptr(colidx), _ptr(rowptr), num_nodes, nnz, 16, block_w, _ptr(bp), _ptr(e2c),
                                     _ptr(e2r), _ptr(rwo), _ptr(ws), ws_bytes, C.byref(n_tcb), C.byref(max_tcb),
                                     _stream(dev)))
    return bp


def sddmm_umma(tcb: dict, num_nodes: int, q, k, out=None):
    """``f3s_sddmm_umma``: masked, unscaled score tiles ``[nTCB*block_w/8 * 128]`` fp32 computed with
    tcgen05.mma / tensor memory (one head, head_dim 64).  Returns the tensor; raises if the kernel reported
    a failed wait."""
    import torch

    bw = tcb["block_w"]
    n_rw = tcb["rowWindowOffset"].numel() - 1
    n_tcb = tcb["sparseAToXidx"].numel() // bw
    dev = q.device
    if q.dim() != 2 or k.dim() != 2:
        raise F3SError(ERR_INVALID_ARG, "one head: q and k must be [N, 64]")
    with torch.cuda.device(dev):
        if out is None:
            out = torch.empty(n_tcb * 16 * bw, dtype=torch.float32, device=dev)
        ws = torch.empty(64, dtype=torch.uint8, device=dev)
        check(lib().f3s_sddmm_umma(_ptr(tcb["rowWindowOffset"]), _ptr(tcb["sparseAToXidx"]), _ptr(tcb["tcbBitMap"]),
                                   num_nodes, n_rw, n_tcb, bw, q.shape[-1], _ld(q, 1, q.shape[-1]), _ptr(q),
                                   _ld(k, 1, k.shape[-1]), _ptr(k), _ptr(out), _ptr(ws), 64, _stream(dev)))
        check(lib().f3s_forward_status(_ptr(ws), None, _stream(dev)))
    return out


def validate_plan(tcb: dict, num_kv_rows: int, scheduled: bool = True) -> None:
    """``f3s_validate_plan``: raises ``F3SError`` (``ERR_INVALID_ARG``) if the plan holds an index the
    kernels would dereference out of range for K / V tensors of ``num_kv_rows`` rows.  For plans that
    were read from a file or assembled from parts; blocks until the answer is known."""
    import torch

    bw = tcb["block_w"]
    rwo = tcb["rowWindowOffset"]
    dev = rwo.device
    with torch.cuda.device(dev):
        scratch = torch.empty(16, dtype=torch.uint8, device=dev)
        check(lib().f3s_validate_plan(_ptr(rwo), _ptr(tcb["sortedRowWindows"] if scheduled else None),
                                      _ptr(tcb["sparseAToXidx"]), rwo.numel() - 1,
                                      tcb["sparseAToXidx"].numel() // bw, bw, int(num_kv_rows), _ptr(scratch), 16,
                                      _stream(dev)))


def forward(tcb: dict, num_nodes: int, q, k, v, scale_divisor: float = 1.0, apply_softmax: bool = True,
            scheduled: bool = True, sddmm_out=None, out_dtype=None):
    """One fused forward call through ``f3s_forward`` (or ``f3s_forward_f16out`` when
    ``out_dtype=torch.float16``); returns the output tensor."""
    import torch

    with torch.cuda.device(q.device):
        plan = ForwardPlan(tcb, num_nodes, q, k, v, scale_divisor, apply_softmax, scheduled, sddmm_out=sddmm_out,
                           out_dtype=out_dtype)
        plan.launch()
    return plan.out


def _row_stride(q, k, v):
    heads = q.shape[1] if q.dim() == 3 else 1
    dim = q.shape[-1]
    ld = int(q.stride(0)) if q.shape[0] > 1 else heads * dim
    for name, t in (("q", q), ("k", k), ("v", v)):
        inner_ok = t.stride(-1) == 1 and (t.dim() == 2 or t.stride(1) == dim)
        row_ok = t.shape[0] <= 1 or t.stride(0) == ld
        if not (inner_ok and row_ok and ld >= heads * dim):
            raise F3SError(ERR_INVALID_ARG, f"{name}: rows must be contiguous and share one row stride")
    return heads, dim, ld


def transpose_csr(rowptr, colidx, num_nodes: int):
    """CSR of A^T on the device of ``colidx`` (int32 tensors in and out): row j of the result lists,
    ascending, the rows i of A that hold column j.  Repeated entries of A are kept once."""
    import torch

    dev = colidx.device
    deg = (rowptr[1:] - rowptr[:-1]).long()
    rows = torch.repeat_interleave(torch.arange(num_nodes, device=dev), deg)
    keys = torch.unique(colidx.long() * num_nodes + rows)  # sorted
    cols_t = (keys % num_nodes).to(torch.int32)
    counts = torch.bincount(keys // num_nodes, minlength=num_nodes)
    rowptr_t = torch.zeros(num_nodes + 1, dtype=torch.int64, device=dev)
    rowptr_t[1:] = torch.cumsum(counts, 0)
    return rowptr_t.to(torch.int32), cols_t


def forward_lse(tcb: dict, num_nodes: int, q, k, v, scale_divisor: float = 1.0, scheduled: bool = True):
    """``f3s_forward_lse``: softmax forward that also returns the per-row log-sum-exp (log2 domain,
    shape [N, H]) a later ``backward`` needs.  Returns (out fp32, lse)."""
    import torch

    l = lib()
    heads, dim, ld = _row_stride(q, k, v)
    bw = tcb["block_w"]
    n_rw = tcb["rowWindowOffset"].numel() - 1
    n_tcb = tcb["sparseAToXidx"].numel() // bw
    dev = q.device
    with torch.cuda.device(dev):
        out = torch.empty(q.shape, dtype=torch.float32, device=dev)
        lse = torch.empty((num_nodes, heads), dtype=torch.float32, device=dev)
        ws_bytes = l.f3s_forward_workspace_bytes(n_rw, n_tcb, bw, heads, dim)
        if ws_bytes == 0:
            raise F3SError(ERR_UNSUPPORTED, f"unsupported head_dim {dim} / block_w {bw}")
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        check(l.f3s_forward_lse(_ptr(tcb["rowWindowOffset"]), _ptr(tcb["sortedRowWindows"] if scheduled else None),
                                _ptr(tcb["sparseAToXidx"]), _ptr(tcb["tcbBitMap"]), num_nodes, n_rw, n_tcb, bw, heads,
                                dim, ld, _ptr(q), _ptr(k), _ptr(v), float(scale_divisor), _ptr(out), _ptr(lse),
                                _ptr(ws), ws_bytes, _stream(dev)))
    return out, lse


def backward(tcb: dict, tcb_t: dict, num_nodes: int, q, k, v, out, lse, d_out, scale_divisor: float = 1.0,
             grad_dtype=None):
    """``f3s_backward``: (dq, dk, dv), each [N, H, d] (or [N, d]) contiguous, fp32 unless
    ``grad_dtype=torch.float16``.  ``tcb_t`` is the preprocess result of the transposed graph
    (``transpose_csr`` + ``preprocess``); ``out``/``lse`` come from ``forward_lse``; ``d_out`` is fp32."""
    import torch

    l = lib()
    heads, dim, ld = _row_stride(q, k, v)
    bw = tcb["block_w"]
    if tcb_t["block_w"] != bw:
        raise F3SError(ERR_INVALID_ARG, "the two plans must use the same block_w")
    n_rw = tcb["rowWindowOffset"].numel() - 1
    n_tcb = tcb["sparseAToXidx"].numel() // bw
    n_tcb_t = tcb_t["sparseAToXidx"].numel() // bw
    if k.shape[0] != num_nodes or v.shape[0] != num_nodes or q.shape[0] != num_nodes:
        raise F3SError(ERR_INVALID_ARG, "backward needs a square graph: q, k, v with num_nodes rows")
    dev = q.device
    gd = torch.float32 if grad_dtype is None else grad_dtype
    if gd not in (torch.float32, torch.float16):
        raise F3SError(ERR_UNSUPPORTED, f"gradient dtype {gd} (fp32 or fp16)")
    with torch.cuda.device(dev):
        out = out.contiguous()
        d_out = d_out.to(torch.float32).contiguous()
        dq = torch.empty(q.shape, dtype=gd, device=dev)
        dk = torch.empty(q.shape, dtype=gd, device=dev)
        dv = torch.empty(q.shape, dtype=gd, device=dev)
        ws_bytes = l.f3s_backward_workspace_bytes(num_nodes, n_tcb, n_tcb_t, bw, heads, dim)
        if ws_bytes == 0 and num_nodes > 0:
            raise F3SError(ERR_UNSUPPORTED, f"unsupported head_dim {dim} / block_w {bw}")
        ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=dev)
        check(l.f3s_backward(_ptr(tcb["rowWindowOffset"]), _ptr(tcb["sortedRowWindows"]), _ptr(tcb["sparseAToXidx"]),
                             _ptr(tcb["tcbBitMap"]), n_tcb, _ptr(tcb_t["rowWindowOffset"]),
                             _ptr(tcb_t["sortedRowWindows"]), _ptr(tcb_t["sparseAToXidx"]), _ptr(tcb_t["tcbBitMap"]),
                             n_tcb_t, num_nodes, n_rw, bw, heads, dim, ld, _ptr(q), _ptr(k), _ptr(v),
                             float(scale_divisor), _ptr(out), _ptr(lse), _ptr(d_out), _ptr(dq), _ptr(dk), _ptr(dv),
                             1 if gd == torch.float16 else 0, _ptr(ws), ws_bytes, _stream(dev)))
    return dq, dk, dv


def _ld(t, heads, dim):
    ld = int(t.stride(0)) if t.shape[0] > 1 else heads * dim
    inner_ok = t.stride(-1) == 1 and (t.dim() == 2 or t.stride(1) == dim)
    if not inner_ok or ld < heads * dim:
        raise F3SError(ERR_INVALID_ARG, "rows must be contiguous")
    return ld


def backward_prepare(out, lse, d_out):
    """``f3s_backward_prepare`` for a block of rows: (fp16 copy of d_out, {lse, delta} pairs [rows, H, 2])."""
    import torch

    rows = out.shape[0]
    heads = out.shape[1] if out.dim() == 3 else 1
    dim = out.shape[-1]
    dev = out.device
    with torch.cuda.device(dev):
        out = out.contiguous()
        d_out = d_out.to(torch.float32).contiguous()
        do_h = torch.empty(out.shape, dtype=torch.float16, device=dev)
        stats = torch.empty((rows, heads, 2), dtype=torch.float32, device=dev)
        check(lib().f3s_backward_prepare(_ptr(out), _ptr(d_out), _ptr(lse), rows, heads, dim, _ptr(do_h), _ptr(stats),
                                         _stream(dev)))
    return do_h, stats


def backward_dq(tcb: dict, num_rows: int, q, k_g, v_g, do_h, stats, scale_divisor: float = 1.0, grad_dtype=None):
    """``f3s_backward_dq``: dq of a block of rows; ``k_g``/``v_g`` are indexed by the plan's column ids."""
    import torch

    l = lib()
    heads = q.shape[1] if q.dim() == 3 else 1
    dim = q.shape[-1]
    bw = tcb["block_w"]
    n_tcb = tcb["sparseAToXidx"].numel() // bw
    dev = q.device
    gd = torch.float32 if grad_dtype is None else grad_dtype
    with torch.cuda.device(dev):
        dq = torch.empty(q.shape, dtype=gd, device=dev)
        ws_bytes = l.f3s_backward_stage_workspace_bytes(n_tcb, bw, heads, dim, 0)
        ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=dev)
        check(l.f3s_backward_dq(_ptr(tcb["rowWindowOffset"]), _ptr(tcb["sortedRowWindows"]),
                                _ptr(tcb["sparseAToXidx"]), _ptr(tcb["tcbBitMap"]), n_tcb, num_rows,
                                tcb["rowWindowOffset"].numel() - 1, bw, heads, dim, _ld(q, heads, dim), _ptr(q),
                                _ld(k_g, heads, dim), _ptr(k_g), _ptr(v_g), float(scale_divisor), _ptr(do_h),
                                _ptr(stats), _ptr(dq), 1 if gd == torch.float16 else 0, _ptr(ws), ws_bytes,
                                _stream(dev)))
    return dq


def backward_dkv(tcb_t: dict, num_rows: int, k, v, q_g, do_h_g, stats_g, scale_divisor: float = 1.0, grad_dtype=None):
    """``f3s_backward_dkv``: dk, dv of a block of key/value rows; ``tcb_t`` is the plan of the transposed
    graph's rows of that block, ``q_g``/``do_h_g``/``stats_g`` are indexed by its column ids."""
    import torch

    l = lib()
    heads = k.shape[1] if k.dim() == 3 else 1
    dim = k.shape[-1]
    bw = tcb_t["block_w"]
    n_tcb = tcb_t["sparseAToXidx"].numel() // bw
    dev = k.device
    gd = torch.float32 if grad_dtype is None else grad_dtype
    with torch.cuda.device(dev):
        dk = torch.empty(k.shape, dtype=gd, device=dev)
        dv = torch.empty(k.shape, dtype=gd, device=dev)
        ws_bytes = l.f3s_backward_stage_workspace_bytes(n_tcb, bw, heads, dim, 1)
        ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=dev)
        check(l.f3s_backward_dkv(_ptr(tcb_t["rowWindowOffset"]), _ptr(tcb_t["sortedRowWindows"]),
                                 _ptr(tcb_t["sparseAToXidx"]), _ptr(tcb_t["tcbBitMap"]), n_tcb, num_rows,
                                 tcb_t["rowWindowOffset"].numel() - 1, bw, heads, dim, _ld(k, heads, dim), _ptr(k),
                                 _ptr(v), _ld(q_g, heads, dim), _ptr(q_g), _ptr(do_h_g), _ptr(stats_g),
                                 float(scale_divisor), _ptr(dk), _ptr(dv), 1 if gd == torch.float16 else 0, _ptr(ws),
                                 ws_bytes, _stream(dev)))
    return dk, dv


STATIC_SCRATCH_BYTES = 32 << 20


def forward_static(tcb: dict, num_nodes: int, q, k, v, out, scale_divisor: float = 1.0, apply_softmax: bool = True,
                   scheduled: bool = True) -> None:
    """``f3s_forward_static``: the fused forward for callers that may not allocate device memory.
    Its scratch is a fixed array inside the library, so nothing is allocated here either: the caller
    passes every buffer, including ``out`` (fp32, contiguous, shape ``(num_nodes,) + q.shape[1:]``, on the
    device of ``q``).  Q, K and V may be strided row views (one shared row stride), as everywhere else.
    Calls on one device must not overlap on the GPU."""
    import torch

    heads, dim, ld = _row_stride(q, k, v)
    bw = tcb["block_w"]
    want_shape = (num_nodes,) + tuple(q.shape[1:])
    if out.dtype != torch.float32 or not out.is_contiguous() or tuple(out.shape) != want_shape or out.device != q.device:
        raise F3SError(ERR_INVALID_ARG, f"out must be a contiguous fp32 tensor of shape {want_shape} on {q.device}")
    with torch.cuda.device(q.device):  # the built-in scratch is looked up on the current device
        check(lib().f3s_forward_static(
            _ptr(tcb["rowWindowOffset"]), _ptr(tcb["sortedRowWindows"] if scheduled else None),
            _ptr(tcb["sparseAToXidx"]), _ptr(tcb["tcbBitMap"]), num_nodes, tcb["rowWindowOffset"].numel() - 1,
            tcb["sparseAToXidx"].numel() // bw, bw, heads, dim, ld, _ptr(q), _ptr(k), _ptr(v), float(scale_divisor),
            1 if apply_softmax else 0, _ptr(out), _stream(q.device)))


def forward_static_status(device) -> None:
    """``f3s_forward_static_status``: blocks, then raises if the last ``forward_static`` call on
    ``device`` reported a device-side failure."""
    import torch

    with torch.cuda.device(device):
        check(lib().f3s_forward_static_status(None, _stream(torch.device(device))))


def gather_rate_gbs(table_bytes: int, device, n_ids: int = 1 << 24, repeats: int = 5) -> float:
    """GB/s at which ``f3s_probe_gather_rows`` gathers 128-byte rows at seeded random ids from a table
    of ``table_bytes`` bytes on ``device`` (best of ``repeats``, CUDA events): the L2 ceiling for the
    fused kernel's gathers when the table fits the cache, the HBM gather ceiling when it does not."""
    import torch

    dev = torch.device(device)
    rows = max(1, int(table_bytes) // 128)
    with torch.cuda.device(dev):
        gen = torch.Generator(device=dev).manual_seed(7)
        table = torch.zeros(rows * 32, dtype=torch.int32, device=dev)
        ids = torch.randint(0, rows, (n_ids,), dtype=torch.int32, device=dev, generator=gen)
        sink = torch.zeros(1, dtype=torch.int32, device=dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        best = float("inf")
        for _ in range(repeats + 1):  # the first call warms the table into the cache
            e0.record()
            check(lib().f3s_probe_gather_rows(_ptr(table), rows, _ptr(ids), n_ids, _ptr(sink), _stream(dev)))
            e1.record()
            e1.synchronize()
            best = min(best, e0.elapsed_time(e1))
    return 128.0 * (n_ids // 32 * 32) / (best * 1e-3) / 1e9


def partition_row_windows(rwo_host, n_parts: int):
    """Host-side cut points of a TCB-balanced contiguous window partition (numpy int32 in/out)."""
    import numpy as np

    rwo_host = np.ascontiguousarray(rwo_host, dtype=np.int32)
    cuts = np.zeros(n_parts + 1, dtype=np.int32)
    check(lib().f3s_partition_row_windows(rwo_host.ctypes.data_as(C.c_void_p), rwo_host.shape[0] - 1, n_parts,
                                          cuts.ctypes.data_as(C.c_void_p)))
    return cuts
