/*
 * f3s_b200 -- C ABI of the B200 (sm_100a) fused sparse-attention path.
 *
 * Plain pointers and sizes only; every pointer is a DEVICE pointer unless its comment says
 * "host".  No entry point allocates or frees device memory (scratch is passed in by the
 * caller, sized by the *_workspace_bytes functions), none terminates the process, and all
 * work is enqueued on the stream passed in.  Every function returns an int status:
 * F3S_OK or a negative F3S_ERR_* code; f3s_last_error_string() gives the text for the
 * calling thread's last failure.
 *
 * Each entry point names the interface of the reference implementation (HPCForge/Fused3S)
 * that it stands in for, by file:line in that repository.
 */
#ifndef F3S_B200_H
#define F3S_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define F3S_OK 0
#define F3S_ERR_INVALID_ARG (-1)  /* null pointer, negative size, bad enum               */
#define F3S_ERR_UNSUPPORTED (-2)  /* head dim / block width outside the supported set    */
#define F3S_ERR_CUDA (-3)         /* a CUDA runtime call or launch failed                */
#define F3S_ERR_WORKSPACE (-4)    /* workspace pointer null/misaligned or too small      */
#define F3S_ERR_DEVICE (-5)       /* a kernel reported an internal error through its status word */

/* stream handle: a cudaStream_t passed as void* so this header needs no CUDA include */
typedef void *f3s_stream_t;

/* Library version (major*10000 + minor*100 + patch). No reference counterpart. */
int f3s_version(void);

/* Number of CUDA kernels this library has launched in this process so far (all entry points, all
 * devices).  For benchmarks that report how many launches a timed region held.  No reference
 * counterpart. */
uint64_t f3s_kernel_launch_count(void);

/* Text of the calling thread's most recent error ("" if none).
 * Replaces the reference's printf + exit(-1) error path (src/F3S_kernel.cu:662-666,
 * src/utils.cu:73-77). */
const char *f3s_last_error_string(void);

/* ------------------------------------------------------------------------------------
 * CSR -> TC-block preprocessing.   Replaces preprocess_gpu (src/F3S.cpp:40-87) and the
 * kernels it drives (src/utils.cu:23-436).
 *
 * Split in two calls because the output sizes depend on the TCB count, which the
 * reference also reads back to the host in the middle of its pipeline
 * (src/utils.cu:307-309).
 * ------------------------------------------------------------------------------------ */

/* Bytes of device scratch both preprocessing calls need.  block_w is 8 or 16. */
size_t f3s_preprocess_workspace_bytes(int64_t num_nodes, int64_t nnz, int block_w);

/*
 * Phase 1: fills edge_to_row[nnz], edge_to_column[nnz], block_partition[nRW] (windows
 * without edges keep the caller's value, as src/utils.cu:141-142 does),
 * row_window_offset[nRW+1]; writes the TCB count and the largest per-window TCB count to
 * the two HOST ints (one device->host copy, stream-synchronising).
 *   colidx[nnz], rowptr[num_nodes+1]: int32 CSR; columns may be unsorted or repeated.
 *   block_h must be 16; block_w 8 or 16.  nRW = ceil(num_nodes/16).
 * Stands in for fill_edgeToRow_cuda, fill_segment_cuda, the sort + generate_edgetocolumn
 * stage and the first scan of seg_sort_dequ (src/utils.cu:276-309, 343-396).
 */
int f3s_preprocess_count(const int32_t *colidx, const int32_t *rowptr, int32_t num_nodes, int64_t nnz,
                         int32_t block_h, int32_t block_w, int32_t *block_partition,
                         int32_t *edge_to_column, int32_t *edge_to_row, int32_t *row_window_offset,
                         void *workspace, size_t workspace_bytes, int32_t *n_tcb_host,
                         int32_t *max_tcb_per_window_host, f3s_stream_t stream);

/*
 * Same as f3s_preprocess_count for a rectangular slice of the adjacency: num_nodes rows,
 * column ids in [0, num_cols).  Used when the row windows of one graph are sharded over
 * several GPUs (each holds a contiguous block of rows and all columns).  The reference is
 * single-GPU and square; this variant has no counterpart there.
 */
int f3s_preprocess_count_rect(const int32_t *colidx, const int32_t *rowptr, int32_t num_nodes, int32_t num_cols,
                              int64_t nnz, int32_t block_h, int32_t block_w, int32_t *block_partition,
                              int32_t *edge_to_column, int32_t *edge_to_row, int32_t *row_window_offset,
                              void *workspace, size_t workspace_bytes, int32_t *n_tcb_host,
                              int32_t *max_tcb_per_window_host, f3s_stream_t stream);

/*
 * Phase 2: fills the remaining members of the tuple preprocess_gpu returns
 * (src/F3S.cpp:83-86): sorted_row_windows[nRW], tcblock_rowid[nTCB], tcblocktile_id[nnz],
 * tcblock_offset[nTCB+1], sparse_a_to_x_idx[nTCB*block_w], tcb_bitmap[nTCB*16*block_w/64].
 * All six arrays are fully written (padding slots and empty bitmaps become 0), so the
 * caller need not zero them.  Inputs are the arrays phase 1 produced.  The arrays need only their
 * natural alignment; sparse_a_to_x_idx and tcb_bitmap that start on a 16-byte boundary (any torch
 * or cudaMalloc allocation) are written with 16-byte stores.  Rows whose columns do not ascend, or
 * that hold an edge twice, are legal (tile ids then follow CSR order, as in the reference).
 * Stands in for generate_tcblock_rowid_cuda, generate_tcoffset_id_atob_cuda, the second
 * scan and sort_row_windows_by_tcb_count (src/utils.cu:53-78, 173-267, 310-341, 400-436).
 */
int f3s_preprocess_fill(const int32_t *colidx, const int32_t *rowptr, int32_t num_nodes, int64_t nnz,
                        int32_t block_h, int32_t block_w, const int32_t *edge_to_column,
                        const int32_t *edge_to_row, const int32_t *row_window_offset, int32_t n_tcb,
                        int32_t *sorted_row_windows, int32_t *tcblock_rowid, uint8_t *tcblocktile_id,
                        int32_t *tcblock_offset, int32_t *sparse_a_to_x_idx, uint64_t *tcb_bitmap,
                        void *workspace, size_t workspace_bytes, f3s_stream_t stream);

/* ------------------------------------------------------------------------------------
 * Fused SDDMM -> softmax -> SpMM forward.   Replaces the five launchers
 * f3sCuda1tb1tcb / f3sCuda1tb1rw / f3sCuda1tb1rwScheduled (+Clocked twins)
 * (src/F3S_kernel.cu:324-671) and the kernels behind them (src/F3S_kernel.cu:677-2326).
 * ------------------------------------------------------------------------------------ */

/* Bytes of device scratch f3s_forward needs for this problem (schedule, and partial
 * results of row windows that are split across warps). */
size_t f3s_forward_workspace_bytes(int32_t n_row_windows, int64_t n_tcb, int32_t block_w, int32_t heads,
                                   int32_t head_dim);

/*
 * out[r, h, :] = softmax_over_row_r( mask(Q[r,h,:] . K[c,h,:] / scale_divisor) ) . V[c,h,:]
 * for the columns c of CSR row r, using the TC-block arrays of f3s_preprocess_*.
 *
 *   row_window_offset[nRW+1], sparse_a_to_x_idx[nTCB*block_w], tcb_bitmap[...]: as produced
 *       by preprocessing with the same block_w (16 for the reference's f3s_1tb1rw* ops,
 *       8 for f3s_1tb1tcb).
 *   sorted_row_windows[nRW] or NULL: processing order of the windows (the reference's
 *       "scheduled" variants, src/F3S_kernel.cu:82-97); NULL = natural order.
 *   q, k, v: fp16, row r / head h / feature f at  ptr[r*ld + h*head_dim + f];  ld >= heads*head_dim
 *       and a multiple of 8 elements; pointers 16-byte aligned.  heads = 1 is the
 *       reference's layout [N, d].
 *   scale_divisor: scores are DIVIDED by it (src/F3S_kernel.cu:1666-1667); 1.0 = none.
 *   apply_softmax = 0 gives (mask(QK^T)/scale_divisor) V, the reference's f2sKernel1tb1rw
 *       (src/F3S_kernel.cu:2186-2326).
 *   out: fp32 [num_nodes, heads*head_dim] contiguous; every element is written (rows
 *       without edges become 0), so it need not be zeroed.
 *   sddmm_out or NULL: when given, receives the masked, unscaled scores of every 16x8 tile
 *       in tile-major, row-major order ([nTCB*block_w/8][16][8] fp32) -- the optional
 *       third output of f3s_1tb1tcb (src/F3S_kernel.cu:99-115); heads must be 1.
 *   head_dim: a multiple of 16 from 16 to 128 (32, 64 and 128 run natively, the others zero-padded
 *       on chip to the next of those).  The reference needs d % 16 == 0 as well (d % 32 for its
 *       permuted kernels, src/F3S_kernel.cu:1640).
 */
int f3s_forward(const int32_t *row_window_offset, const int32_t *sorted_row_windows,
                const int32_t *sparse_a_to_x_idx, const uint64_t *tcb_bitmap, int32_t num_nodes,
                int32_t n_row_windows, int64_t n_tcb, int32_t block_w, int32_t heads, int32_t head_dim,
                int64_t ld, const void *q, const void *k, const void *v, float scale_divisor,
                int32_t apply_softmax, float *out, float *sddmm_out, void *workspace,
                size_t workspace_bytes, f3s_stream_t stream);

/*
 * The score stage alone on the 5th-generation tensor cores (tcgen05.mma, accumulator in tensor memory):
 * sddmm_out receives what f3s_forward's sddmm_out receives -- the masked, unscaled scores of every 16x8
 * tile, [n_tcb*block_w/8][16][8] fp32 -- i.e. the optional third output of the reference's f3s_1tb1tcb
 * (saveSddmmResult, src/F3S_kernel.cu:99-115), computed as S^T = K_g Q^T with M = 128 gathered key rows,
 * N = 16 query rows per product.  head_dim must be 64, one head; q rows at ld_q, k rows at ld_k elements.
 * workspace: 64 bytes of device scratch (16-byte aligned) whose status word f3s_forward_status reads: a
 * bounded wait that ran out is reported there.
 */
int f3s_sddmm_umma(const int32_t *row_window_offset, const int32_t *sparse_a_to_x_idx, const uint64_t *tcb_bitmap,
                   int32_t num_nodes, int32_t n_row_windows, int64_t n_tcb, int32_t block_w, int32_t head_dim,
                   int64_t ld_q, const void *q, int64_t ld_k, const void *k, float *sddmm_out, void *workspace,
                   size_t workspace_bytes, f3s_stream_t stream);

/*
 * f3s_forward writing an fp16 output ([num_nodes, heads*head_dim], 16-byte aligned) instead
 * of fp32: half the output bytes for callers whose next layer consumes fp16.  Accumulation
 * stays fp32; only the final store is rounded.  No reference counterpart (its ops always
 * return fp32, src/F3S_kernel.cu:600); arguments otherwise as f3s_forward, without sddmm_out.
 */
int f3s_forward_f16out(const int32_t *row_window_offset, const int32_t *sorted_row_windows,
                       const int32_t *sparse_a_to_x_idx, const uint64_t *tcb_bitmap, int32_t num_nodes,
                       int32_t n_row_windows, int64_t n_tcb, int32_t block_w, int32_t heads, int32_t head_dim,
                       int64_t ld, const void *q, const void *k, const void *v, float scale_divisor,
                       int32_t apply_softmax, void *out_f16, void *workspace, size_t workspace_bytes,
                       f3s_stream_t stream);

/*
 * f3s_forward that also records, per SM, when the launch first started and last finished
 * work there.  Replaces the reference's "Clocked" kernel twins and their timer array
 * (f3sCuda1tb1rwClocked / f3sCuda1tb1rwScheduledClocked, src/F3S_kernel.cu:460-579, stamps at
 * :30-40 and :1363-1367), which its ops select with checkSMActiveTime=True.
 *   sm_trace: device array of 2*F3S_SM_TRACE_SLOTS uint64; before the call the caller sets
 *       every even entry to UINT64_MAX and every odd entry to 0; afterwards entry 2*s is the
 *       earliest and 2*s+1 the latest %globaltimer value (ns) seen on SM s (untouched
 *       entries: SM not used).  Arguments otherwise as f3s_forward, without sddmm_out.
 */
#define F3S_SM_TRACE_SLOTS 512
int f3s_forward_traced(const int32_t *row_window_offset, const int32_t *sorted_row_windows,
                       const int32_t *sparse_a_to_x_idx, const uint64_t *tcb_bitmap, int32_t num_nodes,
                       int32_t n_row_windows, int64_t n_tcb, int32_t block_w, int32_t heads, int32_t head_dim,
                       int64_t ld, const void *q, const void *k, const void *v, float scale_divisor,
                       int32_t apply_softmax, float *out, void *workspace, size_t workspace_bytes,
                       uint64_t *sm_trace, f3s_stream_t stream);

/*
 * Repeated calls on one graph.  f3s_forward schedules the row windows (a memset and a small kernel)
 * before every launch, as the reference re-derives its launch geometry on every call
 * (src/F3S_kernel.cu:581-612).  A caller that runs the same graph many times (every layer and step of
 * a model) can schedule once and then pay one kernel launch per call:
 *   f3s_forward_plan:    fills `workspace` (f3s_forward_workspace_bytes bytes, 256-byte aligned) with the
 *                        schedule for (row_window_offset, sorted_row_windows, heads, head_dim).
 *   f3s_forward_planned: the fused kernel alone, on a workspace prepared by f3s_forward_plan with the same
 *                        sizes.  The kernel leaves the scratch ready for the next call.  Beyond f3s_forward:
 *                        k and v have their own row stride ld_kv (for instance K and V rows interleaved in one
 *                        gathered buffer), and the output may be fp16 (out_is_half).  No score dump.
 * Calls that share a workspace must not overlap on the GPU.  After a call whose status
 * (f3s_forward_status) is not F3S_OK the workspace must be planned again.
 */
int f3s_forward_plan(const int32_t *row_window_offset, const int32_t *sorted_row_windows, int32_t num_nodes,
                     int32_t n_row_windows, int64_t n_tcb, int32_t block_w, int32_t heads, int32_t head_dim,
                     void *workspace, size_t workspace_bytes, f3s_stream_t stream);
int f3s_forward_planned(const int32_t *row_window_offset, const int32_t *sorted_row_windows,
                        const int32_t *sparse_a_to_x_idx, const uint64_t *tcb_bitmap, int32_t num_nodes,
                        int32_t n_row_windows, int64_t n_tcb, int32_t block_w, int32_t heads, int32_t head_dim,
                        int64_t ld_q, const void *q, int64_t ld_kv, const void *k, const void *v,
                        float scale_divisor, int32_t apply_softmax, void *out, int32_t out_is_half, void *workspace,
                        size_t workspace_bytes, f3s_stream_t stream);

/*
 * Two-phase forward for row-sharded attention (no reference counterpart: the reference is single-GPU).
 * A rank that owns a block of rows holds its own K / V rows before the step and receives the others'
 * through a collective.  Phase 1 works on the columns with id >= col_split (by convention the rank's
 * own rows, which the caller numbers last) and can run while the collective is in flight; phase 2 works
 * on the columns with id < col_split, continues from the unnormalised result phase 1 left in the scratch
 * (running max, running sum, accumulator per row) and writes the output.  Together they compute exactly
 * what f3s_forward computes (same masking and softmax; the order of accumulation differs).
 *   phase_split[n_row_windows]: for every window the index (into the TC-block arrays) of its first TC
 *       block whose first column id is >= col_split, or row_window_offset[w+1] if it has none.  The block
 *       before it is the only one that may hold columns of both kinds; both phases visit it, each masking
 *       the other's columns.
 *   workspace: f3s_forward_phased_workspace_bytes(...) bytes, 256-byte aligned, prepared once per graph
 *       by f3s_forward_phased_plan; then any number of (phase 1, phase 2) pairs.  `out` may be NULL in
 *       phase 1.  head_dim must be 64; softmax is always applied.
 */
size_t f3s_forward_phased_workspace_bytes(int32_t n_row_windows, int64_t n_tcb, int32_t block_w, int32_t heads,
                                          int32_t head_dim);
int f3s_forward_phased_plan(const int32_t *row_window_offset, const int32_t *sorted_row_windows,
                            const int32_t *phase_split, int32_t num_nodes, int32_t n_row_windows, int64_t n_tcb,
                            int32_t block_w, int32_t heads, int32_t head_dim, void *workspace,
                            size_t workspace_bytes, f3s_stream_t stream);
int f3s_forward_phase(int32_t phase, const int32_t *row_window_offset, const int32_t *sorted_row_windows,
                      const int32_t *sparse_a_to_x_idx, const uint64_t *tcb_bitmap, const int32_t *phase_split,
                      int32_t col_split, int32_t num_nodes, int32_t n_row_windows, int64_t n_tcb, int32_t block_w,
                      int32_t heads, int32_t head_dim, int64_t ld_q, const void *q, int64_t ld_kv, const void *k,
                      const void *v, float scale_divisor, float *out, void *workspace, size_t workspace_bytes,
                      f3s_stream_t stream);

/*
 * Co-scheduling with a collective (no reference counterpart).  The fused kernels are persistent: one
 * CTA per SM, each holding the SM's whole shared memory and register file until the call's work is
 * done.  A collective launched beside them (NCCL's kernels need SMs of their own) would wait for that.
 * f3s_set_max_ctas(n) makes every later forward launch of this process use at most n CTAs, leaving the
 * other SMs to the collective; 0 removes the cap.  Returns the previous value, so that a caller can put it
 * back.  The environment variable F3S_MAX_CTAS sets the initial value.
 */
int32_t f3s_set_max_ctas(int32_t max_ctas);

/*
 * Results that do not depend on how the work is divided (no reference counterpart).  By default the
 * forward cuts heavy row windows into chunks whose size follows the load of the call (graph size, head
 * count, SM count) and picks its kernel by the graph's shape; the partial results of the chunks are
 * merged in a fixed order, so a call is deterministic, but two calls that see the same window inside
 * different problems (one GPU vs. a row shard of it, one head vs. eight, workspace vs. built-in scratch)
 * may round differently.  f3s_set_canonical_chunk_tiles(t) with t > 0 fixes the chunk size at t 8-column
 * tiles (rounded up to a whole step of 4), always uses the scheduled kernels and one data path per head
 * dimension: every window is then computed by the same sequence of operations in every such call and the
 * outputs are equal bit for bit, provided the windows list their columns in the same order (row shards
 * numbered in the padded gather layout that keeps the global order).  It costs a few per cent (more,
 * smaller chunks on big graphs; no one-launch mode on small ones).  0 restores the default.  Process-wide.
 * 128 is a sensible value.
 */
void f3s_set_canonical_chunk_tiles(int32_t tiles);

/*
 * Device-side error reporting.  The reference's kernels report nothing and its host code ends the
 * process on any CUDA error (printf + exit(-1), src/F3S_kernel.cu:662-666); here a kernel that cannot
 * finish its work writes a status word into the scratch of the call and returns, and the host reads it.
 *
 * f3s_forward_status: status of the most recent f3s_forward / _f16out / _lse / _traced call that used
 *   `workspace`, issued on `stream`.
 *     status_host == NULL: blocks until the stream has drained, returns F3S_OK or F3S_ERR_DEVICE
 *       (text through f3s_last_error_string): the schedule's unit list overflowed, or a bounded wait
 *       for an asynchronous copy ran out -- in both cases some output rows were not written.
 *     status_host != NULL (HOST pointer, pinned for a truly asynchronous copy): enqueues a 4-byte copy
 *       of the raw word and returns at once; after synchronising, f3s_status_word_to_code(*status_host)
 *       gives the same code and text.
 * f3s_forward_static_status: the same for the built-in scratch of f3s_forward_static.
 * f3s_debug_set_unit_list_limit: testing aid without effect on results in normal use -- caps the
 *   capacity of the schedule's unit list (0 removes the cap) so that the overflow report can be
 *   exercised by a test; with a cap in place heavy row windows may be left unprocessed and the status
 *   call says so.
 */
int f3s_forward_status(const void *workspace, int32_t *status_host, f3s_stream_t stream);
int f3s_forward_static_status(int32_t *status_host, f3s_stream_t stream);
int f3s_status_word_to_code(int32_t word);
void f3s_debug_set_unit_list_limit(int32_t limit);

/*
 * Checks every index of a plan that the forward and backward kernels dereference without a test of
 * their own: row_window_offset starts at 0, never decreases and ends at n_tcb; every entry of
 * sorted_row_windows (may be NULL) lies in [0, n_row_windows); every column id of sparse_a_to_x_idx
 * lies in [0, num_kv_rows), the row count of the K / V tensors the plan will be used with.  Plans made
 * by f3s_preprocess_* satisfy this by construction (columns are range-checked there); plans read from
 * a file or assembled from parts should be checked once before their first use.  Blocks until the
 * answer is known.  Returns F3S_OK, or F3S_ERR_INVALID_ARG with the first violation in the error text.
 *   workspace: 16 bytes of device scratch, 16-byte aligned.
 * The reference has no such check (its kernels index K and V with whatever the plan holds,
 * src/F3S_kernel.cu:1652-1662).
 */
int f3s_validate_plan(const int32_t *row_window_offset, const int32_t *sorted_row_windows,
                      const int32_t *sparse_a_to_x_idx, int32_t n_row_windows, int64_t n_tcb, int32_t block_w,
                      int32_t num_kv_rows, void *workspace, size_t workspace_bytes, f3s_stream_t stream);

/*
 * Training support.  The reference is inference-only (src/F3S.cpp:298-305 exports forward ops and
 * no gradient); these three entry points have no reference counterpart.
 *
 * f3s_forward_lse: f3s_forward with softmax that also returns lse[row * heads + head], the
 *   log-sum-exp of the row's scaled scores in the log2 domain (natural-log value = lse * ln 2):
 *   the probability of edge (i, j) is exp2(q_i . k_j * log2(e) / scale_divisor - lse_i).
 *   Rows without edges get 0.
 *
 * f3s_backward: dq, dk, dv ([N, H, d] contiguous, fp32 or fp16 when grads_are_half) from
 *   d_out = dL/d(out) ([N, H, d] contiguous fp32), the forward's out and lse, and q, k, v as
 *   given to the forward (row stride ld).  Needs the TC-block arrays of the graph AND of its
 *   transpose (f3s_preprocess_* run on the CSR of A^T: row j lists the i with an edge (i, j));
 *   both with the same block_w.  The graph must be square: K and V have num_nodes rows.
 *   Deterministic: no atomics on the gradients.  head_dim: a multiple of 16, 16..128.
 *   workspace: f3s_backward_workspace_bytes(...) bytes, 256-byte aligned.
 */
int f3s_forward_lse(const int32_t *row_window_offset, const int32_t *sorted_row_windows,
                    const int32_t *sparse_a_to_x_idx, const uint64_t *tcb_bitmap, int32_t num_nodes,
                    int32_t n_row_windows, int64_t n_tcb, int32_t block_w, int32_t heads, int32_t head_dim,
                    int64_t ld, const void *q, const void *k, const void *v, float scale_divisor, float *out,
                    float *lse, void *workspace, size_t workspace_bytes, f3s_stream_t stream);

size_t f3s_backward_workspace_bytes(int32_t num_nodes, int64_t n_tcb, int64_t n_tcb_t, int32_t block_w,
                                    int32_t heads, int32_t head_dim);

int f3s_backward(const int32_t *row_window_offset, const int32_t *sorted_row_windows,
                 const int32_t *sparse_a_to_x_idx, const uint64_t *tcb_bitmap, int64_t n_tcb,
                 const int32_t *row_window_offset_t, const int32_t *sorted_row_windows_t,
                 const int32_t *sparse_a_to_x_idx_t, const uint64_t *tcb_bitmap_t, int64_t n_tcb_t,
                 int32_t num_nodes, int32_t n_row_windows, int32_t block_w, int32_t heads, int32_t head_dim,
                 int64_t ld, const void *q, const void *k, const void *v, float scale_divisor, const float *out,
                 const float *lse, const float *d_out, void *dq, void *dk, void *dv, int32_t grads_are_half,
                 void *workspace, size_t workspace_bytes, f3s_stream_t stream);

/*
 * The stages of f3s_backward as separate calls, for row-sharded training (no reference counterpart).
 * A rank owns a block of rows: its queries and the same block of keys / values.  Gathered operands
 * may then hold more rows than the block and are indexed by the column ids of the plan that is
 * passed (for instance the padded all-gather layout), so the plans are rectangular.
 *   f3s_backward_prepare: d_out_f16 = fp16(d_out) ([num_rows, H, d]) and stats[(row*H + head)*2 + {0,1}]
 *       = {lse, delta = d_out . out} for the block.
 *   f3s_backward_dq:  dq of the block.  q: the block's rows; k, v: gathered, indexed by the plan's
 *       column ids; d_out_f16, stats: of the block.
 *   f3s_backward_dkv: dk, dv of the block from the plan of the TRANSPOSED graph's rows of the block.
 *       k, v: the block's rows; q_g, d_out_f16_g, stats_g: of ALL query rows, gathered, indexed by
 *       that plan's column ids.
 *   workspace: f3s_backward_stage_workspace_bytes(n_tcb of the plan, ..., dkv = 0 or 1).
 */
int f3s_backward_prepare(const float *out, const float *d_out, const float *lse, int32_t num_rows, int32_t heads,
                         int32_t head_dim, void *d_out_f16, float *stats, f3s_stream_t stream);

size_t f3s_backward_stage_workspace_bytes(int64_t n_tcb, int32_t block_w, int32_t heads, int32_t head_dim,
                                          int32_t dkv);

int f3s_backward_dq(const int32_t *row_window_offset, const int32_t *sorted_row_windows,
                    const int32_t *sparse_a_to_x_idx, const uint64_t *tcb_bitmap, int64_t n_tcb, int32_t num_rows,
                    int32_t n_row_windows, int32_t block_w, int32_t heads, int32_t head_dim, int64_t ld_q,
                    const void *q, int64_t ld_kv, const void *k, const void *v, float scale_divisor,
                    const void *d_out_f16, const float *stats, void *dq, int32_t grads_are_half, void *workspace,
                    size_t workspace_bytes, f3s_stream_t stream);

int f3s_backward_dkv(const int32_t *row_window_offset_t, const int32_t *sorted_row_windows_t,
                     const int32_t *sparse_a_to_x_idx_t, const uint64_t *tcb_bitmap_t, int64_t n_tcb_t,
                     int32_t num_rows, int32_t n_row_windows, int32_t block_w, int32_t heads, int32_t head_dim,
                     int64_t ld_kv, const void *k, const void *v, int64_t ld_q, const void *q_g,
                     const void *d_out_f16_g, const float *stats_g, float scale_divisor, void *dk, void *dv,
                     int32_t grads_are_half, void *workspace, size_t workspace_bytes, f3s_stream_t stream);

/*
 * f3s_forward for hosts that are not allowed to allocate device memory while they run.
 * (No counterpart in the reference, whose launchers allocate their outputs and scratch
 * with torch on every call, src/F3S_kernel.cu:596-600.)
 *
 * Who needs it: a process whose device-memory budget is frozen once its plugins are loaded
 * (an inference server, an embedded runtime), and a runtime that calls this library from
 * inside its own execution callback, where cudaMalloc would synchronise the device or
 * re-enter the host's allocator.  Such a caller has nowhere to take f3s_forward's
 * workspace from, so this variant keeps the schedule and the partial results of split
 * row windows in an array built into the library: F3S_STATIC_SCRATCH_BYTES (32 MiB) of
 * device memory on every GPU that loads the library, held until the process exits.
 *
 * Arguments are those of f3s_forward without sddmm_out, workspace and workspace_bytes.
 * Inputs and the output are still the caller's buffers.  The call makes no cudaMalloc,
 * cudaFree or other allocating call.  Results agree with f3s_forward's to rounding (heavy
 * row windows may be cut into fewer, larger chunks so that the scratch fits).
 *
 * Limits and rules:
 *   - A problem whose schedule does not fit the array is rejected with F3S_ERR_WORKSPACE
 *     and a message naming the bytes needed; nothing is launched.  To make a schedule fit,
 *     chunks of heavy windows are allowed to grow up to 65 536 8-column tiles; with head
 *     dimension 64 that admits roughly 10^8 tiles x heads per call (about ten times a
 *     Reddit-sized graph) before the call is refused.
 *   - The first call on each device looks up the array's device address (one
 *     cudaGetSymbolAddress, with that device current) and keeps it; make that first call
 *     outside any stream capture.
 *   - All calls on one device share the array and it keeps the previous call's contents.
 *     The counters that must start at zero are cleared on the stream at the start of every
 *     call.  Two calls that may overlap on the GPU (different streams, or another thread)
 *     race on the array and give wrong results: serialise them.
 */
#define F3S_STATIC_SCRATCH_BYTES (32u << 20)
int f3s_forward_static(const int32_t *row_window_offset, const int32_t *sorted_row_windows,
                       const int32_t *sparse_a_to_x_idx, const uint64_t *tcb_bitmap, int32_t num_nodes,
                       int32_t n_row_windows, int64_t n_tcb, int32_t block_w, int32_t heads, int32_t head_dim,
                       int64_t ld, const void *q, const void *k, const void *v, float scale_divisor,
                       int32_t apply_softmax, float *out, f3s_stream_t stream);

/* ------------------------------------------------------------------------------------
 * Measurement aid (no reference counterpart): gathers n_ids rows of 128 bytes from `table`
 * (table_rows rows, 16-byte aligned) at the row ids given (each in [0, table_rows); not checked) and
 * discards them -- loads only, eight 16-byte loads in flight per thread.  Timed by the caller with
 * events on `stream`, 128 * n_ids bytes / time is the gather rate this GPU can sustain from L2 (table
 * smaller than L2) or from HBM (larger): the ceiling for the fused kernel's K / V row gathers.
 * n_ids is rounded down to a multiple of 32.  sink: 4 bytes of device memory (never written in practice).
 * ------------------------------------------------------------------------------------ */
int f3s_probe_gather_rows(const void *table, int64_t table_rows, const int32_t *row_ids, int64_t n_ids, void *sink,
                          f3s_stream_t stream);

/* ------------------------------------------------------------------------------------
 * Multi-GPU planning (host only, no device work): cut points of a contiguous row-window
 * partition with near-equal TCB counts.  The reference is single-GPU; this has no
 * counterpart there.
 *   row_window_offset_host[nRW+1]: HOST copy of the window offsets.
 *   cuts_host[n_parts+1]: HOST output, window indices, cuts[0]=0, cuts[n_parts]=nRW.
 * ------------------------------------------------------------------------------------ */
int f3s_partition_row_windows(const int32_t *row_window_offset_host, int32_t n_row_windows, int32_t n_parts,
                              int32_t *cuts_host);

#ifdef __cplusplus
}
#endif
#endif /* F3S_B200_H */
