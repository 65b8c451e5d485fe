// CSR -> TC-block preprocessing for sm_100a, all on the device, no global sort.
//
// The reference sorts every (window, column) pair of the graph with Thrust and then walks
// each 16-row window with ONE thread (src/utils.cu:131-153, 173-224).  Here a window is owned
// by one warp (at most SMALL_N edges; eight windows per CTA, no block barrier) or by one CTA
// (larger windows, taken from a list the warp kernel builds):
//   phase 1 (window_rank_small / window_rank_kernel): rank of every edge's column among the
//       window's distinct columns, TCB count = ceil(U/bw).  When the window's column range
//       fits, an occupancy bitmap of the range in shared memory replaces sorting: one atomicOr
//       per edge, prefix sum of the words' popcounts, rank = prefix + popcount of the lower
//       bits.  Otherwise a stable LSD radix sort (shared memory, or an L2-resident slice of
//       the workspace), distinct compaction and binary search.
//   scan -> window offsets, one device->host copy of the TCB count.
//   phase 2 (window_fill_small / window_fill_kernel): original-column list and occupancy
//       bitmaps (assembled in shared memory, stored once), per-TCB edge counts and the tile ids
//       regrouped by TCB.  The CTA kernel derives counts and tile ids from the occupancy words
//       alone when every row's columns ascend strictly (CSR order inside a TC block is then the
//       row-major order of its bits); otherwise, and in the warp kernel, a stable radix sort
//       (key = TCB id inside the window, payload = tile id, packed in one word) regroups them.
//   The CTA kernels pull their windows from a counter and ask for the next window's header, row
//   pointers and edge slices (prefetch into L2) while the current one is worked on: a pass over
//   a window's edges is otherwise bound by one DRAM round trip per step.
//   scan -> TCB edge offsets; one CTA radix-sorts the windows by TCB count (descending,
//       stable) for the schedule.
// Outputs are bit-identical to the reference's arrays for inputs on which its
// fill_edgeToRow stride defect (src/utils.cu:348) is inert, and implement the intended
// semantics (every edge gets its row) otherwise.
#include <limits.h>

#include "common.cuh"

namespace f3s {

constexpr int WIN_THREADS = 256;
constexpr int WIN_WARPS = WIN_THREADS / 32;
constexpr int WIN_CAP = 4096;  // largest window (edges) sorted entirely in shared memory
constexpr int SCHED_THREADS = 1024;
constexpr int SCHED_WARPS = SCHED_THREADS / 32;

enum { PH_ERROR = 0, PH_MAX_TCB = 1, PH_SUM_TCB = 2, PH_N_LARGE = 3, PH_N_LARGE_FILL = 4, PH_FILL_NEXT = 5, PH_RANK_NEXT = 6, PH_INTS = 16 };

// ---- block-wide helpers ---------------------------------------------------------------

// Exclusive scan of one int per thread; returns the exclusive prefix, `total` = block sum.
// aux: >= 33 ints of shared memory.  Contains __syncthreads.
template <int WARPS>
__device__ __forceinline__ int block_excl_scan(int v, int *aux, int &total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  __syncthreads();  // protects aux against the previous use
  if (lane == 31) aux[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = (lane < WARPS) ? aux[lane] : 0;
    int winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int t = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += t;
    }
    if (lane < WARPS) aux[lane] = winc - w;
    if (lane == 31) aux[32] = winc;
  }
  __syncthreads();
  total = aux[32];
  return aux[warp] + inc - v;
}

// Lanes of the warp that hold the same digit as this lane (bit b of the result = lane b); lanes
// with valid == false form a group of their own.  (One match.any; building the mask from one
// ballot per digit bit was measured 20 % slower on the regrouping sort.)
__device__ __forceinline__ unsigned same_digit_lanes(unsigned d, bool valid) {
  return __match_any_sync(0xffffffffu, valid ? d : 0xffffffffu);
}

// One stable LSD radix pass over `dbits` (<= 10) bits of W-typed words: dst = src ordered by
// (src >> shift) & (2^dbits - 1), ties in source order.  Every warp owns a contiguous slice so
// that source order is preserved.  hist: WARPS << dbits ints, aux: 33 ints of shared memory.
// AHEAD > 1: a lane fetches that many of its words before it uses the first (for callers that run
// as a single CTA, where nothing else hides the latency of the loads).
template <typename W, int WARPS, int AHEAD = 1>
__device__ void radix_pass(const W *src, W *dst, int n, int shift, int dbits, int *hist, int *aux) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nd = 1 << dbits;
  const unsigned dmask = (unsigned)nd - 1u;
  for (int i = tid; i < WARPS * nd; i += WARPS * 32) hist[i] = 0;
  __syncthreads();
  const int per = ((n + WARPS - 1) / WARPS + 31) & ~31;
  const int beg = min(n, warp * per), end = min(n, beg + per);
  int *myh = hist + warp * nd;
  if (AHEAD > 1) {
    for (int i0 = beg + lane; i0 < end; i0 += 32 * AHEAD) {
      W k[AHEAD];
#pragma unroll
      for (int u = 0; u < AHEAD; ++u) k[u] = (i0 + 32 * u < end) ? src[i0 + 32 * u] : W(0);
#pragma unroll
      for (int u = 0; u < AHEAD; ++u)
        if (i0 + 32 * u < end) atomicAdd(&myh[(unsigned)(k[u] >> shift) & dmask], 1);
    }
  } else {
    for (int i = beg + lane; i < end; i += 32) atomicAdd(&myh[(unsigned)(src[i] >> shift) & dmask], 1);
  }
  __syncthreads();
  {  // digit-major, warp-minor exclusive offsets
    int carry = 0;
    for (int base = 0; base < nd; base += WARPS * 32) {
      const int d = base + tid;
      int tot = 0;
      if (d < nd)
        for (int w = 0; w < WARPS; ++w) tot += hist[w * nd + d];
      int total;
      int run = carry + block_excl_scan<WARPS>(tot, aux, total);
      if (d < nd)
        for (int w = 0; w < WARPS; ++w) {
          const int t = hist[w * nd + d];
          hist[w * nd + d] = run;
          run += t;
        }
      carry += total;
    }
  }
  __syncthreads();
  for (int j0 = beg; j0 < end; j0 += 32 * AHEAD) {
    W k[AHEAD];
#pragma unroll
    for (int u = 0; u < AHEAD; ++u) {
      const int i = j0 + 32 * u + lane;
      k[u] = (i < end) ? src[i] : W(0);
    }
#pragma unroll
    for (int u = 0; u < AHEAD; ++u) {
      const int i0 = j0 + 32 * u;
      if (i0 >= end) break;  // warp-uniform
      const bool valid = i0 + lane < end;
      const W key = k[u];
      const unsigned d = (unsigned)(key >> shift) & dmask;
      const unsigned peers = same_digit_lanes(d, valid);
      const int rank = __popc(peers & ((1u << lane) - 1u));
      const int base = valid ? myh[d] : 0;
      __syncwarp();
      if (valid) {
        dst[base + rank] = key;
        if (lane == __ffs(peers) - 1) myh[d] = base + __popc(peers);
      }
      __syncwarp();
    }
  }
  __syncthreads();
}

// The same pass for ONE warp (no block barrier): hist holds 1 << dbits ints of that warp.
template <typename W>
__device__ void warp_radix_pass(const W *src, W *dst, int n, int shift, int dbits, int *hist) {
  const int lane = threadIdx.x & 31;
  const int nd = 1 << dbits;
  const unsigned dmask = (unsigned)nd - 1u;
  for (int i = lane; i < nd; i += 32) hist[i] = 0;
  __syncwarp();
  for (int i = lane; i < n; i += 32) atomicAdd(&hist[(unsigned)(src[i] >> shift) & dmask], 1);
  __syncwarp();
  {  // exclusive offsets: every lane owns a run of consecutive digits
    const int per = (nd + 31) / 32;
    const int b = min(nd, lane * per), e = min(nd, b + per);
    int local = 0;
    for (int i = b; i < e; ++i) local += hist[i];
    int inc = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += t;
    }
    int run = inc - local;
    for (int i = b; i < e; ++i) {
      const int t = hist[i];
      hist[i] = run;
      run += t;
    }
  }
  __syncwarp();
  for (int i0 = 0; i0 < n; i0 += 32) {
    const int i = i0 + lane;
    const bool valid = i < n;
    const W key = valid ? src[i] : W(0);
    const unsigned d = (unsigned)(key >> shift) & dmask;
    const unsigned peers = same_digit_lanes(d, valid);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    const int base = valid ? hist[d] : 0;
    __syncwarp();
    if (valid) {
      dst[base + rank] = key;
      if (lane == __ffs(peers) - 1) hist[d] = base + __popc(peers);
    }
    __syncwarp();
  }
}

__device__ __forceinline__ int lower_bound_dev(const int *a, int n, int key) {
  int lo = 0, hi = n;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (a[mid] < key) lo = mid + 1; else hi = mid;
  }
  return lo;
}

// Windows with at most SMALL_N edges are handled by one WARP each (eight windows per CTA, no block
// barrier, little shared memory, many resident warps); larger windows by one CTA each.  Both
// kernels of a phase are launched over all windows and skip the windows of the other class.
constexpr int SMALL_N = 512;
constexpr int SW_WARPS = 8;

// Requests the 128-byte lines of a[0 .. n) into L2 (no data returned, nothing waits for it).
__device__ __forceinline__ void prefetch_l2_lines(const int *a, int n, int tid, int n_threads) {
  for (int i = tid * 32; i < n; i += n_threads * 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(a + i));
  if (tid == 0 && n > 0) asm volatile("prefetch.global.L2 [%0];" ::"l"(a + n - 1));
}

// What a CTA of window_rank_kernel needs to know about entry li of its window list (nothing is loaded past the list).
struct RankWindow {
  int w, s, n;
};
__device__ __forceinline__ RankWindow rank_window(int li, int n_large, const int *__restrict__ large_list,
                                                  const int *__restrict__ rowptr, int n_nodes) {
  RankWindow f = {0, 0, 0};
  if (li < n_large) {
    f.w = large_list[li];
    const int row0 = f.w * 16, row1 = min(row0 + 16, n_nodes);
    f.s = rowptr[row0];
    f.n = rowptr[row1] - f.s;
  }
  return f;
}
constexpr int RANK_AHEAD = 4;  // loads a thread keeps in flight in the passes over a window's edges
constexpr int RANK_KREG = 32;  // edges per thread that stay in registers between the passes

// ---- phase 1 --------------------------------------------------------------------------
// One CTA per 16-row window.  Restates, for the whole window at once, what the reference's
// sort (src/utils.cu:281-289) + generate_edgetocolumn (src/utils.cu:131-153) + fill_edgeToRow
// (src/utils.cu:343-352, intended semantics) produce.  Two ways to rank the window's columns:
//   * occupancy bitmap over the window's column range [cmin, cmax] in shared memory, when the
//     range fits (<= 32 * BM_WORDS columns) and is not much larger than the edge count: one
//     atomicOr per edge, a prefix sum of the words' popcounts, rank = prefix + popcount of the
//     lower bits.  No sort at all; linear in edges + range / 32.
//   * otherwise the stable LSD radix sort + distinct compaction + binary search.
constexpr int BM_WORDS = 8192;
constexpr int RANK_SMEM_BYTES = 2 * BM_WORDS * (int)sizeof(int);
constexpr int RANK_DBITS = 10;
static_assert(2 * WIN_CAP + (WIN_WARPS << RANK_DBITS) <= 2 * BM_WORDS, "the sort path's buffers share the bitmap path's memory");

__global__ void __launch_bounds__(WIN_THREADS, 3)  // three CTAs per SM: 64 KB of shared memory, 85 registers each
window_rank_kernel(const int *__restrict__ colidx, const int *__restrict__ rowptr, int n_nodes, int n_cols,
                   int bw, const int *__restrict__ large_list, int *__restrict__ block_partition,
                   int *__restrict__ e2c, int *__restrict__ e2r, int *scratch_a, int *scratch_b, int *hdr) {
  extern __shared__ __align__(16) int dsm[];
  __shared__ int s_aux[33];
  __shared__ int s_min[WIN_WARPS], s_max[WIN_WARPS];
  __shared__ int s_rp2[2][17];  // row pointers of the current and of the next window
  __shared__ int s_pull;
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int n_large = hdr[PH_N_LARGE];  // windows with more than SMALL_N edges, listed by window_rank_small
  // A CTA pulls its windows from a counter, two ahead: while window k is worked on, the header and the row
  // pointers of window k+1 are loaded and its slice of colIdx is requested into L2 (a pass over a window's
  // edges otherwise pays DRAM latency per step), and the counter is read for window k+2 -- none of these
  // round trips is waited for.
  if (tid == 0) s_pull = atomicAdd(&hdr[PH_RANK_NEXT], 2);
  __syncthreads();
  int li = s_pull, li_next = li + 1, pulled = 0, buf = 0;
  RankWindow cur = rank_window(li, n_large, large_list, rowptr, n_nodes), ahead = cur;
  if (tid < 17 && li < n_large) s_rp2[0][tid] = rowptr[min(cur.w * 16 + tid, n_nodes)];
  bool staged = true;
  auto stage_next = [&]() {  // what the next window needs from memory, asked for while this one is worked on
    if (staged) return;
    staged = true;
    prefetch_l2_lines(colidx + ahead.s, ahead.n, tid, WIN_THREADS);
    if (tid < 17 && li_next < n_large) s_rp2[buf ^ 1][tid] = rowptr[min(ahead.w * 16 + tid, n_nodes)];
  };
  auto advance = [&]() {
    stage_next();
    if (tid == 0) s_pull = pulled;
    __syncthreads();
    li = li_next;
    li_next = s_pull;
    cur = ahead;
    buf ^= 1;
  };
  for (;; advance()) {
  __syncthreads();  // the previous window's shared memory (and s_pull) is no longer read
  if (li >= n_large) break;
  if (tid == 0) pulled = atomicAdd(&hdr[PH_RANK_NEXT], 1);  // consumed in advance()
  ahead = rank_window(li_next, n_large, large_list, rowptr, n_nodes);  // consumed in stage_next()
  staged = false;
  const int *s_rp = s_rp2[buf];
  const int w = cur.w, s = cur.s, n = cur.n, t = s + n;
  const int row0 = w * 16;

  // column range of the window; columns outside [0, n_cols) are an error
  int cmin = INT_MAX, cmax = INT_MIN;
  bool bad = false;
  // The first RANK_KREG * WIN_THREADS edges of the window stay in registers for all three passes (all their
  // loads are in flight together); what lies beyond is re-read, RANK_AHEAD loads at a time.  Slots past the
  // window's end repeat its last edge: harmless for the range and the occupancy bits, skipped when writing.
  int cv[RANK_KREG];
#pragma unroll
  for (int u = 0; u < RANK_KREG; ++u) {
    if (u * WIN_THREADS >= n) break;  // uniform; the later passes stop at the same slot
    cv[u] = colidx[min(s + tid + u * WIN_THREADS, t - 1)];
  }
#pragma unroll
  for (int u = 0; u < RANK_KREG; ++u) {
    if (u * WIN_THREADS >= n) break;
    bad |= (cv[u] < 0) | (cv[u] >= n_cols);
    cmin = min(cmin, cv[u]);
    cmax = max(cmax, cv[u]);
  }
  const int s_mem = s + RANK_KREG * WIN_THREADS;  // first edge that is not held in registers
  for (int e0 = s_mem + tid; e0 < t; e0 += WIN_THREADS * RANK_AHEAD) {
    int c[RANK_AHEAD];
#pragma unroll
    for (int u = 0; u < RANK_AHEAD; ++u) c[u] = colidx[min(e0 + u * WIN_THREADS, t - 1)];  // in flight together
#pragma unroll
    for (int u = 0; u < RANK_AHEAD; ++u) {
      bad |= (c[u] < 0) | (c[u] >= n_cols);
      cmin = min(cmin, c[u]);
      cmax = max(cmax, c[u]);
    }
  }
  stage_next();
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    cmin = min(cmin, __shfl_xor_sync(0xffffffffu, cmin, o));
    cmax = max(cmax, __shfl_xor_sync(0xffffffffu, cmax, o));
  }
  if (lane == 0) {
    s_min[warp] = cmin;
    s_max[warp] = cmax;
  }
  if (__syncthreads_or(bad)) {  // the host reports the error; nothing else of this window is needed
    if (tid == 0) atomicExch(&hdr[PH_ERROR], 1);
    continue;
  }
  // row of every edge (the row pointers came in above)
  for (int r = warp; r < 16; r += WIN_WARPS) {
    const int a = s_rp[r], b = s_rp[r + 1];
    for (int e = a + lane; e < b; e += 32) e2r[e] = row0 + r;
  }
#pragma unroll
  for (int i = 0; i < WIN_WARPS; ++i) {
    cmin = min(cmin, s_min[i]);
    cmax = max(cmax, s_max[i]);
  }
  const long long words = (((long long)cmax - cmin) >> 5) + 1;
  int n_uniq = 0;

  if (words <= BM_WORDS && words <= 8ll * n) {
    // ---- occupancy bitmap over [cmin, cmax]
    unsigned *bm = reinterpret_cast<unsigned *>(dsm);
    int *pre = dsm + BM_WORDS;
    const int nw = (int)words;
    for (int i = tid; i < nw; i += WIN_THREADS) bm[i] = 0u;
    __syncthreads();
#pragma unroll
    for (int u = 0; u < RANK_KREG; ++u) {
      if (u * WIN_THREADS >= n) break;  // uniform
      const int c = cv[u] - cmin;
      atomicOr(&bm[c >> 5], 1u << (c & 31));  // repeats set the same bit
    }
    for (int e0 = s_mem + tid; e0 < t; e0 += WIN_THREADS * RANK_AHEAD) {
      int c[RANK_AHEAD];
#pragma unroll
      for (int u = 0; u < RANK_AHEAD; ++u) c[u] = colidx[min(e0 + u * WIN_THREADS, t - 1)] - cmin;
#pragma unroll
      for (int u = 0; u < RANK_AHEAD; ++u) atomicOr(&bm[c[u] >> 5], 1u << (c[u] & 31));
    }
    __syncthreads();
    const int per = ((nw + WIN_THREADS - 1) / WIN_THREADS) | 1;  // odd: consecutive threads hit different banks
    const int wb = min(nw, tid * per), we = min(nw, wb + per);
    int local = 0;
    for (int i = wb; i < we; ++i) local += __popc(bm[i]);
    int run = block_excl_scan<WIN_WARPS>(local, s_aux, n_uniq);
    for (int i = wb; i < we; ++i) {
      pre[i] = run;
      run += __popc(bm[i]);
    }
    __syncthreads();
#pragma unroll
    for (int u = 0; u < RANK_KREG; ++u) {
      if (u * WIN_THREADS >= n) break;
      const int e = s + tid + u * WIN_THREADS;
      const int c = cv[u] - cmin;
      const int wi = c >> 5;
      if (e < t) e2c[e] = pre[wi] + __popc(bm[wi] & ((1u << (c & 31)) - 1u));
    }
    for (int e0 = s_mem + tid; e0 < t; e0 += WIN_THREADS * RANK_AHEAD) {
      int c[RANK_AHEAD];
#pragma unroll
      for (int u = 0; u < RANK_AHEAD; ++u) c[u] = colidx[min(e0 + u * WIN_THREADS, t - 1)] - cmin;
#pragma unroll
      for (int u = 0; u < RANK_AHEAD; ++u) {
        const int e = e0 + u * WIN_THREADS;
        const int wi = c[u] >> 5;
        if (e < t) e2c[e] = pre[wi] + __popc(bm[wi] & ((1u << (c[u] & 31)) - 1u));
      }
    }
  } else {
    // ---- stable radix sort of the window's columns, distinct compaction, binary search
    int *s_a = dsm, *s_b = dsm + WIN_CAP, *s_hist = dsm + 2 * WIN_CAP;
    int *buf0 = (n <= WIN_CAP) ? s_a : scratch_a + s;
    int *buf1 = (n <= WIN_CAP) ? s_b : scratch_b + s;
    const int *src = colidx + s;
    int *dst = buf0;
    int bits = 1;
    while (bits < 31 && (1ll << bits) <= (long long)cmax) ++bits;
    const int n_pass = (bits + RANK_DBITS - 1) / RANK_DBITS;
    const int dbits = (bits + n_pass - 1) / n_pass;
    for (int sh = 0; sh < bits; sh += dbits) {
      radix_pass<int, WIN_WARPS>(src, dst, n, sh, min(dbits, bits - sh), s_hist, s_aux);
      src = dst;
      dst = (dst == buf0) ? buf1 : buf0;
    }
    const int *sorted = src;
    int *uniq = dst;
    for (int base = 0; base < n; base += WIN_THREADS) {
      const int i = base + tid;
      int f = 0, val = 0;
      if (i < n) {
        val = sorted[i];
        f = (i == 0) || (sorted[i - 1] != val);
      }
      int total;
      const int pos = block_excl_scan<WIN_WARPS>(f, s_aux, total);
      if (f) uniq[n_uniq + pos] = val;
      n_uniq += total;
    }
    __syncthreads();
    for (int e = s + tid; e < t; e += WIN_THREADS) e2c[e] = lower_bound_dev(uniq, n_uniq, colidx[e]);
  }
  if (tid == 0) {
    const int nb = (n_uniq + bw - 1) / bw;
    block_partition[w] = nb;
    atomicMax(&hdr[PH_MAX_TCB], nb);
    atomicAdd(&hdr[PH_SUM_TCB], nb);
  }
  }  // windows of this CTA
}

// Phase 1 for windows of at most SMALL_N edges, one warp per window.  Column ranges up to 8192
// wide use the occupancy bitmap; wider ones a warp-private radix sort of (column - cmin).
constexpr int SR_INTS = 2 * SMALL_N + 256;

__global__ void __launch_bounds__(SW_WARPS * 32)
window_rank_small(const int *__restrict__ colidx, const int *__restrict__ rowptr, int n_nodes, int n_rw, int n_cols,
                  int bw, int *__restrict__ block_partition, int *__restrict__ e2c, int *__restrict__ e2r,
                  int *hdr, int *__restrict__ large_list) {
  __shared__ int sm[SW_WARPS][SR_INTS];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int w = blockIdx.x * SW_WARPS + warp;
  if (w >= n_rw) return;
  const int row0 = w * 16, row1 = min(row0 + 16, n_nodes);
  const int s = rowptr[row0], t = rowptr[row1];
  const int n = t - s;
  if (n > SMALL_N) {  // left to window_rank_kernel
    if (lane == 0) large_list[atomicAdd(&hdr[PH_N_LARGE], 1)] = w;
    return;
  }
  if (n <= 0) return;  // empty: block_partition[w] keeps the caller's value (src/utils.cu:141-142)
  int *a = sm[warp], *b = a + SMALL_N, *hist = b + SMALL_N;

  for (int r = row0; r < row1; ++r) {
    const int ra = rowptr[r], rb = rowptr[r + 1];
    for (int e = ra + lane; e < rb; e += 32) e2r[e] = r;
  }
  int cmin = INT_MAX, cmax = INT_MIN;
  bool bad = false;
  for (int i = lane; i < n; i += 32) {
    const int c = colidx[s + i];
    a[i] = c;
    bad |= (c < 0) | (c >= n_cols);
    cmin = min(cmin, c);
    cmax = max(cmax, c);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    cmin = min(cmin, __shfl_xor_sync(0xffffffffu, cmin, o));
    cmax = max(cmax, __shfl_xor_sync(0xffffffffu, cmax, o));
  }
  if (__any_sync(0xffffffffu, bad)) {
    if (lane == 0) atomicExch(&hdr[PH_ERROR], 1);
    return;
  }
  __syncwarp();
  const long long range = (long long)cmax - cmin;
  int n_uniq = 0;
  if (range < 256 * 32) {
    unsigned *bm = reinterpret_cast<unsigned *>(b);
    int *pre = hist;
    const int nw = (int)(range >> 5) + 1;
    for (int i = lane; i < nw; i += 32) bm[i] = 0u;
    __syncwarp();
    for (int i = lane; i < n; i += 32) {
      const int c = a[i] - cmin;
      atomicOr(&bm[c >> 5], 1u << (c & 31));
    }
    __syncwarp();
    const int per = (nw + 31) / 32;
    const int wb = min(nw, lane * per), we = min(nw, wb + per);
    int local = 0;
    for (int i = wb; i < we; ++i) local += __popc(bm[i]);
    int inc = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int x = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += x;
    }
    n_uniq = __shfl_sync(0xffffffffu, inc, 31);
    int run = inc - local;
    for (int i = wb; i < we; ++i) {
      pre[i] = run;
      run += __popc(bm[i]);
    }
    __syncwarp();
    for (int i = lane; i < n; i += 32) {
      const int c = a[i] - cmin;
      const int wi = c >> 5;
      e2c[s + i] = pre[wi] + __popc(bm[wi] & ((1u << (c & 31)) - 1u));
    }
  } else {
    for (int i = lane; i < n; i += 32) a[i] -= cmin;
    __syncwarp();
    int bits = 1;
    while (bits < 31 && (1ll << bits) <= range) ++bits;
    const int n_pass = (bits + 7) / 8;
    const int dbits = (bits + n_pass - 1) / n_pass;
    int *src = a, *dst = b;
    for (int sh = 0; sh < bits; sh += dbits) {
      warp_radix_pass<int>(src, dst, n, sh, min(dbits, bits - sh), hist);
      int *tmp = src;
      src = dst;
      dst = tmp;
    }
    for (int base = 0; base < n; base += 32) {  // distinct values of src -> dst
      const int i = base + lane;
      int val = 0;
      bool f = false;
      if (i < n) {
        val = src[i];
        f = (i == 0) || (src[i - 1] != val);
      }
      const unsigned m = __ballot_sync(0xffffffffu, f);
      if (f) dst[n_uniq + __popc(m & ((1u << lane) - 1u))] = val;
      n_uniq += __popc(m);
    }
    __syncwarp();
    for (int i = lane; i < n; i += 32) e2c[s + i] = lower_bound_dev(dst, n_uniq, colidx[s + i] - cmin);
  }
  if (lane == 0) {
    const int nb = (n_uniq + bw - 1) / bw;
    block_partition[w] = nb;
    atomicMax(&hdr[PH_MAX_TCB], nb);
    atomicAdd(&hdr[PH_SUM_TCB], nb);
  }
}

// ---- phase 2 --------------------------------------------------------------------------
// Restates generate_tcblock_rowid (src/utils.cu:53-65) and generate_tcoffset_id_atob +
// update_bitmap (src/utils.cu:23-36, 173-224).  Occupancy words and per-TCB edge counts are
// built in shared memory and stored once (windows of the CTA kernel with more than NB_CAP TC
// blocks use global atomics on zeroed outputs instead).  The tile ids are regrouped by TCB (CSR
// order inside a TCB) with a stable radix sort on the TCB bits.
//
// CTA per window (windows with more than SMALL_N edges, taken from the list window_fill_small
// builds).  Windows of up to FILL_STAGE_MAX edges take their TC blocks NB_CAP at a time and make one
// walk over their edges per range (column list and occupancy words in shared memory); sorted rows
// need nothing else, unsorted ones of up to FILL_KREG * FILL_THREADS edges and NB_CAP TC blocks keep
// their (TCB id, tile id) words in registers for a single stable radix pass.  Everything else takes
// the general path: the words go through the workspace (L2) and a multi-pass radix sort.
constexpr int NB_CAP = 1024;
constexpr int FILL_THREADS = 512;
constexpr int FILL_WARPS = FILL_THREADS / 32;
constexpr int FILL_DBITS = 10;  // NB_CAP TC blocks in one pass
constexpr int FILL_KREG = 32;   // edges per thread on the one-pass path
constexpr int FILL_AHEAD = 8;   // steps of the edge walk whose loads are in flight together
constexpr int FILL_HIST_INTS = FILL_WARPS << FILL_DBITS;
constexpr int FILL_SMEM_BYTES = (FILL_HIST_INTS + NB_CAP) * (int)sizeof(int) + NB_CAP * 4 * 8;
static_assert((1 << FILL_DBITS) >= NB_CAP, "one radix pass must cover every TCB id of the one-pass path");
constexpr int FILL_STAGE_MAX = FILL_HIST_INTS * (int)sizeof(int) - 16;  // tile bytes of one window, staged with a skew
static_assert(FILL_KREG * FILL_THREADS + 16 <= NB_CAP * 4 * 8, "the staged tile bytes (and their skew) reuse the occupancy words' memory");

// Row (0..15) of edge e inside a window whose 17 row pointers are rp: the last row that starts at or before e
// (empty rows share a pointer with their successor and are skipped).
__device__ __forceinline__ int row_of_edge(const int *rp, int e) {
  int r = 0;
  if (rp[r + 8] <= e) r += 8;
  if (rp[r + 4] <= e) r += 4;
  if (rp[r + 2] <= e) r += 2;
  if (rp[r + 1] <= e) r += 1;
  return r;
}

// What a CTA of window_fill_kernel needs to know about entry li of its window list (nothing is loaded past the list).
struct FillWindow {
  int w, s, n, tcb0, nb;
};
__device__ __forceinline__ FillWindow fill_window(int li, int n_large, const int *__restrict__ large_list,
                                                  const int *__restrict__ rowptr, const int *__restrict__ rwo,
                                                  int n_nodes) {
  FillWindow f = {0, 0, 0, 0, 0};
  if (li < n_large) {
    f.w = large_list[li];
    const int row0 = f.w * 16, row1 = min(row0 + 16, n_nodes);
    f.s = rowptr[row0];
    f.n = rowptr[row1] - f.s;
    f.tcb0 = rwo[f.w];
    f.nb = rwo[f.w + 1] - f.tcb0;
  }
  return f;
}

// Tile ids (row * BW + column) of the occupied positions of one TC block in row-major order, from its
// occupancy words: word (c / 8) * (BW / 8) + (r / 8) holds position (r, c) at bit 63 - ((r % 8) * 8 + c % 8),
// i.e. byte 7 - r % 8 of a word is the 8-column strip of row r, column 0 in its top bit.  The strips are
// regrouped into 32-bit words of consecutive positions (top bit first), so that the tile id of a set bit is
// 32 * word + count of leading zeros.
template <int BW>
__device__ __forceinline__ unsigned char *tile_bytes_of_block(const unsigned long long (&wv)[4], unsigned char *out) {
  constexpr int NW = 16 * BW / 32;
  unsigned m[NW];
  if (BW == 16) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {  // rows 8h .. 8h+7: left strips in wv[h], right strips in wv[2 + h]
      const unsigned l_hi = (unsigned)(wv[h] >> 32), l_lo = (unsigned)wv[h];
      const unsigned r_hi = (unsigned)(wv[2 + h] >> 32), r_lo = (unsigned)wv[2 + h];
      m[4 * h + 0] = __byte_perm(l_hi, r_hi, 0x3726);  // rows 8h, 8h+1
      m[4 * h + 1] = __byte_perm(l_hi, r_hi, 0x1504);  // rows 8h+2, 8h+3
      m[4 * h + 2] = __byte_perm(l_lo, r_lo, 0x3726);
      m[4 * h + 3] = __byte_perm(l_lo, r_lo, 0x1504);
    }
  } else {
#pragma unroll
    for (int h = 0; h < 2; ++h) {  // 8-wide blocks: a word already holds rows 8h .. 8h+7 in row-major order
      m[2 * h + 0] = (unsigned)(wv[h] >> 32);
      m[2 * h + 1] = (unsigned)wv[h];
    }
  }
#pragma unroll
  for (int k = 0; k < NW; ++k) {
    unsigned x = m[k];
    while (x) {
      const int z = __clz(x);
      *out++ = (unsigned char)(32 * k + z);
      x &= ~(0x80000000u >> z);
    }
  }
  return out;
}

__global__ void __launch_bounds__(FILL_THREADS, 2)  // two CTAs per SM: 64 registers, 100 KB of shared memory each
window_fill_kernel(const int *__restrict__ colidx, const int *__restrict__ rowptr, int n_nodes, int n_rw, int bw,
                   const int *__restrict__ e2c, const int *__restrict__ e2r, const int *__restrict__ rwo,
                   const int *__restrict__ large_list, int *hdr, int *__restrict__ tcb_rowid,
                   unsigned char *__restrict__ tile_id, int *__restrict__ tcb_off, int *__restrict__ atox,
                   unsigned long long *__restrict__ bitmap, int *scratch_a, int *scratch_b) {
  extern __shared__ __align__(16) int dsm[];
  __shared__ int s_aux[33];
  __shared__ int s_rp2[2][17];  // row pointers of the current and of the next window: the row of an edge follows
                                // from its position
  __shared__ int s_pull;
  int *s_hist = dsm, *s_cnt = s_hist + FILL_HIST_INTS;
  unsigned long long *s_bmp = reinterpret_cast<unsigned long long *>(s_cnt + NB_CAP);
  unsigned *s_bmp32 = reinterpret_cast<unsigned *>(s_bmp);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n_large = hdr[PH_N_LARGE_FILL];
  const int wpt = 16 * bw / 64;
  const int sub_per_col = bw / 8;
  const int lbw = (bw == 16) ? 4 : 3;
  const bool vec16 = ((reinterpret_cast<uintptr_t>(bitmap) | reinterpret_cast<uintptr_t>(atox)) & 15) == 0;
  // A CTA pulls its windows from a counter (they differ in size by 10x), two ahead: while window k is worked
  // on, the header and the row pointers of window k+1 are loaded and its slices of edgeToColumn and colIdx are
  // requested into L2 (the walk over a window's edges otherwise pays DRAM latency per step), and the counter is
  // read for window k+2 -- none of these round trips is waited for.
  if (tid == 0) s_pull = atomicAdd(&hdr[PH_FILL_NEXT], 2);
  __syncthreads();
  int li = s_pull, li_next = li + 1, pulled = 0, buf = 0;
  FillWindow cur = fill_window(li, n_large, large_list, rowptr, rwo, n_nodes), ahead = cur;
  if (tid < 17 && li < n_large) s_rp2[0][tid] = rowptr[min(cur.w * 16 + tid, n_nodes)];
  bool staged = true;
  auto stage_next = [&]() {  // what the next window needs from memory, asked for while this one is worked on
    if (staged) return;
    staged = true;
    prefetch_l2_lines(e2c + ahead.s, ahead.n, tid, FILL_THREADS);
    prefetch_l2_lines(colidx + ahead.s, ahead.n, tid, FILL_THREADS);
    if (tid < 17 && li_next < n_large) s_rp2[buf ^ 1][tid] = rowptr[min(ahead.w * 16 + tid, n_nodes)];
  };
  auto advance = [&]() {
    stage_next();
    if (tid == 0) s_pull = pulled;
    __syncthreads();
    li = li_next;
    li_next = s_pull;
    cur = ahead;
    buf ^= 1;
  };
  for (;; advance()) {
    __syncthreads();  // the previous window's shared memory (and s_pull) is no longer read
    if (li >= n_large) break;
    if (tid == 0) pulled = atomicAdd(&hdr[PH_FILL_NEXT], 1);  // consumed in advance()
    ahead = fill_window(li_next, n_large, large_list, rowptr, rwo, n_nodes);  // consumed in stage_next()
    staged = false;
    const int *s_rp = s_rp2[buf];
    const int w = cur.w, s = cur.s, n = cur.n, tcb0 = cur.tcb0, nb = cur.nb;
    const int tcb1 = tcb0 + nb;
    if (nb <= 0) continue;
    const bool in_smem = nb <= NB_CAP;
    int bits = 0;
    while ((1 << bits) < nb) ++bits;
    for (int i = tid; i < nb; i += FILL_THREADS) tcb_rowid[tcb0 + i] = w;

    if (n <= FILL_STAGE_MAX) {
      // Common case.  The window's TC blocks are taken NB_CAP at a time (nearly always all at once); for every
      // such range one walk over the window's edges builds the column list and the occupancy words in shared
      // memory.  If every row's columns ascend strictly (checked in the first walk), the CSR order of the edges
      // inside a TC block is the row-major order of its occupancy bits, so the tile ids and the per-block edge
      // counts follow from the occupancy words alone: one thread per TC block, no second walk, no sort.
      int *s_atox = s_hist;  // at most NB_CAP * 16 = FILL_HIST_INTS column slots
      bool slow = false;
      int edges_done = 0;
      const int per = ((n + FILL_WARPS - 1) / FILL_WARPS + 31) & ~31;
      const int beg = min(n, warp * per), end = min(n, beg + per);
      for (int tl0 = 0; tl0 < nb; tl0 += NB_CAP) {
        const int nbc = min(NB_CAP, nb - tl0);
        if (tl0 > 0) __syncthreads();  // the previous range's tile bytes have left
        {
          uint4 *z = reinterpret_cast<uint4 *>(s_bmp);  // an even number of 64-bit words per TC block
          for (int i = tid; i < nbc * wpt / 2; i += FILL_THREADS) z[i] = make_uint4(0u, 0u, 0u, 0u);
          // every column slot is written by at least one edge, but for the unused ones of the last block: they read 0
          if (tl0 + nbc == nb && tid < bw) s_atox[(nbc - 1) * bw + tid] = 0;
        }
        __syncthreads();
        // Warp `warp` walks the contiguous slice [beg, end) of the window's edges, 32 at a time: a lane's edges
        // ascend, so its row only moves forward (rp_r, nxt: the pointers of its row and of the next one), and the
        // edge before lane 0's is lane 31's of the previous step.
        bool unsorted = false;
        int r = 0, rp_r = s_rp[0], nxt = s_rp[1];
        int prev_last = (beg > 0 && beg < end) ? e2c[s + beg - 1] : -1;
        for (int i0 = beg; i0 < end; i0 += 32 * FILL_AHEAD) {  // warp-uniform bounds: the shuffles below are full-warp
          int rk[FILL_AHEAD], cl[FILL_AHEAD];
#pragma unroll
          for (int u = 0; u < FILL_AHEAD; ++u) {  // all loads of FILL_AHEAD steps are in flight before the first use
            const int e = s + min(i0 + 32 * u + lane, end - 1);
            rk[u] = e2c[e];
            cl[u] = colidx[e];
          }
#pragma unroll
          for (int u = 0; u < FILL_AHEAD; ++u) {
            if (i0 + 32 * u >= end) break;
            const int i = i0 + 32 * u + lane;
            const bool valid = i < end;
            const int e = s + i;
            const int rank = rk[u];
            int prev = __shfl_up_sync(0xffffffffu, rank, 1);
            if (lane == 0) prev = prev_last;
            prev_last = __shfl_sync(0xffffffffu, rank, 31);
            const int tl = (rank >> lbw) - tl0, c = rank & (bw - 1);
            if (valid) {
              while (nxt <= e) {  // s_rp[16] is the window's end: never reached
                rp_r = nxt;
                ++r;
                nxt = s_rp[r + 1];
              }
              unsorted |= (e > rp_r) & (prev >= rank);
              if ((unsigned)tl < (unsigned)nbc) {
                s_atox[(tl << lbw) + c] = cl[u];
                // 32-bit half and bit of position (r, c): word (c / 8) * (bw / 8) + r / 8, bit 63 - ((r % 8) * 8 + c % 8)
                const int half = ((tl * wpt + (c >> 3) * sub_per_col + (r >> 3)) << 1) + 1 - ((r >> 2) & 1);
                atomicOr(&s_bmp32[half], 0x80000000u >> (((r & 3) << 3) + (c & 7)));
              }
            }
          }
        }
        if (tl0 == 0) {
          slow = __syncthreads_or(unsorted);
          stage_next();
          if (slow && !(in_smem && n <= FILL_KREG * FILL_THREADS)) break;  // left to the general path
        } else {
          __syncthreads();
        }
        {  // both lists start on a 16-byte boundary in shared and in global memory and hold a multiple of 16 bytes
          const size_t g0 = (size_t)tcb0 + tl0;
          if (vec16) {
            const uint4 *sb = reinterpret_cast<const uint4 *>(s_bmp), *sa = reinterpret_cast<const uint4 *>(s_atox);
            uint4 *gb = reinterpret_cast<uint4 *>(bitmap + g0 * wpt);
            uint4 *ga = reinterpret_cast<uint4 *>(atox + g0 * bw);
            for (int i = tid; i < nbc * wpt / 2; i += FILL_THREADS) gb[i] = sb[i];
            for (int i = tid; i < nbc * bw / 4; i += FILL_THREADS) ga[i] = sa[i];
          } else {  // output arrays that do not start on a 16-byte boundary
            for (int i = tid; i < nbc * wpt; i += FILL_THREADS) bitmap[g0 * wpt + i] = s_bmp[i];
            for (int i = tid; i < nbc * bw; i += FILL_THREADS) atox[g0 * bw + i] = s_atox[i];
          }
        }
        // The tile bytes are staged at the offset that gives them the alignment (mod 16) of their place in
        // tcblocktile_id, so that all but the ragged ends leave as 16-byte stores.
        unsigned char *gt = tile_id + s + edges_done;
        const int skew = (int)(reinterpret_cast<uintptr_t>(gt) & 15);
        unsigned char *stage;
        int n_stage;

        if (!slow) {
          __syncthreads();  // the column list has left; its memory takes the staged tile bytes
          stage = reinterpret_cast<unsigned char *>(s_hist) + skew;
          int carry = 0;
          for (int base = 0; base < nbc; base += FILL_THREADS) {
            const int d = base + tid;
            unsigned long long wv[4] = {0ull, 0ull, 0ull, 0ull};
            int cnt = 0;
            if (d < nbc) {
#pragma unroll
              for (int k = 0; k < 4; ++k)
                if (k < wpt) {
                  wv[k] = s_bmp[d * wpt + k];
                  cnt += __popcll(wv[k]);
                }
              tcb_off[1 + tcb0 + tl0 + d] = cnt;  // edges of the TC block (scanned into offsets afterwards)
            }
            int total;
            const int off = carry + block_excl_scan<FILL_WARPS>(cnt, s_aux, total);
            carry += total;
            if (cnt > 0) {
              if (bw == 16) tile_bytes_of_block<16>(wv, stage + off);
              else tile_bytes_of_block<8>(wv, stage + off);
            }
          }
          n_stage = carry;
        } else {
          // Unsorted rows or repeated edges, window small enough for registers: stable single-pass radix sort
          // of the (TC block, tile id) words on the TC-block bits.  (Here the range is the whole window.)
          const int nd = 1 << bits;
          __syncthreads();  // the column list has left; its memory takes the histograms
          for (int i = tid; i < FILL_WARPS * nd; i += FILL_THREADS) s_hist[i] = 0;
          __syncthreads();
          // the same slices as above (CSR order), lane l of a warp the elements beg + 32 j + l: the order the
          // stable scatter below relies on
          int *myh = s_hist + warp * nd;
          int keys[FILL_KREG];
#pragma unroll
          for (int j = 0; j < FILL_KREG; ++j) {
            const int i = beg + j * 32 + lane;
            keys[j] = -1;
            if (i < end) {
              const int e = s + i;
              const int rank = e2c[e];
              const int tl = rank >> lbw, c = rank & (bw - 1);
              const int r = row_of_edge(s_rp, e);
              atomicAdd(&myh[tl], 1);  // the per-TCB edge counts are the column sums of these histograms
              keys[j] = (tl << 8) | ((r << lbw) + c);
            }
          }
          __syncthreads();
          {  // TCB-major, warp-minor exclusive offsets of the per-warp histograms
            int carry = 0;
            for (int base = 0; base < nd; base += FILL_THREADS) {
              const int d = base + tid;
              int tot = 0;
              if (d < nd)
                for (int x = 0; x < FILL_WARPS; ++x) tot += s_hist[x * nd + d];
              if (d < nb) tcb_off[1 + tcb0 + d] = tot;  // edges of TC block d (scanned into offsets afterwards)
              int total;
              int run = carry + block_excl_scan<FILL_WARPS>(tot, s_aux, total);
              if (d < nd)
                for (int x = 0; x < FILL_WARPS; ++x) {
                  const int v = s_hist[x * nd + d];
                  s_hist[x * nd + d] = run;
                  run += v;
                }
              carry += total;
            }
          }
          __syncthreads();  // offsets complete; the occupancy words have been stored, their memory is reused
          stage = reinterpret_cast<unsigned char *>(s_bmp) + skew;
#pragma unroll
          for (int j = 0; j < FILL_KREG; ++j) {
            if (beg + j * 32 >= end) break;  // warp-uniform
            const int key = keys[j];
            const bool valid = key >= 0;
            const unsigned d = (unsigned)key >> 8;
            const unsigned peers = same_digit_lanes(d, valid);
            const int rank = __popc(peers & ((1u << lane) - 1u));
            const int base = valid ? myh[d] : 0;
            __syncwarp();
            if (valid) {
              stage[base + rank] = (unsigned char)(key & 255);
              if (lane == __ffs(peers) - 1) myh[d] = base + __popc(peers);
            }
            __syncwarp();
          }
          n_stage = n;
        }
        __syncthreads();
        {
          const int head = min(n_stage, (16 - skew) & 15);  // bytes before the first 16-byte boundary of the output
          const int n16 = (n_stage - head) >> 4;
          if (tid < head) gt[tid] = stage[tid];
          const uint4 *sv = reinterpret_cast<const uint4 *>(stage + head);
          uint4 *gv = reinterpret_cast<uint4 *>(gt + head);
          for (int i = tid; i < n16; i += FILL_THREADS) gv[i] = sv[i];
          const int done = head + (n16 << 4);
          if (tid < n_stage - done) gt[done + tid] = stage[done + tid];
        }
        edges_done += n_stage;
      }
      if (!slow || (in_smem && n <= FILL_KREG * FILL_THREADS)) continue;
    }

    // ---- general path: windows of more than FILL_STAGE_MAX edges, and unsorted ones too large for registers
    __syncthreads();
    if (in_smem) {
      for (int i = tid; i < nb; i += FILL_THREADS) s_cnt[i] = 0;
      for (int i = tid; i < nb * wpt; i += FILL_THREADS) s_bmp[i] = 0ull;
    } else {
      for (int i = tid; i < nb; i += FILL_THREADS) tcb_off[1 + tcb0 + i] = 0;
      for (int i = tid; i < nb * wpt; i += FILL_THREADS) bitmap[(size_t)tcb0 * wpt + i] = 0ull;
    }
    // every TCB but the last is full; the last one's unused column slots read 0
    for (int i = tid; i < bw; i += FILL_THREADS) atox[(size_t)(tcb1 - 1) * bw + i] = 0;
    __syncthreads();
    int *buf0 = scratch_a + s, *buf1 = scratch_b + s;
    for (int i = tid; i < n; i += FILL_THREADS) {
      const int e = s + i;
      const int rank = e2c[e];
      const int tl = rank >> lbw, c = rank & (bw - 1);
      const int r = e2r[e] & 15;
      const size_t tg = (size_t)tcb0 + tl;
      atox[(tg << lbw) + c] = colidx[e];
      const int sub = (c >> 3) * sub_per_col + (r >> 3);
      const int bitpos = 63 - ((r & 7) * 8 + (c & 7));
      if (in_smem) {  // 32-bit halves of the 64-bit words: native shared-memory atomics
        atomicOr(&s_bmp32[((tl * wpt + sub) << 1) + (bitpos >> 5)], 1u << (bitpos & 31));
        atomicAdd(&s_cnt[tl], 1);
      } else {
        atomicOr(&bitmap[tg * wpt + sub], 1ull << bitpos);
        atomicAdd(&tcb_off[1 + tg], 1);
      }
      buf0[i] = (tl << 8) | ((r << lbw) + c);
    }
    __syncthreads();
    if (in_smem) {
      for (int i = tid; i < nb; i += FILL_THREADS) tcb_off[1 + tcb0 + i] = s_cnt[i];
      for (int i = tid; i < nb * wpt; i += FILL_THREADS) bitmap[(size_t)tcb0 * wpt + i] = s_bmp[i];
    }
    const int n_pass = (bits + FILL_DBITS - 1) / FILL_DBITS;
    const int dbits = n_pass > 0 ? (bits + n_pass - 1) / n_pass : 0;
    const int *src = buf0;
    int *dst = buf1;
    for (int sh = 0; sh < bits; sh += dbits) {
      radix_pass<int, FILL_WARPS>(src, dst, n, 8 + sh, min(dbits, bits - sh), s_hist, s_aux);
      const int *tsrc = src;
      src = dst;
      dst = const_cast<int *>(tsrc);
    }
    for (int i = tid; i < n; i += FILL_THREADS) tile_id[s + i] = (unsigned char)(src[i] & 255);
  }
}

// Warp per window, windows of at most SMALL_N edges (hence at most SMALL_N / 8 TC blocks).
constexpr int SF_NB = SMALL_N / 8;
constexpr int SF_INTS = 2 * SMALL_N + SF_NB + SF_NB + 2 * 128;  // buffers, histogram, counts, 128 occupancy words
static_assert(SF_NB * 2 <= 128 && (SF_NB / 2) * 4 <= 128, "occupancy words of a small window");
static_assert((2 * SMALL_N + 2 * SF_NB) % 2 == 0 && SF_INTS % 2 == 0, "64-bit alignment of the occupancy words");

__global__ void __launch_bounds__(SW_WARPS * 32)
window_fill_small(const int *__restrict__ colidx, const int *__restrict__ rowptr, int n_nodes, int n_rw, int bw,
                  const int *__restrict__ e2c, const int *__restrict__ e2r, const int *__restrict__ rwo,
                  int *__restrict__ tcb_rowid, unsigned char *__restrict__ tile_id, int *__restrict__ tcb_off,
                  int *__restrict__ atox, unsigned long long *__restrict__ bitmap, int *hdr,
                  int *__restrict__ large_list) {
  __shared__ __align__(8) int sm[SW_WARPS][SF_INTS];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int w = blockIdx.x * SW_WARPS + warp;
  if (w >= n_rw) return;
  if (w == 0 && lane == 0) tcb_off[0] = 0;
  const int row0 = w * 16, row1 = min(row0 + 16, n_nodes);
  const int s = rowptr[row0], t = rowptr[row1];
  const int n = t - s;
  if (n > SMALL_N) {  // left to window_fill_kernel
    if (lane == 0) large_list[atomicAdd(&hdr[PH_N_LARGE_FILL], 1)] = w;
    return;
  }
  if (n <= 0) return;
  const int tcb0 = rwo[w], tcb1 = rwo[w + 1];
  const int nb = tcb1 - tcb0;
  if (nb <= 0) return;
  int *buf0 = sm[warp], *buf1 = buf0 + SMALL_N, *hist = buf1 + SMALL_N, *cnt = hist + SF_NB;
  unsigned long long *bmp = reinterpret_cast<unsigned long long *>(cnt + SF_NB);
  const int wpt = 16 * bw / 64;
  for (int i = lane; i < nb; i += 32) {
    tcb_rowid[tcb0 + i] = w;
    cnt[i] = 0;
  }
  for (int i = lane; i < nb * wpt; i += 32) bmp[i] = 0ull;
  for (int i = lane; i < bw; i += 32) atox[(size_t)(tcb1 - 1) * bw + i] = 0;
  __syncwarp();
  const int sub_per_col = bw / 8;
  const int lbw = (bw == 16) ? 4 : 3;
  unsigned *bmp32 = reinterpret_cast<unsigned *>(bmp);
  for (int i = lane; i < n; i += 32) {
    const int e = s + i;
    const int rank = e2c[e];
    const int tl = rank >> lbw, c = rank & (bw - 1);
    const int r = e2r[e] & 15;
    atox[(((size_t)tcb0 + tl) << lbw) + c] = colidx[e];
    const int sub = (c >> 3) * sub_per_col + (r >> 3);
    const int bitpos = 63 - ((r & 7) * 8 + (c & 7));
    atomicOr(&bmp32[((tl * wpt + sub) << 1) + (bitpos >> 5)], 1u << (bitpos & 31));
    atomicAdd(&cnt[tl], 1);
    buf0[i] = (tl << 8) | ((r << lbw) + c);
  }
  __syncwarp();
  for (int i = lane; i < nb; i += 32) tcb_off[1 + tcb0 + i] = cnt[i];
  for (int i = lane; i < nb * wpt; i += 32) bitmap[(size_t)tcb0 * wpt + i] = bmp[i];
  int bits = 0;
  while ((1 << bits) < nb) ++bits;  // <= 6
  const int *src = buf0;
  if (bits > 0) {
    warp_radix_pass<int>(buf0, buf1, n, 8, bits, hist);
    src = buf1;
  }
  __syncwarp();
  for (int i = lane; i < n; i += 32) tile_id[s + i] = (unsigned char)(src[i] & 255);
}

// ---- scans ----------------------------------------------------------------------------
// In-place inclusive scan of x[0..n): three launches (tile sums, scan of the sums, apply).
constexpr int SCAN_THREADS = 1024;
constexpr int SCAN_ITEMS = 4;
constexpr int SCAN_TILE = SCAN_THREADS * SCAN_ITEMS;

__global__ void __launch_bounds__(SCAN_THREADS) scan_tile_sums(const int *__restrict__ x, long long n, int *sums) {
  __shared__ int aux[33];
  const long long base = (long long)blockIdx.x * SCAN_TILE + threadIdx.x * SCAN_ITEMS;
  int v = 0;
#pragma unroll
  for (int j = 0; j < SCAN_ITEMS; ++j)
    if (base + j < n) v += x[base + j];
  int total;
  block_excl_scan<SCAN_THREADS / 32>(v, aux, total);
  if (threadIdx.x == 0) sums[blockIdx.x] = total;
}

__global__ void __launch_bounds__(SCAN_THREADS) scan_sums(int *sums, int n_tiles) {
  __shared__ int aux[33];
  int running = 0;
  for (int base = 0; base < n_tiles; base += SCAN_THREADS) {
    const int i = base + threadIdx.x;
    const int v = (i < n_tiles) ? sums[i] : 0;
    int total;
    const int ex = block_excl_scan<SCAN_THREADS / 32>(v, aux, total);
    if (i < n_tiles) sums[i] = running + ex;  // exclusive prefix of the tile sums
    running += total;
  }
}

__global__ void __launch_bounds__(SCAN_THREADS) scan_apply(int *x, long long n, const int *sums) {
  __shared__ int aux[33];
  const long long base = (long long)blockIdx.x * SCAN_TILE + threadIdx.x * SCAN_ITEMS;
  int v[SCAN_ITEMS];
  int sum = 0;
#pragma unroll
  for (int j = 0; j < SCAN_ITEMS; ++j) {
    v[j] = (base + j < n) ? x[base + j] : 0;
    sum += v[j];
  }
  int total;
  int run = block_excl_scan<SCAN_THREADS / 32>(sum, aux, total) + sums[blockIdx.x];
#pragma unroll
  for (int j = 0; j < SCAN_ITEMS; ++j) {
    run += v[j];
    if (base + j < n) x[base + j] = run;
  }
}

__global__ void copy_shifted(const int *__restrict__ in, int *__restrict__ out, int n) {
  // out[0] = 0, out[1 + i] = in[i]
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i == 0) out[0] = 0;
  if (i < n) out[1 + i] = in[i];
}

static int inclusive_scan_inplace(int *x, long long n, int *tile_sums, cudaStream_t stream) {
  if (n <= 0) return F3S_OK;
  const int n_tiles = (int)((n + SCAN_TILE - 1) / SCAN_TILE);
  scan_tile_sums<<<n_tiles, SCAN_THREADS, 0, stream>>>(x, n, tile_sums);
  scan_sums<<<1, SCAN_THREADS, 0, stream>>>(tile_sums, n_tiles);
  scan_apply<<<n_tiles, SCAN_THREADS, 0, stream>>>(x, n, tile_sums);
  note_launches(2);
  F3S_CHECK_LAUNCH();
  return F3S_OK;
}

// ---- schedule -------------------------------------------------------------------------
// Windows by TCB count, descending, ties by ascending window id (the order the reference
// gets from thrust::sort_by_key with thrust::greater, src/utils.cu:400-436).  One CTA;
// words are (max_count - count) << 32 | window, sorted on the count bits only -- the sort
// is stable and the ids start ascending, so ties stay in id order.
__global__ void __launch_bounds__(SCHED_THREADS)
schedule_kernel(const int *__restrict__ rwo, int n_rw, int *__restrict__ sorted_rw, unsigned long long *buf0,
                unsigned long long *buf1) {
  __shared__ int s_hist[SCHED_WARPS * 256];
  __shared__ int s_aux[33];
  __shared__ int s_max;
  const int tid = threadIdx.x;
  if (tid == 0) s_max = 0;
  __syncthreads();
  int mx = 0;
  for (int i = tid; i < n_rw; i += SCHED_THREADS) mx = max(mx, rwo[i + 1] - rwo[i]);
  atomicMax(&s_max, mx);
  __syncthreads();
  const int maxc = s_max;
  for (int i = tid; i < n_rw; i += SCHED_THREADS)
    buf0[i] = ((unsigned long long)(unsigned)(maxc - (rwo[i + 1] - rwo[i])) << 32) | (unsigned)i;
  __syncthreads();
  int bits = 0;
  while (bits < 31 && (1ll << bits) <= (long long)maxc) ++bits;
  const unsigned long long *src = buf0;
  unsigned long long *dst = buf1;
  for (int sh = 0; sh < bits; sh += 8) {
    radix_pass<unsigned long long, SCHED_WARPS, 8>(src, dst, n_rw, 32 + sh, 8, s_hist, s_aux);
    const unsigned long long *tsrc = src;
    src = dst;
    dst = const_cast<unsigned long long *>(tsrc);
  }
  for (int i = tid; i < n_rw; i += SCHED_THREADS) sorted_rw[i] = (int)(src[i] & 0xffffffffull);
}

struct PreWs {
  size_t off_hdr, off_a, off_b, off_sums, off_s0, off_s1, off_list, total;
};

static PreWs pre_ws(long long n_nodes, long long nnz) {
  PreWs L;
  const long long n_rw = (n_nodes + 15) / 16;
  size_t off = 0;
  L.off_hdr = off; off = align_up(off + PH_INTS * sizeof(int), 256);
  L.off_a = off; off = align_up(off + (size_t)nnz * sizeof(int), 256);
  L.off_b = off; off = align_up(off + (size_t)nnz * sizeof(int), 256);
  const long long longest = (nnz > n_rw ? nnz : n_rw) + 1;
  L.off_sums = off; off = align_up(off + (size_t)(longest / SCAN_TILE + 2) * sizeof(int), 256);
  L.off_s0 = off; off = align_up(off + (size_t)n_rw * sizeof(unsigned long long), 256);
  L.off_s1 = off; off = align_up(off + (size_t)n_rw * sizeof(unsigned long long), 256);
  L.off_list = off; off = align_up(off + (size_t)n_rw * sizeof(int), 256);  // windows left to the CTA-per-window kernels
  L.total = off;
  return L;
}

}  // namespace f3s

using namespace f3s;

extern "C" size_t f3s_preprocess_workspace_bytes(int64_t num_nodes, int64_t nnz, int block_w) {
  if (num_nodes < 0 || nnz < 0 || (block_w != 8 && block_w != 16)) return 0;
  return pre_ws(num_nodes, nnz).total;
}

static int check_pre_args(int32_t num_nodes, int64_t nnz, int32_t block_h, int32_t block_w, const void *ws,
                          size_t ws_bytes) {
  F3S_REQUIRE(num_nodes >= 0 && nnz >= 0, F3S_ERR_INVALID_ARG, "negative size");
  F3S_REQUIRE(nnz < (1ll << 31), F3S_ERR_UNSUPPORTED, "nnz exceeds int32");
  F3S_REQUIRE(block_h == 16, F3S_ERR_UNSUPPORTED, "block_h must be 16, got %d", block_h);
  F3S_REQUIRE(block_w == 8 || block_w == 16, F3S_ERR_UNSUPPORTED, "block_w must be 8 or 16, got %d", block_w);
  F3S_REQUIRE(ws != nullptr && (reinterpret_cast<uintptr_t>(ws) & 255) == 0, F3S_ERR_WORKSPACE,
              "workspace must be non-null and 256-byte aligned");
  F3S_REQUIRE(ws_bytes >= pre_ws(num_nodes, nnz).total, F3S_ERR_WORKSPACE, "workspace too small: %zu < %zu",
              ws_bytes, pre_ws(num_nodes, nnz).total);
  return F3S_OK;
}

extern "C" int f3s_preprocess_count_rect(const int32_t *colidx, const int32_t *rowptr, int32_t num_nodes,
                                         int32_t num_cols, int64_t nnz, int32_t block_h, int32_t block_w,
                                         int32_t *block_partition, int32_t *edge_to_column, int32_t *edge_to_row,
                                         int32_t *row_window_offset, void *workspace, size_t workspace_bytes,
                                         int32_t *n_tcb_host, int32_t *max_tcb_per_window_host,
                                         f3s_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  F3S_REQUIRE(num_cols >= 0, F3S_ERR_INVALID_ARG, "negative num_cols");
  if (int rc = check_pre_args(num_nodes, nnz, block_h, block_w, workspace, workspace_bytes)) return rc;
  F3S_REQUIRE(n_tcb_host && max_tcb_per_window_host, F3S_ERR_INVALID_ARG, "null host output pointer");
  F3S_REQUIRE(row_window_offset && rowptr, F3S_ERR_INVALID_ARG, "null pointer argument");
  F3S_REQUIRE(nnz == 0 || (colidx && edge_to_column && edge_to_row), F3S_ERR_INVALID_ARG, "null edge array");
  const int n_rw = (num_nodes + 15) / 16;
  F3S_REQUIRE(n_rw == 0 || block_partition, F3S_ERR_INVALID_ARG, "null block_partition");
  const PreWs L = pre_ws(num_nodes, nnz);
  unsigned char *ws = static_cast<unsigned char *>(workspace);
  int *hdr = reinterpret_cast<int *>(ws + L.off_hdr);
  F3S_CUDA_TRY(cudaMemsetAsync(hdr, 0, PH_INTS * sizeof(int), stream));
  if (n_rw > 0) {
    int *large_list = reinterpret_cast<int *>(ws + L.off_list);
    window_rank_small<<<(n_rw + SW_WARPS - 1) / SW_WARPS, SW_WARPS * 32, 0, stream>>>(
        colidx, rowptr, num_nodes, n_rw, num_cols, block_w, block_partition, edge_to_column, edge_to_row, hdr,
        large_list);
    F3S_CHECK_LAUNCH();
    F3S_CUDA_TRY(cudaFuncSetAttribute(window_rank_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, RANK_SMEM_BYTES));
    window_rank_kernel<<<min(n_rw, sm_count() * 3), WIN_THREADS, RANK_SMEM_BYTES, stream>>>(
        colidx, rowptr, num_nodes, num_cols, block_w, large_list, block_partition, edge_to_column, edge_to_row,
        reinterpret_cast<int *>(ws + L.off_a), reinterpret_cast<int *>(ws + L.off_b), hdr);
    F3S_CHECK_LAUNCH();
    copy_shifted<<<(n_rw + 255) / 256, 256, 0, stream>>>(block_partition, row_window_offset, n_rw);
    F3S_CHECK_LAUNCH();
    if (int rc = inclusive_scan_inplace(row_window_offset + 1, n_rw, reinterpret_cast<int *>(ws + L.off_sums), stream))
      return rc;
  } else {
    F3S_CUDA_TRY(cudaMemsetAsync(row_window_offset, 0, sizeof(int), stream));
  }
  int host_hdr[PH_INTS];
  int scanned_total = 0;
  F3S_CUDA_TRY(cudaMemcpyAsync(host_hdr, hdr, sizeof(host_hdr), cudaMemcpyDeviceToHost, stream));
  F3S_CUDA_TRY(cudaMemcpyAsync(&scanned_total, row_window_offset + n_rw, sizeof(int), cudaMemcpyDeviceToHost, stream));
  F3S_CUDA_TRY(cudaStreamSynchronize(stream));
  F3S_REQUIRE(host_hdr[PH_ERROR] == 0, F3S_ERR_INVALID_ARG, "colidx holds a value outside [0, %d)", num_cols);
  // Windows without edges keep the caller's block_partition entry (as src/utils.cu:141-142 does), so a
  // caller that did not zero the array gets offsets that disagree with the TCB count; every array sized
  // by that count would then be overrun by the second phase.  Refuse instead.
  F3S_REQUIRE(scanned_total == host_hdr[PH_SUM_TCB], F3S_ERR_INVALID_ARG,
              "block_partition was not zeroed by the caller: its entries for row windows without edges add %d "
              "TC blocks that do not exist", scanned_total - host_hdr[PH_SUM_TCB]);
  *n_tcb_host = host_hdr[PH_SUM_TCB];
  *max_tcb_per_window_host = host_hdr[PH_MAX_TCB];
  return F3S_OK;
}

extern "C" int f3s_preprocess_count(const int32_t *colidx, const int32_t *rowptr, int32_t num_nodes, int64_t nnz,
                                    int32_t block_h, int32_t block_w, int32_t *block_partition,
                                    int32_t *edge_to_column, int32_t *edge_to_row, int32_t *row_window_offset,
                                    void *workspace, size_t workspace_bytes, int32_t *n_tcb_host,
                                    int32_t *max_tcb_per_window_host, f3s_stream_t stream) {
  return f3s_preprocess_count_rect(colidx, rowptr, num_nodes, num_nodes, nnz, block_h, block_w, block_partition,
                                   edge_to_column, edge_to_row, row_window_offset, workspace, workspace_bytes,
                                   n_tcb_host, max_tcb_per_window_host, stream);
}

extern "C" int f3s_preprocess_fill(const int32_t *colidx, const int32_t *rowptr, int32_t num_nodes, int64_t nnz,
                                   int32_t block_h, int32_t block_w, const int32_t *edge_to_column,
                                   const int32_t *edge_to_row, const int32_t *row_window_offset, int32_t n_tcb,
                                   int32_t *sorted_row_windows, int32_t *tcblock_rowid, uint8_t *tcblocktile_id,
                                   int32_t *tcblock_offset, int32_t *sparse_a_to_x_idx, uint64_t *tcb_bitmap,
                                   void *workspace, size_t workspace_bytes, f3s_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (int rc = check_pre_args(num_nodes, nnz, block_h, block_w, workspace, workspace_bytes)) return rc;
  F3S_REQUIRE(n_tcb >= 0, F3S_ERR_INVALID_ARG, "negative n_tcb");
  F3S_REQUIRE((long long)n_tcb < (1ll << 23) * 16, F3S_ERR_UNSUPPORTED, "n_tcb too large");
  F3S_REQUIRE(tcblock_offset && row_window_offset && rowptr, F3S_ERR_INVALID_ARG, "null pointer argument");
  const int n_rw = (num_nodes + 15) / 16;
  const PreWs L = pre_ws(num_nodes, nnz);
  unsigned char *ws = static_cast<unsigned char *>(workspace);
  if (n_rw == 0) {
    F3S_CUDA_TRY(cudaMemsetAsync(tcblock_offset, 0, sizeof(int), stream));
    return F3S_OK;
  }
  F3S_REQUIRE(sorted_row_windows, F3S_ERR_INVALID_ARG, "null sorted_row_windows");
  F3S_REQUIRE(n_tcb == 0 || (tcblock_rowid && sparse_a_to_x_idx && tcb_bitmap), F3S_ERR_INVALID_ARG,
              "null TCB output array");
  F3S_REQUIRE(nnz == 0 || (colidx && edge_to_column && edge_to_row && tcblocktile_id), F3S_ERR_INVALID_ARG,
              "null edge array");
  int *hdr = reinterpret_cast<int *>(ws + L.off_hdr);
  int *large_list = reinterpret_cast<int *>(ws + L.off_list);
  static_assert(PH_FILL_NEXT == PH_N_LARGE_FILL + 1, "one memset clears both");
  F3S_CUDA_TRY(cudaMemsetAsync(hdr + PH_N_LARGE_FILL, 0, 2 * sizeof(int), stream));
  window_fill_small<<<(n_rw + SW_WARPS - 1) / SW_WARPS, SW_WARPS * 32, 0, stream>>>(
      colidx, rowptr, num_nodes, n_rw, block_w, edge_to_column, edge_to_row, row_window_offset, tcblock_rowid,
      tcblocktile_id, tcblock_offset, sparse_a_to_x_idx, reinterpret_cast<unsigned long long *>(tcb_bitmap), hdr,
      large_list);
  F3S_CHECK_LAUNCH();
  F3S_CUDA_TRY(cudaFuncSetAttribute(window_fill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FILL_SMEM_BYTES));
  window_fill_kernel<<<min(n_rw, sm_count() * 2), FILL_THREADS, FILL_SMEM_BYTES, stream>>>(
      colidx, rowptr, num_nodes, n_rw, block_w, edge_to_column, edge_to_row, row_window_offset, large_list, hdr,
      tcblock_rowid, tcblocktile_id, tcblock_offset, sparse_a_to_x_idx,
      reinterpret_cast<unsigned long long *>(tcb_bitmap), reinterpret_cast<int *>(ws + L.off_a),
      reinterpret_cast<int *>(ws + L.off_b));
  F3S_CHECK_LAUNCH();
  if (int rc = inclusive_scan_inplace(tcblock_offset + 1, n_tcb, reinterpret_cast<int *>(ws + L.off_sums), stream))
    return rc;
  schedule_kernel<<<1, SCHED_THREADS, 0, stream>>>(row_window_offset, n_rw, sorted_row_windows,
                                                   reinterpret_cast<unsigned long long *>(ws + L.off_s0),
                                                   reinterpret_cast<unsigned long long *>(ws + L.off_s1));
  F3S_CHECK_LAUNCH();
  return F3S_OK;
}
