// Device pieces shared by the forward and backward attention kernels: the unit list and its
// schedule kernel, the per-warp unit iterator, the swizzled shared-memory tile and the
// A(16 x D) x gathered-rows^T tensor-core product.
#pragma once

#include "common.cuh"

namespace f3s {

struct UnitDesc {        // 32 bytes
  int window;            // row window id
  int t8_begin, t8_end;  // global 8-column-tile range [begin, end)
  int slot_base;         // first partial slot of the window
  int chunk, n_chunks;
  int pad0, pad1;
};

// Header of the scratch area.  U_HEAVY: units in the list (chunks of heavy windows);
// LIGHT_INV: n_rw - (first position in the window order that holds a light window).
// COUNTER: next position of the work order; DONE: warps that have run out of work (the last of them
// resets both, so that a launch leaves the scratch ready for the next one).
enum { HDR_U_HEAVY = 0, HDR_LIGHT_INV = 1, HDR_COUNTER = 2, HDR_STATUS = 3, HDR_DONE = 4, HDR_INTS = 16 };
enum { STATUS_LIST_OVERFLOW = 1, STATUS_WAIT_TIMEOUT = 2 };

struct FwdParams {
  const int *rwo;
  const int *sorted;  // may be null
  const int *atox;
  const unsigned long long *bitmap;
  const __half *q, *k, *v;
  float *out;     // fp32 output, or null when out_h is used
  __half *out_h;  // fp16 output (extension), or null
  float *sddmm;   // may be null
  float *lse;     // may be null: [n_nodes][heads] log2-domain log-sum-exp of the scaled scores of every row
  int n_nodes, n_rw, heads;
  int d_real;     // head dimension of the tensors; the kernels' D is d_real rounded up to 32, 64 or 128
  long long ld;     // row stride of q in elements
  long long ld_kv;  // row stride of k and v in elements
  int t8_per_tcb;
  int direct;    // 1: no schedule, static round-robin over windows
  int ch8;       // windows with more tiles than this are processed as chunks from the list
  int negate_q;  // 1: the divisor is negative, scores change sign (softmax path only)
  float scale;   // softmax: log2(e)/|divisor| (> 0); otherwise 1/divisor
  int *hdr;
  const UnitDesc *units;
  int *arrive;
  float *partial;
  int max_slots;
  unsigned long long *sm_trace;  // may be null: [F3S_SM_TRACE_SLOTS][2] first-start / last-end ns per SM
  // Two-phase calls (row-sharded attention that starts on the columns it already holds while the others
  // are still in flight).  phase 0: the whole window.  phase 1: only columns with id >= col_split; the
  // unnormalised result (running max, running sum, accumulator) goes to state[] instead of the output.
  // phase 2: only columns with id < col_split, continuing from state[]; writes the output.
  // phase_split[w]: first TC block of window w whose first column id is >= col_split (rwo[w+1] if none),
  // so the block before it is the only one that can hold columns of both kinds.
  int phase, col_split;
  const int *phase_split;
  float *state;  // [heads][n_rw] slots in the layout of a partial
};

// TC-block range of window w that a launch works on (see FwdParams::phase).
template <class P>
__device__ __forceinline__ void window_blocks(const P &p, int w, int &a, int &z) {
  a = p.rwo[w];
  z = p.rwo[w + 1];
  if (p.phase == 1) a = max(a, p.phase_split[w] - 1);
  else if (p.phase == 2) z = min(z, p.phase_split[w]);
}

constexpr unsigned FULL = 0xffffffffu;
constexpr float NEG_INF = -INFINITY;

// Per-SM busy interval of a launch (the reference's "Clocked" kernels stamp %globaltimer and
// %smid per CTA, src/F3S_kernel.cu:30-40, 1363-1367): earliest start and latest end per SM.
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ unsigned sm_id() {
  unsigned s;
  asm("mov.u32 %0, %%smid;" : "=r"(s));
  return s;
}
__device__ __forceinline__ void trace_begin(const FwdParams &p) {
  if (p.sm_trace != nullptr && threadIdx.x == 0) {
    const unsigned s = sm_id();
    if (s < F3S_SM_TRACE_SLOTS) atomicMin(&p.sm_trace[2 * s], global_timer_ns());
  }
}
__device__ __forceinline__ void trace_end(const FwdParams &p, int lane) {
  if (p.sm_trace != nullptr && lane == 0) {
    const unsigned s = sm_id();
    if (s < F3S_SM_TRACE_SLOTS) atomicMax(&p.sm_trace[2 * s + 1], global_timer_ns());
  }
}

// ---------------------------------------------------------------------------------------
// Schedule kernel: one thread per window position, no ordering between threads.  A heavy
// window appends its chunks to the unit list (warp-aggregated atomicAdd); light windows
// record the first position that is light, from which the fused kernel walks the window
// order directly.  The header and the arrival counters are zeroed by a memset before it.
// ---------------------------------------------------------------------------------------
constexpr int PLAN_THREADS = 256;

struct PlanArgs {  // the members window_blocks reads
  const int *rwo;
  int phase;
  const int *phase_split;
};

static __global__ void __launch_bounds__(PLAN_THREADS)
plan_kernel(const PlanArgs pa, const int *__restrict__ sorted, int n_rw, int t8_per_tcb, int ch8,
            int nt8, int *hdr, UnitDesc *units, int max_units) {
  const int i = blockIdx.x * PLAN_THREADS + threadIdx.x;
  const int lane = threadIdx.x & 31;
  int w = 0, first = 0, n8 = 0, nch = 0, per = 0;
  bool heavy = false;
  if (i < n_rw) {
    w = sorted ? sorted[i] : i;
    int a, b;
    window_blocks(pa, w, a, b);
    first = a * t8_per_tcb;
    n8 = (b - a) * t8_per_tcb;
    heavy = n8 > ch8;
    if (heavy) {
      const int want = (n8 + ch8 - 1) / ch8;
      per = ((n8 + want - 1) / want + nt8 - 1) / nt8 * nt8;
      nch = (n8 + per - 1) / per;
    }
  }
  int inc = nch;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(FULL, inc, o);
    if (lane >= o) inc += t;
  }
  const int total = __shfl_sync(FULL, inc, 31);
  int base = 0;
  if (lane == 31 && total > 0) base = atomicAdd(&hdr[HDR_U_HEAVY], total);
  base = __shfl_sync(FULL, base, 31);
  if (heavy) {
    const int unit0 = base + inc - nch;
    if (unit0 + nch <= max_units) {
      for (int c = 0; c < nch; ++c) {
        UnitDesc d;
        d.window = w;
        d.t8_begin = first + c * per;
        d.t8_end = first + min(n8, (c + 1) * per);
        d.slot_base = unit0;
        d.chunk = c;
        d.n_chunks = nch;
        d.pad0 = d.pad1 = 0;
        units[unit0 + c] = d;
      }
    } else {
      // Does not fit: report it, and leave no unwritten entry below the capacity (consumers skip
      // entries whose window is negative).  The window's rows stay unwritten; the host learns why.
      atomicExch(&hdr[HDR_STATUS], STATUS_LIST_OVERFLOW);
      UnitDesc d;
      d.window = -1;
      d.t8_begin = d.t8_end = d.slot_base = d.chunk = 0;
      d.n_chunks = 1;
      d.pad0 = d.pad1 = 0;
      for (int c = 0; c < nch && unit0 + c < max_units; ++c) units[unit0 + c] = d;
    }
  }
  int inv = (i < n_rw && !heavy) ? n_rw - i : 0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) inv = max(inv, __shfl_xor_sync(FULL, inv, o));
  if (lane == 0 && inv > 0) atomicMax(&hdr[HDR_LIGHT_INV], inv);
}

// ---------------------------------------------------------------------------------------
// Pieces shared by both data paths
// ---------------------------------------------------------------------------------------
template <int D>
struct Tile {
  static constexpr int ROW_BYTES = D * 2;
  static constexpr int CHUNKS = D / 8;  // 16-byte chunks per row
  // physical chunk position of logical chunk c in row r (bank-conflict-free ldmatrix; for
  // 128-byte rows this is also the TMA 128-byte swizzle of a 1024-byte-aligned tile)
  __device__ static __forceinline__ int swz(int r, int c) {
    if (D == 32) return c ^ ((r >> 1) & 3);
    return c ^ (r & 7);
  }
  __device__ static __forceinline__ uint32_t addr(uint32_t base, int r, int c) {
    return base + r * ROW_BYTES + swz(r, c) * 16;
  }
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct Unit {
  int head, window, t8b, t8e, slot_base, chunk, n_chunks;
};

// Per-warp iterator over the units of one launch.
struct UnitSource {
  long long x, total;
  int n_units, u_heavy, first_light, stride;

  template <class P>
  __device__ __forceinline__ void init(const P &p, int gwarp, int total_warps) {
    if (p.direct) {
      u_heavy = 0;
      first_light = 0;
    } else {
      u_heavy = min(p.hdr[HDR_U_HEAVY], p.max_slots);  // a list that overflowed holds max_slots entries at most
      first_light = p.n_rw - p.hdr[HDR_LIGHT_INV];
    }
    n_units = u_heavy + (p.n_rw - first_light);
    total = (long long)n_units * p.heads;
    x = gwarp;
    stride = total_warps;
  }
  // false when the work is exhausted
  template <class P>
  __device__ __forceinline__ bool next(const P &p, int lane, Unit &u) {
    for (;;) {
      long long cur;
      if (p.direct) {
        cur = x;
        x += stride;
      } else {
        int xi = 0;
        if (lane == 0) xi = atomicAdd(&p.hdr[HDR_COUNTER], 1);
        cur = __shfl_sync(FULL, xi, 0);
      }
      if (cur >= total) return false;
      u.head = (int)(cur / n_units);
      const int uu = (int)(cur - (long long)u.head * n_units);
      u.slot_base = -1;
      u.chunk = 0;
      u.n_chunks = 1;
      if (uu < u_heavy) {
        const UnitDesc d = p.units[uu];
        if (d.window < 0) continue;  // placeholder of a window the list had no room for
        u.window = d.window; u.t8b = d.t8_begin; u.t8e = d.t8_end;
        u.slot_base = d.slot_base; u.chunk = d.chunk; u.n_chunks = d.n_chunks;
        return true;
      }
      const int i = first_light + (uu - u_heavy);
      u.window = p.sorted ? p.sorted[i] : i;
      int a, z;
      window_blocks(p, u.window, a, z);
      u.t8b = a * p.t8_per_tcb;
      u.t8e = z * p.t8_per_tcb;
      if (p.direct || u.t8e - u.t8b <= p.ch8) return true;
      // a heavy window behind the first light one (window order not descending): it is in the list
    }
  }
};

// Called once by every warp of a scheduled launch after its last unit: the last warp to get here puts
// the work counter back to zero, so the scratch can serve the next launch without a memset (every warp
// has stopped drawing from the counter by then).
template <class P>
__device__ __forceinline__ void retire_warp(const P &p, int lane, int total_warps) {
  if (p.direct || lane != 0) return;
  __threadfence();
  if (atomicAdd(&p.hdr[HDR_DONE], 1) == total_warps - 1) {
    p.hdr[HDR_COUNTER] = 0;
    p.hdr[HDR_DONE] = 0;
    __threadfence();
  }
}

// The same iterator for kernels that mostly see short windows (a step or two).  There the chain
// counter -> window order -> window offsets, three dependent global loads, dominates a unit, so a
// warp takes up to UNIT_BATCH positions per counter increment and its lanes decode them side by side
// into a descriptor area in shared memory (UNIT_DESC_INTS ints per warp).  The batch is 1 unless there
// are many more units than warps.  (Measured on B200: 9 % faster on batches of small graphs; the
// kernels for long windows keep the plain iterator, with which they are 5-20 % faster.)
constexpr int UNIT_BATCH = 8;
constexpr int UNIT_DESC_INTS = UNIT_BATCH * 8;

struct BatchedUnitSource {
  long long x, total;
  int n_units, u_heavy, first_light, stride;
  int batch, have, pos;
  int *desc;  // shared memory of this warp, or null (batch = 1)

  template <class P>
  __device__ __forceinline__ void init(const P &p, int gwarp, int total_warps, int *desc_smem = nullptr) {
    if (p.direct) {
      u_heavy = 0;
      first_light = 0;
    } else {
      u_heavy = min(p.hdr[HDR_U_HEAVY], p.max_slots);  // a list that overflowed holds max_slots entries at most
      first_light = p.n_rw - p.hdr[HDR_LIGHT_INV];
    }
    n_units = u_heavy + (p.n_rw - first_light);
    total = (long long)n_units * p.heads;
    x = gwarp;
    stride = total_warps;
    desc = desc_smem;
    have = pos = 0;
    const long long per_warp = total / ((long long)total_warps * 8);  // batches of b need >= 8 b units per warp
    batch = (desc_smem == nullptr || per_warp < 2) ? 1 : (per_warp > UNIT_BATCH ? UNIT_BATCH : (int)per_warp);
  }

  // Decode position cur of the scheduled order; window = -1: nothing to do there (a heavy window
  // behind the first light one, which only happens when the window order is not descending: it is
  // in the list).
  template <class P>
  __device__ __forceinline__ void decode(const P &p, long long cur, Unit &u) const {
    u.head = (int)(cur / n_units);
    const int uu = (int)(cur - (long long)u.head * n_units);
    u.slot_base = -1;
    u.chunk = 0;
    u.n_chunks = 1;
    if (uu < u_heavy) {
      const UnitDesc d = p.units[uu];
      u.window = d.window; u.t8b = d.t8_begin; u.t8e = d.t8_end;
      u.slot_base = d.slot_base; u.chunk = d.chunk; u.n_chunks = d.n_chunks;
      return;
    }
    const int i = first_light + (uu - u_heavy);
    u.window = p.sorted ? p.sorted[i] : i;
    int a, z;
    window_blocks(p, u.window, a, z);
    u.t8b = a * p.t8_per_tcb;
    u.t8e = z * p.t8_per_tcb;
    if (!p.direct && u.t8e - u.t8b > p.ch8) u.window = -1;
  }

  // false when the work is exhausted
  template <class P>
  __device__ __forceinline__ bool next(const P &p, int lane, Unit &u) {
    if (p.direct) {
      const long long cur = x;
      x += stride;
      if (cur >= total) return false;
      decode(p, cur, u);
      return true;
    }
    for (;;) {
      if (batch == 1) {
        int xi = 0;
        if (lane == 0) xi = atomicAdd(&p.hdr[HDR_COUNTER], 1);
        const long long cur = __shfl_sync(FULL, xi, 0);
        if (cur >= total) return false;
        decode(p, cur, u);
        if (u.window >= 0) return true;
        continue;
      }
      if (pos >= have) {  // take the next batch of positions; lane l decodes position base + l
        int xi = 0;
        if (lane == 0) xi = atomicAdd(&p.hdr[HDR_COUNTER], batch);
        const long long base = __shfl_sync(FULL, xi, 0);
        if (base >= total) return false;
        const long long left = total - base;
        have = left < batch ? (int)left : batch;
        pos = 0;
        __syncwarp();  // the previous batch has been read by every lane
        if (lane < have) {
          Unit m;
          decode(p, base + lane, m);
          int4 *d4 = reinterpret_cast<int4 *>(desc + lane * 8);
          d4[0] = make_int4(m.head, m.window, m.t8b, m.t8e);
          d4[1] = make_int4(m.slot_base, m.chunk, m.n_chunks, 0);
        }
        __syncwarp();
      }
      const int4 *d4 = reinterpret_cast<const int4 *>(desc + pos * 8);
      const int4 a = d4[0], b = d4[1];
      ++pos;
      u.head = a.x; u.window = a.y; u.t8b = a.z; u.t8e = a.w;
      u.slot_base = b.x; u.chunk = b.y; u.n_chunks = b.z;
      if (u.window >= 0) return true;
    }
  }
};

// S = Q K^T for NT8 tiles of 8 gathered columns (K rows in shared memory at ksm).
template <int D, int NT8>
__device__ __forceinline__ void score_tiles(uint32_t ksm, const uint32_t (&qa)[D / 16][4], float (&s)[NT8][4],
                                            int lane) {
  using T = Tile<D>;
  constexpr int KS = D / 16;
#pragma unroll
  for (int nt = 0; nt < NT8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
  for (int k2 = 0; k2 < KS / 2; ++k2) {
    uint32_t b[NT8][4];
#pragma unroll
    for (int nt = 0; nt < NT8; ++nt) ldmatrix_x4(b[nt], T::addr(ksm, nt * 8 + (lane & 7), k2 * 4 + (lane >> 3)));
    // products on different accumulators back to back; the two on one tile are NT8 issues apart
#pragma unroll
    for (int nt = 0; nt < NT8; ++nt) mma_16816(s[nt], qa[2 * k2], b[nt][0], b[nt][1]);
#pragma unroll
    for (int nt = 0; nt < NT8; ++nt) mma_16816(s[nt], qa[2 * k2 + 1], b[nt][2], b[nt][3]);
  }
}

}  // namespace f3s
