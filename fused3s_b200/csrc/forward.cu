// Fused SDDMM -> online softmax -> SpMM over TC blocks for sm_100a.
//
// Work decomposition
//   * The unit of work is (head, row window, range of 8-column tiles).  A window is 16 query
//     rows; its distinct key columns are listed in sparse_a_to_x_idx and grouped in tiles of
//     8 columns (a 16-wide TCB is two tiles, an 8-wide TCB is one), each with two 64-bit
//     occupancy words (rows 0-7, rows 8-15).  Both TCB widths therefore look the same here.
//   * One warp owns one unit at a time.  Large problems: warps pull units from a global
//     counter.  Windows with more tiles than a threshold ("heavy") are cut into chunks by a
//     small, fully parallel schedule kernel; their chunks are processed first, then the
//     remaining windows in the order of sorted_row_windows (largest first), so the tail of
//     the kernel is made of the smallest windows.  Every chunk writes an unnormalised
//     partial (running max, running sum, 16 x d accumulator) to scratch and the last chunk
//     to arrive merges them in chunk order.  Small problems ("direct" mode): no schedule
//     kernel and no counter; a CTA walks its share of the window order and its warps share the
//     long windows among themselves -- one launch per call.  No warp ever spins on another.
//   * Per step a warp handles 32 gathered columns.  Three data paths bring the gathered K and
//     V rows into the warp's private, swizzled shared-memory stages:
//       - 16-byte cp.async.cg per lane with separate K and V rings (d = 64, the default there);
//       - 16-byte cp.async.cg per lane with combined K+V stages (every other d, short windows,
//         the small-problem kernel, the score dump);
//       - d = 64 on request: TMA.  One cp.async.bulk.tensor...tile::gather4 per four rows (issued
//         by eight lanes at once), one bulk copy for the step's bitmap words, one tiled TMA load
//         for the Q window; completion through one mbarrier per stage, every wait bounded.
//     The score tile S = Q K^T and the update O += P V run on the tensor cores
//     (ldmatrix + mma.sync m16n8k16, fp16 in, fp32 accumulate); S, P, the running max/sum and
//     O live in registers, S never leaves the SM.
//
// Numerics (same contract as the reference kernel src/F3S_kernel.cu:1586-1800): fp16
// operands, fp32 scores, probabilities rounded to fp16 before P V, fp32 running sum and
// output.  Masking uses the bitmap (masked = -inf), not the reference's "score == 0 means
// masked" shortcut (src/F3S_kernel.cu:1097-1098), and the running max starts at -inf
// rather than 0 (src/F3S_kernel.cu:1021).
#include <cuda.h>
#include <limits.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "attn_common.cuh"

namespace f3s {

// Mask the score tiles by the bitmap, update the online softmax, O += P V (V rows at vsm).
// s is consumed (overwritten by the probabilities).
// FILTER: additionally mask by cm, one bit per gathered column of the step (set = column takes part).
template <int D, int NT8, bool SOFTMAX, bool CHECK_TAIL, bool SDDMM = true, bool FILTER = false>
__device__ __forceinline__ void softmax_pv(const FwdParams &p, float (&s)[NT8][4], uint32_t vsm, const uint32_t *bm32,
                                           int n_valid, int t8_first, float (&o)[D / 8][4], float (&m_run)[2],
                                           float (&l_run)[2], int lane, int bm_shift, uint32_t cm = 0xffffffffu);

// One step of the fused loop on tiles already in shared memory: S = Q K^T, mask, online
// softmax, O += P V.  n_valid (warp-uniform) = tiles of this step that belong to the unit;
// CHECK_TAIL is set when stale bitmap words may sit behind them.
template <int D, int NT8, bool SOFTMAX, bool CHECK_TAIL, bool FILTER = false>
__device__ __forceinline__ void compute_step(const FwdParams &p, uint32_t ksm, uint32_t vsm, const uint32_t *bm32,
                                             int n_valid, int t8_first, const uint32_t (&qa)[D / 16][4],
                                             float (&o)[D / 8][4], float (&m_run)[2], float (&l_run)[2], int lane,
                                             int bm_shift, uint32_t cm = 0xffffffffu) {
  float s[NT8][4];
  score_tiles<D, NT8>(ksm, qa, s, lane);
  softmax_pv<D, NT8, SOFTMAX, CHECK_TAIL, true, FILTER>(p, s, vsm, bm32, n_valid, t8_first, o, m_run, l_run, lane,
                                                       bm_shift, cm);
}

template <int D, int NT8, bool SOFTMAX, bool CHECK_TAIL, bool SDDMM, bool FILTER>
__device__ __forceinline__ void softmax_pv(const FwdParams &p, float (&s)[NT8][4], uint32_t vsm, const uint32_t *bm32,
                                           int n_valid, int t8_first, float (&o)[D / 8][4], float (&m_run)[2],
                                           float (&l_run)[2], int lane, int bm_shift, uint32_t cm) {
  using T = Tile<D>;
  constexpr int NF = D / 8;
  const int g = lane >> 2, qd = lane & 3;
  float mx[2] = {NEG_INF, NEG_INF};
#pragma unroll
  for (int nt = 0; nt < NT8; ++nt) {
    uint32_t h0 = bm32[nt * 4] << bm_shift, h1 = bm32[nt * 4 + 2] << bm_shift;
    if (CHECK_TAIL && nt >= n_valid) h0 = h1 = 0u;
    if (FILTER) {  // columns 2qd and 2qd+1 of tile nt: clear their occupancy bits unless the column takes part
      const uint32_t cb = cm >> (nt * 8 + 2 * qd);
      const uint32_t keep = ((cb & 1u) << 31) | ((cb & 2u) << 29);
      h0 &= keep;
      h1 &= keep;
    }
    const bool v0 = (int)h0 < 0, v1 = (int)(h0 << 1) < 0, v2 = (int)h1 < 0, v3 = (int)(h1 << 1) < 0;
    if (SDDMM && p.sddmm != nullptr) {
      if (nt < n_valid) {
        float *dst = p.sddmm + (size_t)(t8_first + nt) * 128 + g * 8 + 2 * qd;
        *reinterpret_cast<float2 *>(dst) = make_float2(v0 ? s[nt][0] : 0.f, v1 ? s[nt][1] : 0.f);
        *reinterpret_cast<float2 *>(dst + 64) = make_float2(v2 ? s[nt][2] : 0.f, v3 ? s[nt][3] : 0.f);
      }
    }
    if (SOFTMAX) {
      s[nt][0] = v0 ? s[nt][0] : NEG_INF;
      s[nt][1] = v1 ? s[nt][1] : NEG_INF;
      s[nt][2] = v2 ? s[nt][2] : NEG_INF;
      s[nt][3] = v3 ? s[nt][3] : NEG_INF;
      mx[0] = fmaxf(mx[0], fmaxf(s[nt][0], s[nt][1]));
      mx[1] = fmaxf(mx[1], fmaxf(s[nt][2], s[nt][3]));
    } else {
      s[nt][0] = v0 ? s[nt][0] * p.scale : 0.f;
      s[nt][1] = v1 ? s[nt][1] * p.scale : 0.f;
      s[nt][2] = v2 ? s[nt][2] * p.scale : 0.f;
      s[nt][3] = v3 ? s[nt][3] * p.scale : 0.f;
    }
  }
  if (SOFTMAX) {
    // online softmax in the raw-score domain; the positive scale is folded into the exponent
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(FULL, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(FULL, mx[h], 2));
      mx[h] = fmaxf(mx[h], m_run[h]);
    }
    const bool changed = (mx[0] != m_run[0]) || (mx[1] != m_run[1]);
    if (__any_sync(FULL, changed)) {  // rare after the first steps of a window
      float alpha[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float m_use = (mx[h] == NEG_INF) ? 0.f : mx[h];
        alpha[h] = fast_exp2((m_run[h] - m_use) * p.scale);  // m_run == -inf gives 0
        m_run[h] = mx[h];
        l_run[h] *= alpha[h];
      }
#pragma unroll
      for (int f = 0; f < NF; ++f) {
        o[f][0] *= alpha[0]; o[f][1] *= alpha[0];
        o[f][2] *= alpha[1]; o[f][3] *= alpha[1];
      }
    }
    const float nm0 = -((m_run[0] == NEG_INF) ? 0.f : m_run[0]) * p.scale;
    const float nm1 = -((m_run[1] == NEG_INF) ? 0.f : m_run[1]) * p.scale;
#pragma unroll
    for (int nt = 0; nt < NT8; ++nt) {
      s[nt][0] = fast_exp2(fmaf(s[nt][0], p.scale, nm0));  // masked: exp2(-inf) = 0
      s[nt][1] = fast_exp2(fmaf(s[nt][1], p.scale, nm0));
      s[nt][2] = fast_exp2(fmaf(s[nt][2], p.scale, nm1));
      s[nt][3] = fast_exp2(fmaf(s[nt][3], p.scale, nm1));
    }
  }
  // Row sums of the (fp16-rounded) probabilities come from the tensor cores as well: P times a
  // column of ones.  Every lane of a quad then holds the complete sums of rows g and g+8.
  float la[4] = {l_run[0], l_run[0], l_run[1], l_run[1]};
#pragma unroll
  for (int j = 0; j < NT8 / 2; ++j) {  // O += P V, 16 gathered columns (two tiles) per k-step
    uint32_t pa[4];
    pa[0] = pack_half2(s[2 * j][0], s[2 * j][1]);
    pa[1] = pack_half2(s[2 * j][2], s[2 * j][3]);
    pa[2] = pack_half2(s[2 * j + 1][0], s[2 * j + 1][1]);
    pa[3] = pack_half2(s[2 * j + 1][2], s[2 * j + 1][3]);
    if (SOFTMAX) mma_16816(la, pa, 0x3c003c00u, 0x3c003c00u);
#pragma unroll
    for (int fp = 0; fp < NF / 2; ++fp) {
      uint32_t b[4];
      const int m = lane >> 3;
      ldmatrix_x4_trans(b, T::addr(vsm, j * 16 + (m & 1) * 8 + (lane & 7), 2 * fp + (m >> 1)));
      mma_16816(o[2 * fp], pa, b[0], b[1]);
      mma_16816(o[2 * fp + 1], pa, b[2], b[3]);
    }
  }
  if (SOFTMAX) {
    l_run[0] = la[0];
    l_run[1] = la[2];
  }
}

// Q fragments from the (swizzled) Q window in shared memory.
template <int D, bool SOFTMAX>
__device__ __forceinline__ void load_q_frags(const FwdParams &p, uint32_t q_s, uint32_t (&qa)[D / 16][4], int lane) {
  using T = Tile<D>;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const int m = lane >> 3;
    ldmatrix_x4(qa[ks], T::addr(q_s, (m & 1) * 8 + (lane & 7), ks * 2 + (m >> 1)));
    if (SOFTMAX && p.negate_q) {
#pragma unroll
      for (int e = 0; e < 4; ++e) qa[ks][e] ^= 0x80008000u;
    }
  }
}

// Store feature tile f (8 columns) of rows g and g+8 of a window; values already normalised.
template <int D>
__device__ __forceinline__ void store_tile(const FwdParams &p, int head, int window, int f, float v0, float v1,
                                           float v2, float v3, int lane) {
  if (f * 8 >= p.d_real) return;  // feature tiles that only exist as zero padding
  const int g = lane >> 2, qd = lane & 3;
  const int r0 = window * 16 + g, r1 = r0 + 8;
  const size_t ldo = (size_t)p.heads * p.d_real;
  const size_t off0 = (size_t)r0 * ldo + (size_t)head * p.d_real + 2 * qd + f * 8;
  const size_t off1 = (size_t)r1 * ldo + (size_t)head * p.d_real + 2 * qd + f * 8;
  if (p.out_h == nullptr) {
    if (r0 < p.n_nodes) *reinterpret_cast<float2 *>(p.out + off0) = make_float2(v0, v1);
    if (r1 < p.n_nodes) *reinterpret_cast<float2 *>(p.out + off1) = make_float2(v2, v3);
  } else {
    if (r0 < p.n_nodes) *reinterpret_cast<__half2 *>(p.out_h + off0) = __floats2half2_rn(v0, v1);
    if (r1 < p.n_nodes) *reinterpret_cast<__half2 *>(p.out_h + off1) = __floats2half2_rn(v2, v3);
  }
}

// log2-domain log-sum-exp of rows g and g+8 of a window: lse = max * scale + log2(sum), so that the
// probability of an edge is exp2(score * scale - lse).  Rows without edges get 0.  m and l are the
// final running max (raw-score domain) and the running sum of the row.
__device__ __forceinline__ void store_lse(const FwdParams &p, int head, int window, const float (&m)[2],
                                          const float (&l)[2], int lane) {
  if (p.lse == nullptr || (lane & 3) != 0) return;
  const int r0 = window * 16 + (lane >> 2), r1 = r0 + 8;
  if (r0 < p.n_nodes) p.lse[(size_t)r0 * p.heads + head] = (l[0] > 0.f) ? fmaf(m[0], p.scale, log2f(l[0])) : 0.f;
  if (r1 < p.n_nodes) p.lse[(size_t)r1 * p.heads + head] = (l[1] > 0.f) ? fmaf(m[1], p.scale, log2f(l[1])) : 0.f;
}

// Normalise by the row sums and store a whole window.
template <int D, bool SOFTMAX>
__device__ __forceinline__ void store_output(const FwdParams &p, int head, int window, const float (&o)[D / 8][4],
                                             const float (&m_run)[2], const float (&l_run)[2], int lane) {
  float inv0 = 1.f, inv1 = 1.f;
  if (SOFTMAX) {
    inv0 = (l_run[0] > 0.f) ? 1.f / l_run[0] : 0.f;
    inv1 = (l_run[1] > 0.f) ? 1.f / l_run[1] : 0.f;
    store_lse(p, head, window, m_run, l_run, lane);
  }
#pragma unroll
  for (int f = 0; f < D / 8; ++f)
    store_tile<D>(p, head, window, f, o[f][0] * inv0, o[f][1] * inv0, o[f][2] * inv1, o[f][3] * inv1, lane);
}

// Two-phase calls: the unnormalised result of a window (running max, running sum, accumulator) is
// carried from the first launch to the second through state[], in the layout of a partial.
template <int D>
__device__ __forceinline__ float *state_slot(const FwdParams &p, int head, int window) {
  constexpr int PARTIAL_FLOATS = ((D / 8) * 4 + 4) * 32;
  return p.state + ((size_t)head * p.n_rw + window) * PARTIAL_FLOATS;
}

// Start of a unit of the second launch: the first chunk of a window continues from the carried state.
template <int D>
__device__ __forceinline__ void load_state(const FwdParams &p, const Unit &u, float (&o)[D / 8][4],
                                           float (&m_run)[2], float (&l_run)[2], int lane) {
  constexpr int NF = D / 8;
  if (p.phase != 2 || u.chunk != 0) return;
  const float *st = state_slot<D>(p, u.head, u.window);
#pragma unroll
  for (int f = 0; f < NF; ++f)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[f][e] = __ldcg(st + (f * 4 + e) * 32 + lane);
  m_run[0] = __ldcg(st + (NF * 4 + 0) * 32 + lane);
  m_run[1] = __ldcg(st + (NF * 4 + 1) * 32 + lane);
  l_run[0] = __ldcg(st + (NF * 4 + 2) * 32 + lane);
  l_run[1] = __ldcg(st + (NF * 4 + 3) * 32 + lane);
}

// End of a unit: reduce the row sums, publish / merge partials of a split window, store.
template <int D, bool SOFTMAX>
__device__ __forceinline__ void finish_unit(const FwdParams &p, const Unit &u, float (&o)[D / 8][4],
                                            float (&m_run)[2], float (&l_run)[2], int lane) {
  constexpr int NF = D / 8;
  constexpr int PARTIAL_FLOATS = (NF * 4 + 4) * 32;
  bool write_out = true;
  if (u.slot_base >= 0) {
    float *mine = p.partial + ((size_t)u.head * p.max_slots + u.slot_base + u.chunk) * PARTIAL_FLOATS;
#pragma unroll
    for (int f = 0; f < NF; ++f)
#pragma unroll
      for (int e = 0; e < 4; ++e) __stcg(mine + (f * 4 + e) * 32 + lane, o[f][e]);
    __stcg(mine + (NF * 4 + 0) * 32 + lane, m_run[0]);
    __stcg(mine + (NF * 4 + 1) * 32 + lane, m_run[1]);
    __stcg(mine + (NF * 4 + 2) * 32 + lane, l_run[0]);
    __stcg(mine + (NF * 4 + 3) * 32 + lane, l_run[1]);
    __threadfence();
    __syncwarp();
    int prev = 0;
    if (lane == 0) prev = atomicAdd(&p.arrive[(size_t)u.head * p.max_slots + u.slot_base], 1);
    prev = __shfl_sync(FULL, prev, 0);
    write_out = (prev == u.n_chunks - 1);
    if (write_out) {  // last chunk to arrive: merge all chunks in chunk order
      __threadfence();
      const float *base = p.partial + ((size_t)u.head * p.max_slots + u.slot_base) * PARTIAL_FLOATS;
      float mm[2] = {NEG_INF, NEG_INF};
      if (SOFTMAX) {
        for (int c = 0; c < u.n_chunks; ++c) {
          const float *pc = base + (size_t)c * PARTIAL_FLOATS;
          mm[0] = fmaxf(mm[0], __ldcg(pc + (NF * 4 + 0) * 32 + lane));
          mm[1] = fmaxf(mm[1], __ldcg(pc + (NF * 4 + 1) * 32 + lane));
        }
        m_run[0] = mm[0];  // may be -inf (no column seen yet): what a carried state must say
        m_run[1] = mm[1];
        if (mm[0] == NEG_INF) mm[0] = 0.f;
        if (mm[1] == NEG_INF) mm[1] = 0.f;
      }
#pragma unroll
      for (int f = 0; f < NF; ++f) o[f][0] = o[f][1] = o[f][2] = o[f][3] = 0.f;
      l_run[0] = l_run[1] = 0.f;
      for (int c = 0; c < u.n_chunks; ++c) {
        const float *pc = base + (size_t)c * PARTIAL_FLOATS;
        float w0 = 1.f, w1 = 1.f;
        if (SOFTMAX) {
          w0 = fast_exp2((__ldcg(pc + (NF * 4 + 0) * 32 + lane) - mm[0]) * p.scale);
          w1 = fast_exp2((__ldcg(pc + (NF * 4 + 1) * 32 + lane) - mm[1]) * p.scale);
          l_run[0] += w0 * __ldcg(pc + (NF * 4 + 2) * 32 + lane);
          l_run[1] += w1 * __ldcg(pc + (NF * 4 + 3) * 32 + lane);
        }
#pragma unroll
        for (int f = 0; f < NF; ++f) {
          o[f][0] += w0 * __ldcg(pc + (f * 4 + 0) * 32 + lane);
          o[f][1] += w0 * __ldcg(pc + (f * 4 + 1) * 32 + lane);
          o[f][2] += w1 * __ldcg(pc + (f * 4 + 2) * 32 + lane);
          o[f][3] += w1 * __ldcg(pc + (f * 4 + 3) * 32 + lane);
        }
      }
      // every chunk has arrived and been read: leave the counter at zero for the next launch
      if (lane == 0) p.arrive[(size_t)u.head * p.max_slots + u.slot_base] = 0;
    }
  }
  if (!write_out) return;
  if (p.phase == 1) {  // first launch of a two-phase call: carry the unnormalised result
    float *st = state_slot<D>(p, u.head, u.window);
#pragma unroll
    for (int f = 0; f < NF; ++f)
#pragma unroll
      for (int e = 0; e < 4; ++e) __stcg(st + (f * 4 + e) * 32 + lane, o[f][e]);
    __stcg(st + (NF * 4 + 0) * 32 + lane, m_run[0]);
    __stcg(st + (NF * 4 + 1) * 32 + lane, m_run[1]);
    __stcg(st + (NF * 4 + 2) * 32 + lane, l_run[0]);
    __stcg(st + (NF * 4 + 3) * 32 + lane, l_run[1]);
    return;
  }
  store_output<D, SOFTMAX>(p, u.head, u.window, o, m_run, l_run, lane);
}

// ---------------------------------------------------------------------------------------
// Data path 1: cp.async
// ---------------------------------------------------------------------------------------
template <int D, int NT8, int STAGES, int WARPS>
struct FwdCfg {
  static constexpr int ROWS = NT8 * 8;
  static constexpr int TILE_BYTES = ROWS * D * 2;
  static constexpr int BM_BYTES = 128;  // NT8 * 16 rounded up
  static constexpr int STAGE_BYTES = 2 * TILE_BYTES + BM_BYTES;
  static constexpr int Q_BYTES = 16 * D * 2;
  static constexpr int WARP_BYTES = Q_BYTES + STAGES * STAGE_BYTES;
  static constexpr int SMEM_BYTES = WARPS * WARP_BYTES;
  static_assert(NT8 * 16 + 4 <= BM_BYTES, "bitmap slot too small (bitmap words + one column-mask word)");
  static_assert(NT8 % 2 == 0 && ROWS <= 32, "a step is 16 or 32 gathered columns");
  static_assert(SMEM_BYTES + WARPS * UNIT_DESC_INTS * 4 <= 232448, "exceeds the 227 KB of shared memory a CTA can have");
};

// Lane-constant addresses of one warp's staging area.
template <int D, int NT8, int STAGES, int WARPS>
struct WarpStage {
  using C = FwdCfg<D, NT8, STAGES, WARPS>;
  uint32_t q_s, stage0_s;
  const unsigned char *stage0_g;
  int bm_half, bm_shift;
  __device__ __forceinline__ void init(unsigned char *wsm, int lane) {
    const int g = lane >> 2, qd = lane & 3;
    q_s = smem_u32(wsm);
    stage0_s = q_s + C::Q_BYTES;
    stage0_g = wsm + C::Q_BYTES;
    bm_half = (g < 4) ? 1 : 0;  // this lane's rows sit in one 32-bit half of each 64-bit bitmap word
    bm_shift = 8 * (g & 3) + 2 * qd;
  }
};

// The fused loop of one unit (window `window` of head `head`, tiles [t8b, t8e)) on the combined-stage
// cp.async path; accumulates into o / m_run / l_run.  All copies have landed when it returns.
template <int D, int NT8, int STAGES, int WARPS, bool SOFTMAX, bool FILTER = false>
__device__ __forceinline__ void run_unit_cpasync(const FwdParams &p, const WarpStage<D, NT8, STAGES, WARPS> &ws,
                                                 int head, int window, int t8b, int t8e, float (&o)[D / 8][4],
                                                 float (&m_run)[2], float (&l_run)[2], int lane) {
  using C = FwdCfg<D, NT8, STAGES, WARPS>;
  using T = Tile<D>;
  constexpr int KS = D / 16;
  constexpr int ROWS = C::ROWS;
  constexpr int CPL = ROWS * T::CHUNKS / 32;  // 16-byte copies per lane per operand tile
  const int nsteps = (t8e - t8b + NT8 - 1) / NT8;
  if (nsteps <= 0) return;
  const __half *kb = p.k + (size_t)head * p.d_real;
  const __half *vb = p.v + (size_t)head * p.d_real;
  {  // Q window -> shared (joins the first copy group); rows past the last node read as 0
    const int row0 = window * 16;
#pragma unroll
    for (int c = lane; c < 16 * T::CHUNKS; c += 32) {
      const int r = c / T::CHUNKS, ch = c % T::CHUNKS;
      const int gr = row0 + r;
      const bool ok = gr < p.n_nodes && ch * 8 < p.d_real;  // padding chunks and rows read as 0
      const __half *srcq = p.q + (size_t)(ok ? gr : 0) * p.ld + (size_t)head * p.d_real + (ok ? ch * 8 : 0);
      cp_async16(T::addr(ws.q_s, r, ch), srcq, ok ? 16 : 0);
    }
  }
  int idx_next = 0;  // column id of row `lane` of the next step to be issued
  {
    const int lim = (t8e - t8b) * 8;
    if (lane < ROWS && lane < lim) idx_next = __ldg(p.atox + (size_t)t8b * 8 + lane);
  }
  auto issue = [&](int step) {
    const int t8 = t8b + step * NT8;
    const int st = step % STAGES;
    const uint32_t ks = ws.stage0_s + st * C::STAGE_BYTES;
    const uint32_t vs = ks + C::TILE_BYTES;
    const uint32_t bs = vs + C::TILE_BYTES;
    const int lim = (t8e - t8) * 8;  // rows at or beyond lim lie outside the unit
    int idx_cur = idx_next;
    if (FILTER) {  // which of the step's columns take part in this launch; kept beside the bitmap words
      const bool take = p.phase == 1 ? idx_cur >= p.col_split : idx_cur < p.col_split;
      const uint32_t cm = __ballot_sync(FULL, take);
      if (lane == 0) asm volatile("st.shared.u32 [%0], %1;" ::"r"(bs + NT8 * 16), "r"(cm) : "memory");
      // The first launch runs before the other ranks' rows have arrived: a column that does not take part
      // must not even be read there (0 x stale NaN would poison the accumulator), so it reads an own row.
      if (p.phase == 1 && !take) idx_cur = p.col_split;
    }
    {
      const int t8n = t8 + NT8;
      const int limn = (t8e - t8n) * 8;
      idx_next = 0;
      if (lane < ROWS && lane < limn) idx_next = __ldg(p.atox + (size_t)t8n * 8 + lane);
    }
#pragma unroll
    for (int i = 0; i < CPL; ++i) {
      const int c = i * 32 + lane;
      const int r = c / T::CHUNKS, ch = c % T::CHUNKS;
      const int idx = __shfl_sync(FULL, idx_cur, r);
      const bool real = ch * 8 < p.d_real;
      const int nbytes = (r < lim && real) ? 16 : 0;
      const size_t off = (size_t)idx * p.ld_kv + (real ? ch * 8 : 0);
      cp_async16(T::addr(ks, r, ch), kb + off, nbytes);
      cp_async16(T::addr(vs, r, ch), vb + off, nbytes);
    }
    if (lane < NT8) {
      const bool ok = (t8 + lane) < t8e;
      cp_async16(bs + lane * 16, p.bitmap + (ok ? (size_t)(t8 + lane) * 2 : 0), ok ? 16 : 0);
    }
  };
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < nsteps) issue(s);
    cp_async_commit();
  }
  uint32_t qa[KS][4];
  for (int step = 0; step < nsteps; ++step) {
    if (step + STAGES - 1 < nsteps) issue(step + STAGES - 1);
    cp_async_commit();
    cp_async_wait<STAGES - 1>();
    __syncwarp();
    if (step == 0) load_q_frags<D, SOFTMAX>(p, ws.q_s, qa, lane);
    const int st = step % STAGES;
    const uint32_t ksm = ws.stage0_s + st * C::STAGE_BYTES;
    const uint32_t vsm = ksm + C::TILE_BYTES;
    const uint32_t *bm32 =
        reinterpret_cast<const uint32_t *>(ws.stage0_g + st * C::STAGE_BYTES + 2 * C::TILE_BYTES) + ws.bm_half;
    const int t8 = t8b + step * NT8;
    uint32_t cm = 0xffffffffu;
    if (FILTER)
      cm = *reinterpret_cast<const uint32_t *>(ws.stage0_g + st * C::STAGE_BYTES + 2 * C::TILE_BYTES + NT8 * 16);
    compute_step<D, NT8, SOFTMAX, false, FILTER>(p, ksm, vsm, bm32, min(NT8, t8e - t8), t8, qa, o, m_run, l_run, lane,
                                                 ws.bm_shift, cm);
    __syncwarp();  // every lane is done with this stage before it is refilled
  }
  cp_async_wait<0>();
}

template <int D, int NT8, int STAGES, int WARPS, bool SOFTMAX, bool FILTER = false>
__global__ void __launch_bounds__(WARPS * 32, 1) fwd_kernel(const FwdParams p) {
  using C = FwdCfg<D, NT8, STAGES, WARPS>;
  constexpr int NF = D / 8;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  WarpStage<D, NT8, STAGES, WARPS> ws;
  ws.init(smem_raw + warp * C::WARP_BYTES, lane);

  __shared__ __align__(16) int unit_desc[WARPS][UNIT_DESC_INTS];
  trace_begin(p);
  BatchedUnitSource src;
  src.init(p, blockIdx.x * WARPS + warp, gridDim.x * WARPS, unit_desc[warp]);
  Unit u;
  while (src.next(p, lane, u)) {
    float o[NF][4];
#pragma unroll
    for (int f = 0; f < NF; ++f) o[f][0] = o[f][1] = o[f][2] = o[f][3] = 0.f;
    float m_run[2] = {NEG_INF, NEG_INF};  // running max of the raw (unscaled) scores, rows g and g+8
    float l_run[2] = {0.f, 0.f};          // running sum of rows g and g+8
    if (FILTER) load_state<D>(p, u, o, m_run, l_run, lane);
    run_unit_cpasync<D, NT8, STAGES, WARPS, SOFTMAX, FILTER>(p, ws, u.head, u.window, u.t8b, u.t8e, o, m_run, l_run,
                                                             lane);
    finish_unit<D, SOFTMAX>(p, u, o, m_run, l_run, lane);
  }
  retire_warp(p, lane, gridDim.x * WARPS);
  trace_end(p, lane);
}

// ---------------------------------------------------------------------------------------
// Small problems ("direct" mode): one launch, no schedule, no global counter.  Position x of the
// (head, window) order belongs to CTA x mod #CTAs; a CTA walks its positions in rounds of one per
// warp.  In every round the warps publish the step counts of their windows; a window that is
// long compared with the round's average is shared by the whole CTA (warp k runs the k-th
// contiguous slice of its steps, writes its partial result - running max, running sum,
// accumulator - into its own, at that moment idle, staging area, and after a block barrier the
// warps merge the partials feature tile by feature tile and store), every other window is
// handled by its warp alone.  So no warp ever walks a long window on its own, whatever the
// shape of a small graph, and rounds of short windows cost one barrier.
// ---------------------------------------------------------------------------------------
struct DirectItem {
  int head, window, t8b, t8e;
};

__device__ __forceinline__ DirectItem direct_item(const FwdParams &p, long long x) {
  DirectItem it;
  it.head = (int)(x / p.n_rw);
  const int i = (int)(x - (long long)it.head * p.n_rw);
  it.window = p.sorted ? __ldg(p.sorted + i) : i;
  it.t8b = __ldg(p.rwo + it.window) * p.t8_per_tcb;
  it.t8e = __ldg(p.rwo + it.window + 1) * p.t8_per_tcb;
  return it;
}

template <int D, int NT8, int STAGES, int WARPS, bool SOFTMAX>
__global__ void __launch_bounds__(WARPS * 32, 1) fwd_kernel_coop(const FwdParams p) {
  using C = FwdCfg<D, NT8, STAGES, WARPS>;
  constexpr int NF = D / 8;
  constexpr int PART_FLOATS = (NF * 4 + 4) * 32;
  static_assert(PART_FLOATS * 4 <= C::WARP_BYTES, "a partial must fit in a warp's staging area");
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ int steps_s[2][WARPS];  // double-buffered: a fast warp may publish round r+1 while a slow one reads round r
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  WarpStage<D, NT8, STAGES, WARPS> ws;
  ws.init(smem_raw + warp * C::WARP_BYTES, lane);
  float *my_part = reinterpret_cast<float *>(smem_raw + warp * C::WARP_BYTES);

  // One-launch mode has no memset and no schedule kernel: nothing here can fail, so the status word
  // a later f3s_forward_status reads is cleared by the kernel itself.
  if (blockIdx.x == 0 && threadIdx.x == 0) p.hdr[HDR_STATUS] = 0;
  trace_begin(p);
  const long long total = (long long)p.n_rw * p.heads;
  int round = 0;
  for (long long base = blockIdx.x; base < total; base += (long long)gridDim.x * WARPS, ++round) {
    const long long x = base + (long long)warp * gridDim.x;
    DirectItem mine = {0, 0, 0, 0};
    int my_steps = -1;  // -1: no window for this warp in this round
    if (x < total) {
      mine = direct_item(p, x);
      my_steps = (mine.t8e - mine.t8b + NT8 - 1) / NT8;
    }
    if (lane == 0) steps_s[round & 1][warp] = my_steps;
    __syncthreads();
    const int *steps = steps_s[round & 1];
    int sum = 0;
#pragma unroll
    for (int j = 0; j < WARPS; ++j) sum += max(steps[j], 0);
    const int thr = max(2, 2 * ((sum + WARPS - 1) / WARPS));  // longer than this: shared by the CTA

#pragma unroll 1
    for (int j = 0; j < WARPS; ++j) {
      if (steps[j] <= thr) continue;  // the same decision in every warp
      const DirectItem it = direct_item(p, base + (long long)j * gridDim.x);
      const int nsteps = steps[j];
      const int per = (nsteps + WARPS - 1) / WARPS;
      const int s0 = min(nsteps, warp * per), s1 = min(nsteps, s0 + per);
      float o[NF][4];
#pragma unroll
      for (int f = 0; f < NF; ++f) o[f][0] = o[f][1] = o[f][2] = o[f][3] = 0.f;
      float m_run[2] = {NEG_INF, NEG_INF};
      float l_run[2] = {0.f, 0.f};
      run_unit_cpasync<D, NT8, STAGES, WARPS, SOFTMAX>(p, ws, it.head, it.window, it.t8b + s0 * NT8,
                                                       min(it.t8e, it.t8b + s1 * NT8), o, m_run, l_run, lane);
      __syncwarp();
#pragma unroll
      for (int f = 0; f < NF; ++f)
#pragma unroll
        for (int e = 0; e < 4; ++e) my_part[(f * 4 + e) * 32 + lane] = o[f][e];
      my_part[(NF * 4 + 0) * 32 + lane] = m_run[0];
      my_part[(NF * 4 + 1) * 32 + lane] = m_run[1];
      my_part[(NF * 4 + 2) * 32 + lane] = l_run[0];
      my_part[(NF * 4 + 3) * 32 + lane] = l_run[1];
      __syncthreads();
      if (warp < NF) {  // merge: slices in step order; feature tiles are divided among the warps
        float mm[2] = {NEG_INF, NEG_INF}, ll[2] = {0.f, 0.f};
        float wgt[WARPS][2];
#pragma unroll
        for (int c = 0; c < WARPS; ++c) {
          const float *pc = reinterpret_cast<const float *>(smem_raw + c * C::WARP_BYTES);
          wgt[c][0] = pc[(NF * 4 + 0) * 32 + lane];
          wgt[c][1] = pc[(NF * 4 + 1) * 32 + lane];
          mm[0] = fmaxf(mm[0], wgt[c][0]);
          mm[1] = fmaxf(mm[1], wgt[c][1]);
        }
        if (mm[0] == NEG_INF) mm[0] = 0.f;
        if (mm[1] == NEG_INF) mm[1] = 0.f;
#pragma unroll
        for (int c = 0; c < WARPS; ++c) {
          const float *pc = reinterpret_cast<const float *>(smem_raw + c * C::WARP_BYTES);
          if (SOFTMAX) {
            wgt[c][0] = fast_exp2((wgt[c][0] - mm[0]) * p.scale);
            wgt[c][1] = fast_exp2((wgt[c][1] - mm[1]) * p.scale);
            ll[0] += wgt[c][0] * pc[(NF * 4 + 2) * 32 + lane];
            ll[1] += wgt[c][1] * pc[(NF * 4 + 3) * 32 + lane];
          } else {
            wgt[c][0] = wgt[c][1] = 1.f;
          }
        }
        float inv0 = 1.f, inv1 = 1.f;
        if (SOFTMAX) {
          inv0 = (ll[0] > 0.f) ? 1.f / ll[0] : 0.f;
          inv1 = (ll[1] > 0.f) ? 1.f / ll[1] : 0.f;
          if (warp == 0) store_lse(p, it.head, it.window, mm, ll, lane);
        }
        for (int f = warp; f < NF; f += WARPS) {
          float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
          for (int c = 0; c < WARPS; ++c) {
            const float *pc = reinterpret_cast<const float *>(smem_raw + c * C::WARP_BYTES);
            a0 += wgt[c][0] * pc[(f * 4 + 0) * 32 + lane];
            a1 += wgt[c][0] * pc[(f * 4 + 1) * 32 + lane];
            a2 += wgt[c][1] * pc[(f * 4 + 2) * 32 + lane];
            a3 += wgt[c][1] * pc[(f * 4 + 3) * 32 + lane];
          }
          store_tile<D>(p, it.head, it.window, f, a0 * inv0, a1 * inv0, a2 * inv1, a3 * inv1, lane);
        }
      }
      __syncthreads();  // the partials are consumed before any staging area is refilled
    }

    if (my_steps >= 0 && my_steps <= thr) {  // this warp's own window, alone (an empty window stores zeros)
      float o[NF][4];
#pragma unroll
      for (int f = 0; f < NF; ++f) o[f][0] = o[f][1] = o[f][2] = o[f][3] = 0.f;
      float m_run[2] = {NEG_INF, NEG_INF};
      float l_run[2] = {0.f, 0.f};
      run_unit_cpasync<D, NT8, STAGES, WARPS, SOFTMAX>(p, ws, mine.head, mine.window, mine.t8b, mine.t8e, o, m_run,
                                                       l_run, lane);
      store_output<D, SOFTMAX>(p, mine.head, mine.window, o, m_run, l_run, lane);
    }
  }
  trace_end(p, lane);
}

// ---------------------------------------------------------------------------------------
// Data path 1b: cp.async with separate K and V rings (d = 64).  K of step i+1 is waited for
// and multiplied (S_next = Q K^T) *before* the softmax of step i, so the tensor-core latency
// of one step overlaps the ALU/SFU work of the previous one; V of step i is only needed
// after that softmax.  Two K buffers and two V buffers per warp -- the same shared memory
// as two combined stages.  Copy-group order: K0 V0 K1 | V1 K2 | V2 K3 | ...
// ---------------------------------------------------------------------------------------
template <int WARPS>
struct SplitCfg {
  static constexpr int D = 64, NT8 = 4, TILE_BYTES = 32 * D * 2, Q_BYTES = 16 * D * 2;
  static constexpr int WARP_BYTES = Q_BYTES + 4 * TILE_BYTES + 256;
  static constexpr int SMEM_BYTES = WARPS * WARP_BYTES;
  static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB of shared memory a CTA can have");
};

template <int WARPS, bool SOFTMAX, bool FILTER = false>
__global__ void __launch_bounds__(WARPS * 32, 1) fwd_kernel_split(const FwdParams p) {
  using C = SplitCfg<WARPS>;
  constexpr int D = C::D, NT8 = C::NT8, TILE = C::TILE_BYTES;
  using T = Tile<D>;
  constexpr int KS = D / 16, NF = D / 8;

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, qd = lane & 3;
  unsigned char *wsm = smem_raw + warp * C::WARP_BYTES;
  const uint32_t q_s = smem_u32(wsm);
  const uint32_t k_s = q_s + C::Q_BYTES;
  const uint32_t v_s = k_s + 2 * TILE;
  const uint32_t bm_s = v_s + 2 * TILE;
  const unsigned char *bm_g = wsm + C::Q_BYTES + 4 * TILE;
  const int bm_half = (g < 4) ? 1 : 0;
  const int bm_shift = 8 * (g & 3) + 2 * qd;
  // A lane copies chunk `ch` of rows 4i + rl, i = 0..7; the swizzled offset inside a tile only
  // depends on the parity of i.
  const int rl = lane >> 3, ch = lane & 7;
  const uint32_t off_even = rl * 128 + ((ch ^ rl) << 4);
  const uint32_t off_odd = rl * 128 + ((ch ^ (rl | 4)) << 4);
  const unsigned ld_bytes = (unsigned)(p.ld_kv * 2);

  trace_begin(p);
  UnitSource src;
  src.init(p, blockIdx.x * WARPS + warp, gridDim.x * WARPS);
  Unit u;
  while (src.next(p, lane, u)) {
    const int t8b = u.t8b, t8e = u.t8e;
    const int nsteps = (t8e - t8b + NT8 - 1) / NT8;
    const char *kb = reinterpret_cast<const char *>(p.k + (size_t)u.head * D + ch * 8);
    const char *vb = reinterpret_cast<const char *>(p.v + (size_t)u.head * D + ch * 8);
    float o[NF][4];
#pragma unroll
    for (int f = 0; f < NF; ++f) o[f][0] = o[f][1] = o[f][2] = o[f][3] = 0.f;
    float m_run[2] = {NEG_INF, NEG_INF};
    float l_run[2] = {0.f, 0.f};
    if (FILTER) load_state<D>(p, u, o, m_run, l_run, lane);
    // FILTER: which columns of the step being computed / the next / the one after take part
    uint32_t cm_cur = 0xffffffffu, cm_n1 = 0xffffffffu, cm_n2 = 0xffffffffu;

    if (nsteps > 0) {
      {  // Q window -> shared (first copy group); rows past the last node read as 0
        const int row0 = u.window * 16;
#pragma unroll
        for (int c = lane; c < 16 * T::CHUNKS; c += 32) {
          const int r = c / T::CHUNKS, cc = c % T::CHUNKS;
          const int gr = row0 + r;
          const bool ok = gr < p.n_nodes;
          const __half *srcq = p.q + (size_t)(ok ? gr : 0) * p.ld + (size_t)u.head * D + cc * 8;
          cp_async16(T::addr(q_s, r, cc), srcq, ok ? 16 : 0);
        }
      }
      // Column ids: lane l holds the id of row l of a step.  Rows beyond the unit carry id 0 (a
      // valid row); their tiles are masked because their bitmap words are zero-filled.
      int idx_next = 0, idx_kv = 0;
      {
        const int lim = (t8e - t8b) * 8;
        if (lane < lim) idx_next = __ldg(p.atox + (size_t)t8b * 8 + lane);
      }
      auto issue_k = [&](int step) {
        const uint32_t dst = k_s + (step & 1) * TILE;
        idx_kv = idx_next;
        if (FILTER) {
          const bool take = p.phase == 1 ? idx_kv >= p.col_split : idx_kv < p.col_split;
          cm_n2 = __ballot_sync(FULL, take);
          // first launch: columns that do not take part may not have arrived yet and are not read at all
          // (0 x stale NaN would poison the accumulator); they read an own row instead
          if (p.phase == 1 && !take) idx_kv = p.col_split;
        }
        {
          const int t8n = t8b + (step + 1) * NT8;
          const int limn = (t8e - t8n) * 8;
          idx_next = 0;
          if (lane < limn) idx_next = __ldg(p.atox + (size_t)t8n * 8 + lane);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const unsigned idx = (unsigned)__shfl_sync(FULL, idx_kv, i * 4 + rl);
          cp_async16(dst + i * 512 + ((i & 1) ? off_odd : off_even), kb + (size_t)idx * ld_bytes, 16);
        }
      };
      auto issue_v = [&](int step) {  // always follows issue_k(step): same ids
        const uint32_t dst = v_s + (step & 1) * TILE;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const unsigned idx = (unsigned)__shfl_sync(FULL, idx_kv, i * 4 + rl);
          cp_async16(dst + i * 512 + ((i & 1) ? off_odd : off_even), vb + (size_t)idx * ld_bytes, 16);
        }
        if (lane < NT8) {
          const int t8 = t8b + step * NT8 + lane;
          const bool ok = t8 < t8e;
          cp_async16(bm_s + (step & 1) * 128 + lane * 16, p.bitmap + (ok ? (size_t)t8 * 2 : 0), ok ? 16 : 0);
        }
      };
      issue_k(0);
      cp_async_commit();
      cm_cur = cm_n2;
      issue_v(0);
      cp_async_commit();
      if (nsteps > 1) issue_k(1);
      cp_async_commit();
      cm_n1 = cm_n2;
      cp_async_wait<2>();  // Q and K of step 0 have landed
      __syncwarp();
      uint32_t qa[KS][4];
      load_q_frags<D, SOFTMAX>(p, q_s, qa, lane);
      float s_cur[NT8][4];
      score_tiles<D, NT8>(k_s, qa, s_cur, lane);
#pragma unroll 2
      for (int step = 0; step < nsteps; ++step) {
        if (step + 1 < nsteps) issue_v(step + 1);
        cp_async_commit();
        if (step + 2 < nsteps) issue_k(step + 2);
        cp_async_commit();
        cp_async_wait<2>();  // K of step+1 and, before it, V and bitmap of this step have landed
        __syncwarp();
        float s_next[NT8][4];
        if (step + 1 < nsteps) score_tiles<D, NT8>(k_s + ((step + 1) & 1) * TILE, qa, s_next, lane);
        const uint32_t *bm32 = reinterpret_cast<const uint32_t *>(bm_g + (step & 1) * 128) + bm_half;
        const int t8 = t8b + step * NT8;
        softmax_pv<D, NT8, SOFTMAX, false, false, FILTER>(p, s_cur, v_s + (step & 1) * TILE, bm32,
                                                          min(NT8, t8e - t8), t8, o, m_run, l_run, lane, bm_shift,
                                                          cm_cur);
        cm_cur = cm_n1;
        cm_n1 = cm_n2;
        __syncwarp();  // this step's K, V and bitmap buffers may be refilled
#pragma unroll
        for (int nt = 0; nt < NT8; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) s_cur[nt][e] = s_next[nt][e];
      }
      cp_async_wait<0>();
    }
    finish_unit<D, SOFTMAX>(p, u, o, m_run, l_run, lane);
  }
  retire_warp(p, lane, gridDim.x * WARPS);
  trace_end(p, lane);
}

// ---------------------------------------------------------------------------------------
// Data path 2: TMA (d = 64).  Stage = 32 K rows + 32 V rows of 128 bytes, hardware
// 128-byte swizzle, 1024-byte-aligned tiles; two stages per warp; the Q window borrows the
// second stage's V tile until the first step has read it.
// ---------------------------------------------------------------------------------------
namespace tma {

__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after kWaitLimit polls (each poll itself blocks for a bounded,
// hardware-defined time) so that a lost completion can never hang the GPU.
constexpr int kWaitLimit = 1 << 22;
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
  for (int it = 0; it < kWaitLimit; ++it)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void gather4(uint32_t dst, const CUtensorMap *map, int x, int r0, int r1, int r2, int r3,
                                        uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, "
      "%4, %5, %6}], [%7];"
      ::"r"(dst), "l"(map), "r"(x), "r"(r0), "r"(r1), "r"(r2), "r"(r3), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void load_tile_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

constexpr int D = 64, NT8 = 4, ROWS = 32, TILE_BYTES = ROWS * 128, WARP_TILE_BYTES = 4 * TILE_BYTES;
constexpr int AUX_BYTES = 192;  // per warp: two 64-byte bitmap slots, two mbarriers, padding
__host__ __device__ constexpr int smem_bytes(int warps) { return warps * (WARP_TILE_BYTES + AUX_BYTES) + 1024; }

}  // namespace tma

template <int WARPS, bool SOFTMAX>
__global__ void __launch_bounds__(WARPS * 32, 1)
fwd_kernel_tma(const FwdParams p, const __grid_constant__ CUtensorMap tmq, const __grid_constant__ CUtensorMap tmk,
               const __grid_constant__ CUtensorMap tmv) {
  using namespace tma;
  using T = Tile<D>;
  constexpr int KS = D / 16, NF = D / 8;
  static_assert(smem_bytes(WARPS) <= 232448, "exceeds the 227 KB of shared memory a CTA can have");

  extern __shared__ unsigned char smem_raw[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, qd = lane & 3;
  const uint32_t base_s = (smem_u32(smem_raw) + 1023u) & ~1023u;  // tiles must sit on 1024-byte boundaries
  unsigned char *base_g = smem_raw + (base_s - smem_u32(smem_raw));
  const uint32_t tiles_s = base_s + warp * WARP_TILE_BYTES;  // [K0][V0][K1][V1]
  const uint32_t aux_s = base_s + WARPS * WARP_TILE_BYTES + warp * AUX_BYTES;
  const unsigned char *aux_g = base_g + WARPS * WARP_TILE_BYTES + warp * AUX_BYTES;
  const uint32_t bar_s = aux_s + 128;   // two mbarriers
  const uint32_t q_s = tiles_s + 3 * TILE_BYTES;  // Q window borrows stage 1's V tile
  const int bm_half = (g < 4) ? 1 : 0;
  const int bm_shift = 8 * (g & 3) + 2 * qd;

  if (lane == 0) {
    mbar_init(bar_s, 1);
    mbar_init(bar_s + 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  uint32_t phase = 0;  // bit s: parity to wait for on stage s

  trace_begin(p);
  UnitSource src;
  src.init(p, blockIdx.x * WARPS + warp, gridDim.x * WARPS);
  Unit u;
  while (src.next(p, lane, u)) {
    const int t8b = u.t8b, t8e = u.t8e;
    const int nsteps = (t8e - t8b + NT8 - 1) / NT8;
    const int xcol = u.head * D;
    float o[NF][4];
#pragma unroll
    for (int f = 0; f < NF; ++f) o[f][0] = o[f][1] = o[f][2] = o[f][3] = 0.f;
    float m_run[2] = {NEG_INF, NEG_INF};
    float l_run[2] = {0.f, 0.f};

    if (nsteps > 0) {
      int idx_next = 0;  // column id of row `lane` of the next step to be issued
      {
        const int lim = (t8e - t8b) * 8;
        if (lane < lim) idx_next = __ldg(p.atox + (size_t)t8b * 8 + lane);
      }
      // Issue the copies of one step into stage step&1; extra_bytes accounts for the Q tile.
      auto issue = [&](int step, uint32_t extra_bytes) {
        const int t8 = t8b + step * NT8;
        const int st = step & 1;
        const uint32_t ks = tiles_s + st * 2 * TILE_BYTES;
        const uint32_t vs = ks + TILE_BYTES;
        const uint32_t bar = bar_s + st * 8;
        const int tiles_here = min(NT8, t8e - t8);
        const int idx_cur = idx_next;  // rows outside the unit carry id 0: a valid row, masked later
        {
          const int t8n = t8 + NT8;
          const int limn = (t8e - t8n) * 8;
          idx_next = 0;
          if (lane < limn) idx_next = __ldg(p.atox + (size_t)t8n * 8 + lane);
        }
        const int r1 = __shfl_down_sync(FULL, idx_cur, 1);
        const int r2 = __shfl_down_sync(FULL, idx_cur, 2);
        const int r3 = __shfl_down_sync(FULL, idx_cur, 3);
        if (lane == 0) {
          mbar_expect_tx(bar, 2 * TILE_BYTES + tiles_here * 16 + extra_bytes);
          bulk_copy(aux_s + st * 64, p.bitmap + (size_t)t8 * 2, tiles_here * 16, bar);
        }
        if ((lane & 3) == 0) {  // eight lanes, four gathered rows each
          gather4(ks + lane * 128, &tmk, xcol, idx_cur, r1, r2, r3, bar);
          gather4(vs + lane * 128, &tmv, xcol, idx_cur, r1, r2, r3, bar);
        }
      };
      if (lane == 0) load_tile_2d(q_s, &tmq, xcol, u.window * 16, bar_s);  // completes on stage 0's barrier
      issue(0, 16 * D * 2);

      uint32_t qa[KS][4];
      bool ok = true;
      for (int step = 0; step < nsteps; ++step) {
        const int st = step & 1;
        if (step > 0 && step + 1 < nsteps) issue(step + 1, 0);
        const bool landed = mbar_wait_bounded(bar_s + st * 8, (phase >> st) & 1u);
        if (!__all_sync(FULL, landed)) {
          // completion lost: flag it, give in-flight copies one more bounded chance to land, leave
          atomicExch(&p.hdr[HDR_STATUS], STATUS_WAIT_TIMEOUT);
          mbar_wait_bounded(bar_s + st * 8, (phase >> st) & 1u);
          ok = false;
          break;
        }
        phase ^= 1u << st;
        if (step == 0) {
          load_q_frags<D, SOFTMAX>(p, q_s, qa, lane);
          __syncwarp();  // all lanes hold their Q fragments before the tile is overwritten
          if (nsteps > 1) issue(1, 0);
        }
        const uint32_t ksm = tiles_s + st * 2 * TILE_BYTES;
        const uint32_t vsm = ksm + TILE_BYTES;
        const uint32_t *bm32 = reinterpret_cast<const uint32_t *>(aux_g + st * 64) + bm_half;
        const int t8 = t8b + step * NT8;
        compute_step<D, NT8, SOFTMAX, true>(p, ksm, vsm, bm32, min(NT8, t8e - t8), t8, qa, o, m_run, l_run, lane,
                                            bm_shift);
        __syncwarp();  // every lane is done with this stage before it is refilled
      }
      if (!ok) return;
    }
    finish_unit<D, SOFTMAX>(p, u, o, m_run, l_run, lane);
  }
  retire_warp(p, lane, gridDim.x * WARPS);
  trace_end(p, lane);
}

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
enum DataPath { PATH_CPASYNC = 0, PATH_SPLIT = 1, PATH_TMA = 2 };

struct KernelCfg {
  int nt8, stages, warps;
  int path;
};

// Kernel choice per head dimension.  d = 64 defaults to the cp.async kernel with separate K and
// V rings (measured fastest on B200).  F3S_FWD_PATH=cpasync | split | tma (environment, read once)
// selects another data path for d = 64; the parity tests run every path.
static KernelCfg kernel_cfg(int d) {
  if (d == 32) return {4, 2, 16, PATH_CPASYNC};  // 16 warps with two stages beat 8 warps with four
  if (d == 128) return {2, 2, 8, PATH_CPASYNC};  // 8 warps on 16-column steps beat 4 warps on 32-column steps
  static const int path = [] {
    const char *e = getenv("F3S_FWD_PATH");
    if (e && strcmp(e, "cpasync") == 0) return (int)PATH_CPASYNC;
    if (e && strcmp(e, "tma") == 0) return (int)PATH_TMA;
    return (int)PATH_SPLIT;
  }();
  return {4, 2, 12, path};
}

struct Geometry {
  KernelCfg kc;
  int direct;
  int ch8;         // split threshold / chunk size in 8-column tiles
  int max_slots;   // partial slots per head == capacity of the unit list
  size_t off_hdr, off_arrive, off_units, off_partial, total_bytes;
  size_t zero_bytes;  // header + arrival counters, cleared at the start of every scheduled call
};

constexpr int UNITS_PER_WARP = 6;  // chunks of heavy windows per warp: 3..8 measure within 2 % of each other, 12+ lose 3-10 %
constexpr int MIN_CH8 = 64;
constexpr int DIRECT_TILES_PER_WARP = 32;  // below this average load the schedule costs more than it saves
constexpr int MAX_BUDGET_CH8 = 1 << 16;    // largest chunk (in 8-column tiles) a budgeted schedule may use

// Head dimensions: any multiple of 16 up to 128.  The kernels are compiled for 32, 64 and 128;
// other sizes run in the next larger one with the missing feature chunks zero-filled on the way
// into shared memory (they add 0 to every score and produce output columns that are not stored).
static bool dim_supported(int d) { return d >= 16 && d <= 128 && d % 16 == 0; }
static int padded_dim(int d) { return d <= 32 ? 32 : (d <= 64 ? 64 : 128); }

static void layout(Geometry &gm, long long total_t8, int heads, int d) {
  // Capacity of the unit list.  A heavy window of n > ch8 tiles is cut into at most n / ch8 + 1 <= 2 n / ch8
  // chunks, so all heavy windows together need at most 2 * total / ch8 entries: the list cannot overflow
  // (plan_kernel still checks and flags it in the header).
  gm.max_slots = gm.direct ? 0 : (int)(2 * total_t8 / gm.ch8 + 2);
  const size_t partial_floats = (size_t)((d / 8) * 4 + 4) * 32;
  size_t off = 0;
  gm.off_hdr = off; off += HDR_INTS * sizeof(int);
  gm.off_arrive = off; off += (size_t)gm.max_slots * heads * sizeof(int);
  gm.zero_bytes = off;
  off = align_up(off, 256);
  gm.off_units = off; off = align_up(off + (size_t)gm.max_slots * sizeof(UnitDesc), 256);
  gm.off_partial = off; off = align_up(off + (size_t)gm.max_slots * heads * partial_floats * sizeof(float), 256);
  gm.total_bytes = off;
}

// budget_bytes > 0: raise the split threshold (fewer, larger chunks) until the scratch fits.
// Canonical schedule (f3s_set_canonical_chunk_tiles): 0 = off.
static int g_canonical_ch8 = 0;
extern "C" void f3s_set_canonical_chunk_tiles(int32_t tiles) { g_canonical_ch8 = tiles > 0 ? tiles : 0; }

// phased: geometry of one launch of a two-phase call -- always scheduled (never the one-launch mode), never
// the TMA path, and room in the unit list for the TC block per window that both launches work on.
static Geometry geometry(int n_rw, long long n_tcb, int block_w, int heads, int d, size_t budget_bytes = 0,
                         bool phased = false) {
  Geometry gm;
  const int d_real = d;
  d = padded_dim(d);
  gm.kc = kernel_cfg(d);
  if (d_real != d) gm.kc.path = PATH_CPASYNC;  // only the plain kernel zero-fills padded chunks
  if (phased && gm.kc.path == PATH_TMA) gm.kc.path = PATH_SPLIT;
  const long long total_t8 = (n_tcb + (phased ? n_rw : 0)) * (block_w / 8);
  const long long total_warps = (long long)sm_count() * gm.kc.warps;
  const bool canonical = g_canonical_ch8 > 0;
  gm.direct = (!phased && !canonical && total_t8 * heads <= total_warps * DIRECT_TILES_PER_WARP) ? 1 : 0;
  // Many short windows (fewer than four 32-column steps on average, e.g. batches of small graphs):
  // the split-ring kernel's longer prologue costs more than its overlap gains (measured 0.31 vs
  // 0.21 ms on the molecule-batch workload), so the plain two-stage kernel is used there.
  if (gm.kc.path == PATH_SPLIT && !gm.direct && !canonical && total_t8 < 16ll * n_rw) gm.kc.path = PATH_CPASYNC;
  long long ch = (total_t8 * heads) / (total_warps * UNITS_PER_WARP);
  if (canonical) ch = g_canonical_ch8;  // the same cut points whatever the load, the head count or the device
  ch = (ch + gm.kc.nt8 - 1) / gm.kc.nt8 * gm.kc.nt8;
  if (ch < MIN_CH8 && !canonical) ch = MIN_CH8;
  if (ch > (1 << 28)) ch = 1 << 28;
  gm.ch8 = (int)ch;
  layout(gm, total_t8, heads, d);
  if (canonical) return gm;  // no growing of chunks to fit a budget: the call is refused if the scratch is too small
  // With a budget the chunks may grow, but only up to MAX_BUDGET_CH8 tiles: beyond that a single
  // warp would walk hundreds of thousands of columns on its own and the call is refused instead.
  while (budget_bytes > 0 && gm.total_bytes > budget_bytes && gm.ch8 * 2 <= MAX_BUDGET_CH8) {
    gm.ch8 *= 2;
    layout(gm, total_t8, heads, d);
  }
  return gm;
}

template <int D, int NT8, int STAGES, int WARPS>
static int launch(const FwdParams &p, bool softmax, int grid, cudaStream_t stream) {
  using C = FwdCfg<D, NT8, STAGES, WARPS>;
  if (p.phase != 0) {  // two-phase calls exist with softmax only
    if constexpr (D == 64) {
      auto kern = fwd_kernel<D, NT8, STAGES, WARPS, true, true>;
      F3S_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
      kern<<<grid, WARPS * 32, C::SMEM_BYTES, stream>>>(p);
      F3S_CHECK_LAUNCH();
      return F3S_OK;
    } else {
      set_error("two-phase calls need head_dim 64");
      return F3S_ERR_UNSUPPORTED;
    }
  }
  if (softmax) {
    auto kern = fwd_kernel<D, NT8, STAGES, WARPS, true>;
    F3S_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    kern<<<grid, WARPS * 32, C::SMEM_BYTES, stream>>>(p);
  } else {
    auto kern = fwd_kernel<D, NT8, STAGES, WARPS, false>;
    F3S_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    kern<<<grid, WARPS * 32, C::SMEM_BYTES, stream>>>(p);
  }
  F3S_CHECK_LAUNCH();
  return F3S_OK;
}

template <int D, int NT8, int STAGES, int WARPS>
static int launch_coop(const FwdParams &p, bool softmax, int grid, cudaStream_t stream) {
  using C = FwdCfg<D, NT8, STAGES, WARPS>;
  if (softmax) {
    auto kern = fwd_kernel_coop<D, NT8, STAGES, WARPS, true>;
    F3S_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    kern<<<grid, WARPS * 32, C::SMEM_BYTES, stream>>>(p);
  } else {
    auto kern = fwd_kernel_coop<D, NT8, STAGES, WARPS, false>;
    F3S_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    kern<<<grid, WARPS * 32, C::SMEM_BYTES, stream>>>(p);
  }
  F3S_CHECK_LAUNCH();
  return F3S_OK;
}

// cuTensorMapEncodeTiled, looked up through the runtime so that libcuda need not be linked.
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      ptr = nullptr;
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

// 2-D fp16 tensor map over rows of `ld` elements; box = box_cols x box_rows, 128-byte swizzle.
static int make_map(CUtensorMap *m, const void *base, long long ld, unsigned long long rows, int box_cols,
                    int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  F3S_REQUIRE(fn != nullptr, F3S_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {(cuuint64_t)ld, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  F3S_REQUIRE(r == CUDA_SUCCESS, F3S_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return F3S_OK;
}

template <int WARPS>
static int launch_tma(const FwdParams &p, bool softmax, int grid, cudaStream_t stream) {
  CUtensorMap tmq, tmk, tmv;
  // Q: exact row count, so that rows past the last node are zero-filled by the hardware.
  if (int rc = make_map(&tmq, p.q, p.ld, (unsigned long long)p.n_nodes, 64, 16)) return rc;
  // K, V: the row count is not an argument of the C ABI; every column id must have a row.
  if (int rc = make_map(&tmk, p.k, p.ld_kv, 1ull << 31, 64, 1)) return rc;
  if (int rc = make_map(&tmv, p.v, p.ld_kv, 1ull << 31, 64, 1)) return rc;
  const int smem = tma::smem_bytes(WARPS);
  if (softmax) {
    auto kern = fwd_kernel_tma<WARPS, true>;
    F3S_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    kern<<<grid, WARPS * 32, smem, stream>>>(p, tmq, tmk, tmv);
  } else {
    auto kern = fwd_kernel_tma<WARPS, false>;
    F3S_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    kern<<<grid, WARPS * 32, smem, stream>>>(p, tmq, tmk, tmv);
  }
  F3S_CHECK_LAUNCH();
  return F3S_OK;
}

template <int WARPS>
static int launch_split(const FwdParams &p, bool softmax, int grid, cudaStream_t stream) {
  using C = SplitCfg<WARPS>;
  if (p.phase != 0) {  // two-phase calls exist with softmax only
    auto kern = fwd_kernel_split<WARPS, true, true>;
    F3S_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    kern<<<grid, WARPS * 32, C::SMEM_BYTES, stream>>>(p);
    F3S_CHECK_LAUNCH();
    return F3S_OK;
  }
  if (softmax) {
    auto kern = fwd_kernel_split<WARPS, true>;
    F3S_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    kern<<<grid, WARPS * 32, C::SMEM_BYTES, stream>>>(p);
  } else {
    auto kern = fwd_kernel_split<WARPS, false>;
    F3S_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    kern<<<grid, WARPS * 32, C::SMEM_BYTES, stream>>>(p);
  }
  F3S_CHECK_LAUNCH();
  return F3S_OK;
}

}  // namespace f3s

using namespace f3s;

extern "C" size_t f3s_forward_workspace_bytes(int32_t n_row_windows, int64_t n_tcb, int32_t block_w, int32_t heads,
                                              int32_t head_dim) {
  if (n_row_windows < 0 || n_tcb < 0 || heads < 1 || (block_w != 8 && block_w != 16)) return 0;
  if (!dim_supported(head_dim)) return 0;
  return geometry(n_row_windows, n_tcb, block_w, heads, head_dim).total_bytes;
}

// Testing aid: caps the capacity of the schedule's unit list (0 = no cap), so that the overflow report
// of the schedule kernel can be exercised.  Process-wide.
static int g_unit_list_limit = 0;
extern "C" void f3s_debug_set_unit_list_limit(int32_t limit) { g_unit_list_limit = limit > 0 ? limit : 0; }

// Options of the entry points that go beyond f3s_forward.
struct FwdExtra {
  int64_t ld_kv = 0;                  // row stride of k and v (0: same as q's)
  int mode = 0;                       // 0: schedule + launch; 1: schedule only; 2: launch on a scratch scheduled before
  int phase = 0, col_split = 0;       // see FwdParams
  const int32_t *phase_split = nullptr;
  float *state = nullptr;
};
enum { MODE_FULL = 0, MODE_PLAN_ONLY = 1, MODE_PLANNED = 2 };

// Co-scheduling aid: the persistent kernels normally take one CTA on every SM, which leaves a collective
// that is launched beside them (NCCL's kernels need SMs of their own) waiting until they finish.  A cap
// below the SM count keeps that many SMs free.  0 = no cap.  Process-wide; the environment variable
// F3S_MAX_CTAS gives the initial value.
static int g_max_ctas = [] {
  const char *e = getenv("F3S_MAX_CTAS");
  const int v = e ? atoi(e) : 0;
  return v > 0 ? v : 0;
}();
extern "C" int32_t f3s_set_max_ctas(int32_t max_ctas) {
  const int previous = g_max_ctas;
  g_max_ctas = max_ctas > 0 ? max_ctas : 0;
  return previous;
}

// Validation + launch shared by the entry points.  budget_bytes > 0 lets the schedule use
// fewer, larger chunks so that its scratch fits in that many bytes.
static int forward_impl(const int32_t *row_window_offset, const int32_t *sorted_row_windows,
                        const int32_t *sparse_a_to_x_idx, const uint64_t *tcb_bitmap, int32_t num_nodes,
                        int32_t n_row_windows, int64_t n_tcb, int32_t block_w, int32_t heads, int32_t head_dim,
                        int64_t ld, const void *q, const void *k, const void *v, float scale_divisor,
                        int32_t apply_softmax, void *out, int out_is_half, float *sddmm_out, void *workspace,
                        size_t workspace_bytes, size_t budget_bytes, uint64_t *sm_trace, float *lse,
                        f3s_stream_t stream_, const FwdExtra *extra = nullptr) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const FwdExtra ex = extra ? *extra : FwdExtra{};
  const int64_t ld_kv = ex.ld_kv > 0 ? ex.ld_kv : ld;
  const bool plan_only = ex.mode == MODE_PLAN_ONLY;
  F3S_REQUIRE(num_nodes >= 0 && n_row_windows >= 0 && n_tcb >= 0, F3S_ERR_INVALID_ARG, "negative size");
  F3S_REQUIRE(n_row_windows == (num_nodes + 15) / 16, F3S_ERR_INVALID_ARG,
              "n_row_windows (%d) must be ceil(num_nodes/16) (%d)", n_row_windows, (num_nodes + 15) / 16);
  F3S_REQUIRE(block_w == 8 || block_w == 16, F3S_ERR_UNSUPPORTED, "block_w must be 8 or 16, got %d", block_w);
  F3S_REQUIRE(dim_supported(head_dim), F3S_ERR_UNSUPPORTED,
              "head_dim must be a multiple of 16 between 16 and 128, got %d", head_dim);
  F3S_REQUIRE(heads >= 1, F3S_ERR_INVALID_ARG, "heads must be >= 1");
  F3S_REQUIRE(plan_only || (ld >= (int64_t)heads * head_dim && ld % 8 == 0 && ld_kv >= (int64_t)heads * head_dim &&
                            ld_kv % 8 == 0),
              F3S_ERR_INVALID_ARG, "row strides (%lld, %lld) must be >= heads*head_dim and multiples of 8",
              (long long)ld, (long long)ld_kv);
  F3S_REQUIRE(plan_only || (scale_divisor != 0.f && isfinite(scale_divisor)), F3S_ERR_INVALID_ARG,
              "scale_divisor must be finite and non-zero");
  F3S_REQUIRE(n_tcb * block_w < (1ll << 31), F3S_ERR_UNSUPPORTED, "n_tcb*block_w exceeds int32");
  F3S_REQUIRE(ex.phase >= 0 && ex.phase <= 2, F3S_ERR_INVALID_ARG, "phase must be 0, 1 or 2");
  F3S_REQUIRE(ex.phase == 0 || (head_dim == 64 && apply_softmax && ex.phase_split && (plan_only || ex.state)),
              F3S_ERR_UNSUPPORTED, "two-phase calls need head_dim 64, softmax, phase_split and a state array");
  if (num_nodes == 0) return F3S_OK;
  F3S_REQUIRE(row_window_offset, F3S_ERR_INVALID_ARG, "null pointer argument");
  auto misaligned = [](const void *ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) != 0; };
  if (!plan_only) {
    F3S_REQUIRE(q && k && v && (out || ex.phase == 1), F3S_ERR_INVALID_ARG, "null pointer argument");
    F3S_REQUIRE(n_tcb == 0 || (sparse_a_to_x_idx && tcb_bitmap), F3S_ERR_INVALID_ARG, "null TCB array");
    F3S_REQUIRE(sddmm_out == nullptr || heads == 1, F3S_ERR_INVALID_ARG, "sddmm_out needs heads == 1");
    F3S_REQUIRE(!misaligned(q) && !misaligned(k) && !misaligned(v) && !misaligned(out) && !misaligned(tcb_bitmap),
                F3S_ERR_INVALID_ARG, "q, k, v, out and tcb_bitmap must be 16-byte aligned");
  }
  Geometry gm = geometry(n_row_windows, n_tcb, block_w, heads, head_dim, budget_bytes, ex.phase != 0);
  if (!gm.direct && g_unit_list_limit > 0 && gm.max_slots > g_unit_list_limit) gm.max_slots = g_unit_list_limit;
  F3S_REQUIRE(workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 255) == 0, F3S_ERR_WORKSPACE,
              "workspace must be non-null and 256-byte aligned");
  F3S_REQUIRE(workspace_bytes >= gm.total_bytes, F3S_ERR_WORKSPACE, "workspace too small: %zu < %zu",
              workspace_bytes, gm.total_bytes);

  unsigned char *ws = static_cast<unsigned char *>(workspace);
  FwdParams p;
  p.rwo = row_window_offset;
  p.sorted = sorted_row_windows;
  p.atox = sparse_a_to_x_idx;
  p.bitmap = reinterpret_cast<const unsigned long long *>(tcb_bitmap);
  p.q = static_cast<const __half *>(q);
  p.k = static_cast<const __half *>(k);
  p.v = static_cast<const __half *>(v);
  p.out = out_is_half ? nullptr : static_cast<float *>(out);
  p.out_h = out_is_half ? static_cast<__half *>(out) : nullptr;
  p.sddmm = sddmm_out;
  p.lse = lse;
  p.n_nodes = num_nodes;
  p.n_rw = n_row_windows;
  p.heads = heads;
  p.d_real = head_dim;
  p.ld = ld;
  p.ld_kv = ld_kv;
  p.phase = ex.phase;
  p.col_split = ex.col_split;
  p.phase_split = ex.phase_split;
  p.state = ex.state;
  p.t8_per_tcb = block_w / 8;
  p.direct = gm.direct;
  p.ch8 = gm.direct ? INT_MAX : gm.ch8;
  const float inv = 1.f / scale_divisor;
  p.negate_q = (apply_softmax && inv < 0.f) ? 1 : 0;
  p.scale = apply_softmax ? fabsf(inv) * 1.4426950408889634f : inv;
  p.hdr = reinterpret_cast<int *>(ws + gm.off_hdr);
  p.units = reinterpret_cast<const UnitDesc *>(ws + gm.off_units);
  p.arrive = reinterpret_cast<int *>(ws + gm.off_arrive);
  p.partial = reinterpret_cast<float *>(ws + gm.off_partial);
  p.max_slots = gm.max_slots;
  p.sm_trace = reinterpret_cast<unsigned long long *>(sm_trace);

  int grid = sm_count();
  if (g_max_ctas > 0 && grid > g_max_ctas) grid = g_max_ctas;
  if (gm.direct) {  // one launch; no more CTAs than there are (head, window) pairs
    const long long units = (long long)n_row_windows * heads;
    if (units < grid) grid = (int)(units > 0 ? units : 1);
  } else if (ex.mode != MODE_PLANNED) {
    F3S_CUDA_TRY(cudaMemsetAsync(ws + gm.off_hdr, 0, gm.zero_bytes, stream));
    plan_kernel<<<(n_row_windows + PLAN_THREADS - 1) / PLAN_THREADS, PLAN_THREADS, 0, stream>>>(
        PlanArgs{row_window_offset, ex.phase, ex.phase_split}, sorted_row_windows, n_row_windows, p.t8_per_tcb,
        gm.ch8, gm.kc.nt8, p.hdr, reinterpret_cast<UnitDesc *>(ws + gm.off_units), gm.max_slots);
    F3S_CHECK_LAUNCH();
  }
  if (plan_only) return F3S_OK;
  const bool sm = apply_softmax != 0;
  const KernelCfg kc = gm.kc;
  if (gm.direct) {
#define F3S_LAUNCH_COOP(D_, N_, S_, W_) \
  if (padded_dim(head_dim) == D_ && kc.nt8 == N_ && kc.stages == S_ && kc.warps == W_) return launch_coop<D_, N_, S_, W_>(p, sm, grid, stream)
    F3S_LAUNCH_COOP(32, 4, 2, 16);
    F3S_LAUNCH_COOP(128, 2, 2, 8);
    F3S_LAUNCH_COOP(64, 4, 2, 12);
#undef F3S_LAUNCH_COOP
  }
  // the score dump is only implemented in the plain cp.async kernel
  if (head_dim == 64 && sddmm_out == nullptr) {
    if (kc.path == PATH_SPLIT) return launch_split<12>(p, sm, grid, stream);
    if (kc.path == PATH_TMA) return launch_tma<12>(p, sm, grid, stream);
  }
#define F3S_LAUNCH(D_, N_, S_, W_) \
  if (padded_dim(head_dim) == D_ && kc.nt8 == N_ && kc.stages == S_ && kc.warps == W_) return launch<D_, N_, S_, W_>(p, sm, grid, stream)
  F3S_LAUNCH(32, 4, 2, 16);
  F3S_LAUNCH(128, 2, 2, 8);
  F3S_LAUNCH(64, 4, 2, 12);
#undef F3S_LAUNCH
  set_error("no kernel instance for head_dim %d", head_dim);
  return F3S_ERR_UNSUPPORTED;
}

extern "C" int f3s_forward(const int32_t *row_window_offset, const int32_t *sorted_row_windows,
                           const int32_t *sparse_a_to_x_idx, const uint64_t *tcb_bitmap, int32_t num_nodes,
                           int32_t n_row_windows, int64_t n_tcb, int32_t block_w, int32_t heads, int32_t head_dim,
                           int64_t ld, const void *q, const void *k, const void *v, float scale_divisor,
                           int32_t apply_softmax, float *out, float *sddmm_out, void *workspace,
                           size_t workspace_bytes, f3s_stream_t stream) {
  return forward_impl(row_window_offset, sorted_row_windows, sparse_a_to_x_idx, tcb_bitmap, num_nodes, n_row_windows,
                      n_tcb, block_w, heads, head_dim, ld, q, k, v, scale_divisor, apply_softmax, out, 0, sddmm_out,
                      workspace, workspace_bytes, 0, nullptr, nullptr, stream);
}

// f3s_forward with an fp16 output tensor (halves the output bytes; for layers that consume fp16).
extern "C" int f3s_forward_f16out(const int32_t *row_window_offset, const int32_t *sorted_row_windows,
                                  const int32_t *sparse_a_to_x_idx, const uint64_t *tcb_bitmap, int32_t num_nodes,
                                  int32_t n_row_windows, int64_t n_tcb, int32_t block_w, int32_t heads,
                                  int32_t head_dim, int64_t ld, const void *q, const void *k, const void *v,
                                  float scale_divisor, int32_t apply_softmax, void *out_f16, void *workspace,
                                  size_t workspace_bytes, f3s_stream_t stream) {
  return forward_impl(row_window_offset, sorted_row_windows, sparse_a_to_x_idx, tcb_bitmap, num_nodes, n_row_windows,
                      n_tcb, block_w, heads, head_dim, ld, q, k, v, scale_divisor, apply_softmax, out_f16, 1, nullptr,
                      workspace, workspace_bytes, 0, nullptr, nullptr, stream);
}

// f3s_forward that also returns, per row and head, the log2-domain log-sum-exp of the scaled scores
// (what a backward pass needs to recompute the probabilities): lse[row * heads + head].
extern "C" int f3s_forward_lse(const int32_t *row_window_offset, const int32_t *sorted_row_windows,
                               const int32_t *sparse_a_to_x_idx, const uint64_t *tcb_bitmap, int32_t num_nodes,
                               int32_t n_row_windows, int64_t n_tcb, int32_t block_w, int32_t heads, int32_t head_dim,
                               int64_t ld, const void *q, const void *k, const void *v, float scale_divisor,
                               float *out, float *lse, void *workspace, size_t workspace_bytes,
                               f3s_stream_t stream) {
  F3S_REQUIRE(lse != nullptr || num_nodes == 0, F3S_ERR_INVALID_ARG, "null lse");
  return forward_impl(row_window_offset, sorted_row_windows, sparse_a_to_x_idx, tcb_bitmap, num_nodes, n_row_windows,
                      n_tcb, block_w, heads, head_dim, ld, q, k, v, scale_divisor, 1, out, 0, nullptr, workspace,
                      workspace_bytes, 0, nullptr, lse, stream);
}

// f3s_forward plus a per-SM busy-interval trace (see trace_begin / trace_end).
extern "C" int f3s_forward_traced(const int32_t *row_window_offset, const int32_t *sorted_row_windows,
                                  const int32_t *sparse_a_to_x_idx, const uint64_t *tcb_bitmap, int32_t num_nodes,
                                  int32_t n_row_windows, int64_t n_tcb, int32_t block_w, int32_t heads,
                                  int32_t head_dim, int64_t ld, const void *q, const void *k, const void *v,
                                  float scale_divisor, int32_t apply_softmax, float *out, void *workspace,
                                  size_t workspace_bytes, uint64_t *sm_trace, f3s_stream_t stream) {
  F3S_REQUIRE(sm_trace != nullptr, F3S_ERR_INVALID_ARG, "null sm_trace");
  return forward_impl(row_window_offset, sorted_row_windows, sparse_a_to_x_idx, tcb_bitmap, num_nodes, n_row_windows,
                      n_tcb, block_w, heads, head_dim, ld, q, k, v, scale_divisor, apply_softmax, out, 0, nullptr,
                      workspace, workspace_bytes, 0, sm_trace, nullptr, stream);
}

// ---------------------------------------------------------------------------------------
// Repeated calls on one graph: schedule once, then one kernel launch per call.
// ---------------------------------------------------------------------------------------
extern "C" int f3s_forward_plan(const int32_t *row_window_offset, const int32_t *sorted_row_windows,
                                int32_t num_nodes, int32_t n_row_windows, int64_t n_tcb, int32_t block_w,
                                int32_t heads, int32_t head_dim, void *workspace, size_t workspace_bytes,
                                f3s_stream_t stream) {
  FwdExtra ex;
  ex.mode = MODE_PLAN_ONLY;
  return forward_impl(row_window_offset, sorted_row_windows, nullptr, nullptr, num_nodes, n_row_windows, n_tcb,
                      block_w, heads, head_dim, 0, nullptr, nullptr, nullptr, 1.f, 1, nullptr, 0, nullptr, workspace,
                      workspace_bytes, 0, nullptr, nullptr, stream, &ex);
}

extern "C" int f3s_forward_planned(const int32_t *row_window_offset, const int32_t *sorted_row_windows,
                                   const int32_t *sparse_a_to_x_idx, const uint64_t *tcb_bitmap, int32_t num_nodes,
                                   int32_t n_row_windows, int64_t n_tcb, int32_t block_w, int32_t heads,
                                   int32_t head_dim, int64_t ld_q, const void *q, int64_t ld_kv, const void *k,
                                   const void *v, float scale_divisor, int32_t apply_softmax, void *out,
                                   int32_t out_is_half, void *workspace, size_t workspace_bytes,
                                   f3s_stream_t stream) {
  FwdExtra ex;
  ex.mode = MODE_PLANNED;
  ex.ld_kv = ld_kv;
  return forward_impl(row_window_offset, sorted_row_windows, sparse_a_to_x_idx, tcb_bitmap, num_nodes, n_row_windows,
                      n_tcb, block_w, heads, head_dim, ld_q, q, k, v, scale_divisor, apply_softmax, out,
                      out_is_half ? 1 : 0, nullptr, workspace, workspace_bytes, 0, nullptr, nullptr, stream, &ex);
}

// ---------------------------------------------------------------------------------------
// Two-phase calls: first the columns a rank already holds, then -- once they have arrived -- the rest.
// Scratch: [schedule of phase 1][schedule of phase 2][state of every (head, window)].
// ---------------------------------------------------------------------------------------
namespace {
struct PhasedLayout {
  size_t sched_bytes, off_state, total;
};
PhasedLayout phased_layout(int n_rw, long long n_tcb, int block_w, int heads, int d) {
  PhasedLayout L;
  L.sched_bytes = align_up(geometry(n_rw, n_tcb, block_w, heads, d, 0, true).total_bytes, 256);
  L.off_state = 2 * L.sched_bytes;
  const size_t partial_floats = (size_t)((padded_dim(d) / 8) * 4 + 4) * 32;
  L.total = L.off_state + align_up((size_t)n_rw * heads * partial_floats * sizeof(float), 256);
  return L;
}
}  // namespace

extern "C" size_t f3s_forward_phased_workspace_bytes(int32_t n_row_windows, int64_t n_tcb, int32_t block_w,
                                                     int32_t heads, int32_t head_dim) {
  if (n_row_windows < 0 || n_tcb < 0 || heads < 1 || (block_w != 8 && block_w != 16) || head_dim != 64) return 0;
  return phased_layout(n_row_windows, n_tcb, block_w, heads, head_dim).total;
}

extern "C" int f3s_forward_phased_plan(const int32_t *row_window_offset, const int32_t *sorted_row_windows,
                                       const int32_t *phase_split, int32_t num_nodes, int32_t n_row_windows,
                                       int64_t n_tcb, int32_t block_w, int32_t heads, int32_t head_dim,
                                       void *workspace, size_t workspace_bytes, f3s_stream_t stream) {
  F3S_REQUIRE(head_dim == 64, F3S_ERR_UNSUPPORTED, "two-phase calls need head_dim 64");
  F3S_REQUIRE(n_row_windows >= 0 && n_tcb >= 0 && heads >= 1 && (block_w == 8 || block_w == 16), F3S_ERR_INVALID_ARG,
              "bad size");
  const PhasedLayout L = phased_layout(n_row_windows, n_tcb, block_w, heads, head_dim);
  F3S_REQUIRE(workspace && workspace_bytes >= L.total, F3S_ERR_WORKSPACE, "workspace too small: %zu < %zu",
              workspace_bytes, L.total);
  unsigned char *ws = static_cast<unsigned char *>(workspace);
  for (int phase = 1; phase <= 2; ++phase) {
    FwdExtra ex;
    ex.mode = MODE_PLAN_ONLY;
    ex.phase = phase;
    ex.phase_split = phase_split;
    if (int rc = forward_impl(row_window_offset, sorted_row_windows, nullptr, nullptr, num_nodes, n_row_windows, n_tcb,
                              block_w, heads, head_dim, 0, nullptr, nullptr, nullptr, 1.f, 1, nullptr, 0, nullptr,
                              ws + (phase - 1) * L.sched_bytes, L.sched_bytes, 0, nullptr, nullptr, stream, &ex))
      return rc;
  }
  return F3S_OK;
}

extern "C" int f3s_forward_phase(int32_t phase, const int32_t *row_window_offset, const int32_t *sorted_row_windows,
                                 const int32_t *sparse_a_to_x_idx, const uint64_t *tcb_bitmap,
                                 const int32_t *phase_split, int32_t col_split, int32_t num_nodes,
                                 int32_t n_row_windows, int64_t n_tcb, int32_t block_w, int32_t heads,
                                 int32_t head_dim, int64_t ld_q, const void *q, int64_t ld_kv, const void *k,
                                 const void *v, float scale_divisor, float *out, void *workspace,
                                 size_t workspace_bytes, f3s_stream_t stream) {
  F3S_REQUIRE(phase == 1 || phase == 2, F3S_ERR_INVALID_ARG, "phase must be 1 or 2");
  F3S_REQUIRE(head_dim == 64, F3S_ERR_UNSUPPORTED, "two-phase calls need head_dim 64");
  F3S_REQUIRE(n_row_windows >= 0 && n_tcb >= 0 && heads >= 1 && (block_w == 8 || block_w == 16), F3S_ERR_INVALID_ARG,
              "bad size");
  const PhasedLayout L = phased_layout(n_row_windows, n_tcb, block_w, heads, head_dim);
  F3S_REQUIRE(workspace && workspace_bytes >= L.total, F3S_ERR_WORKSPACE, "workspace too small: %zu < %zu",
              workspace_bytes, L.total);
  unsigned char *ws = static_cast<unsigned char *>(workspace);
  FwdExtra ex;
  ex.mode = MODE_PLANNED;
  ex.ld_kv = ld_kv;
  ex.phase = phase;
  ex.col_split = col_split;
  ex.phase_split = phase_split;
  ex.state = reinterpret_cast<float *>(ws + L.off_state);
  return forward_impl(row_window_offset, sorted_row_windows, sparse_a_to_x_idx, tcb_bitmap, num_nodes, n_row_windows,
                      n_tcb, block_w, heads, head_dim, ld_q, q, k, v, scale_divisor, 1, out, 0, nullptr,
                      ws + (phase - 1) * L.sched_bytes, L.sched_bytes, 0, nullptr, nullptr, stream, &ex);
}

// Reads the status word the kernels of the last forward call on `workspace` left behind.
extern "C" int f3s_forward_status(const void *workspace, int32_t *status_host, f3s_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  F3S_REQUIRE(workspace != nullptr, F3S_ERR_INVALID_ARG, "null workspace");
  const int *word = static_cast<const int *>(workspace) + HDR_STATUS;
  if (status_host != nullptr) {  // non-blocking form: the caller synchronises and decodes
    F3S_CUDA_TRY(cudaMemcpyAsync(status_host, word, sizeof(int), cudaMemcpyDeviceToHost, stream));
    return F3S_OK;
  }
  int st = 0;
  F3S_CUDA_TRY(cudaMemcpyAsync(&st, word, sizeof(int), cudaMemcpyDeviceToHost, stream));
  F3S_CUDA_TRY(cudaStreamSynchronize(stream));
  return f3s_status_word_to_code(st);
}

extern "C" int f3s_status_word_to_code(int32_t word) {
  if (word == 0) return F3S_OK;
  if (word == STATUS_LIST_OVERFLOW)
    set_error("device status %d: the schedule's unit list overflowed; some row windows were not processed", word);
  else if (word == STATUS_WAIT_TIMEOUT)
    set_error("device status %d: a bounded wait for an asynchronous copy ran out; some row windows were not stored",
              word);
  else
    set_error("device status %d: unknown", word);
  return F3S_ERR_DEVICE;
}

// ---------------------------------------------------------------------------------------
// Entry point for callers that must not allocate device memory.
// ---------------------------------------------------------------------------------------
// Some hosts of this library cannot call cudaMalloc or any allocator at all once they are
// running: a serving process whose device-memory budget is fixed when it loads its plugins,
// or a runtime that calls into this library from inside its own execution callback, where an
// allocation would synchronise the device or re-enter the host's allocator.  For them the
// schedule and the partial results of split row windows live in this fixed array instead of
// a caller-provided workspace.  Every device that loads the library carries the array until
// the process exits.
static_assert(F3S_STATIC_SCRATCH_BYTES == (32u << 20), "keep the header's documented capacity in sync");
static __device__ __align__(256) unsigned char g_static_scratch[F3S_STATIC_SCRATCH_BYTES];

// Device address of g_static_scratch on the current device.  In host code the array's name
// is only a handle for the runtime, not an address a kernel could use; the address has to be
// asked for, once per device, with that device current.
static int static_scratch_ptr(void **out) {
  static void *cached[64] = {nullptr};
  int dev = 0;
  F3S_CUDA_TRY(cudaGetDevice(&dev));
  F3S_REQUIRE(dev >= 0 && dev < 64, F3S_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  if (cached[dev] == nullptr) {
    void *ptr = nullptr;
    F3S_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_scratch));
    F3S_REQUIRE(ptr != nullptr, F3S_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    cached[dev] = ptr;
  }
  *out = cached[dev];
  return F3S_OK;
}

extern "C" int f3s_forward_static(const int32_t *row_window_offset, const int32_t *sorted_row_windows,
                                  const int32_t *sparse_a_to_x_idx, const uint64_t *tcb_bitmap,
                                  int32_t num_nodes, int32_t n_row_windows, int64_t n_tcb, int32_t block_w,
                                  int32_t heads, int32_t head_dim, int64_t ld, const void *q, const void *k,
                                  const void *v, float scale_divisor, int32_t apply_softmax, float *out,
                                  f3s_stream_t stream) {
  // sizes are checked again by forward_impl; here only what decides whether the problem fits
  F3S_REQUIRE(n_row_windows >= 0 && n_tcb >= 0 && heads >= 1, F3S_ERR_INVALID_ARG, "negative size");
  F3S_REQUIRE(block_w == 8 || block_w == 16, F3S_ERR_UNSUPPORTED, "block_w must be 8 or 16, got %d", block_w);
  F3S_REQUIRE(dim_supported(head_dim), F3S_ERR_UNSUPPORTED,
              "head_dim must be a multiple of 16 between 16 and 128, got %d", head_dim);
  const Geometry gm = geometry(n_row_windows, n_tcb, block_w, heads, head_dim, F3S_STATIC_SCRATCH_BYTES);
  F3S_REQUIRE(gm.total_bytes <= F3S_STATIC_SCRATCH_BYTES, F3S_ERR_WORKSPACE,
              "problem too large for the built-in scratch: %zu bytes needed for %d row windows x %d head(s), "
              "capacity %u bytes; use f3s_forward with a caller-provided workspace",
              gm.total_bytes, n_row_windows, heads, F3S_STATIC_SCRATCH_BYTES);
  void *scratch = nullptr;
  if (int rc = static_scratch_ptr(&scratch)) return rc;
  return forward_impl(row_window_offset, sorted_row_windows, sparse_a_to_x_idx, tcb_bitmap, num_nodes, n_row_windows,
                      n_tcb, block_w, heads, head_dim, ld, q, k, v, scale_divisor, apply_softmax, out, 0, nullptr,
                      scratch, F3S_STATIC_SCRATCH_BYTES, F3S_STATIC_SCRATCH_BYTES, nullptr, nullptr, stream);
}

// f3s_forward_status for the built-in scratch of f3s_forward_static (allocates nothing either).
extern "C" int f3s_forward_static_status(int32_t *status_host, f3s_stream_t stream) {
  void *scratch = nullptr;
  if (int rc = static_scratch_ptr(&scratch)) return rc;
  return f3s_forward_status(scratch, status_host, stream);
}
