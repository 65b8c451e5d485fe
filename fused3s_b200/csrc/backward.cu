// Backward of the fused sparse attention over TC blocks for sm_100a: dQ, dK, dV from dO.
//
// The reference is inference-only (its extension exports forward ops only, src/F3S.cpp:298-305);
// this file is what a training caller of f3s_1tb1rw_scheduled_permuteV_scaleQK needs.  With
//   p_ij = exp2(s_ij * scale - lse_i)      (s = q_i . k_j, lse from the forward pass)
//   delta_i = dO_i . O_i
//   dS_ij = p_ij * (dO_i . v_j - delta_i)
// the gradients are  dQ_i = (1/divisor) sum_j dS_ij k_j,  dK_j = (1/divisor) sum_i dS_ij q_i,
// dV_j = sum_i p_ij dO_i.  S and P are recomputed tile by tile, never stored.
//
// Two launches of one kernel template, both with the forward kernel's work decomposition (one
// warp = one unit = (head, 16-row window, range of 8-column tiles); heavy windows cut into chunks
// whose partial sums are merged by the last chunk to arrive, in chunk order; no atomics on the
// gradients, results are deterministic):
//   * dQ on the TC blocks of the graph itself: window rows i, gathered rows j;
//     window operands (Q, dO), gathered operands (K, V):  dQ += dS K_g.
//   * dK, dV on the TC blocks of the TRANSPOSED graph: window rows j, gathered rows i;
//     window operands (K, V), gathered operands (Q, dO) plus (lse_i, delta_i) per gathered row:
//     S^T = K Q_g^T, dP^T = V dO_g^T, dV += P^T dO_g, dK += dS^T Q_g.
// For head dimension 128 the dK/dV launch runs twice, each time accumulating one half of the
// feature columns (two 16 x 128 fp32 accumulators do not fit in a warp's registers).
#include <limits.h>
#include <math.h>

#include "attn_common.cuh"

namespace f3s {

struct BwdParams {
  // TC-block arrays and schedule; same meaning as in FwdParams (UnitSource reads these names)
  const int *rwo;
  const int *sorted;
  const int *atox;
  const unsigned long long *bitmap;
  int n_nodes, n_rw, heads, d_real, t8_per_tcb, direct, ch8;
  int *hdr;
  const UnitDesc *units;
  int *arrive;
  float *partial;
  int max_slots;
  // operands: a* are read by window row, g* by gathered row
  const __half *a1, *a2, *g1, *g2;
  long long ld_a1, ld_a2, ld_g1, ld_g2;
  const float2 *stats;  // [n_nodes][heads] {lse, delta}
  float scale;          // log2(e) / divisor (signed)
  float out_scale;      // 1 / divisor, applied to the first accumulator
  void *out1, *out2;    // [n_nodes][heads][d_real]; out2 only in the dK/dV launch
  int out_half;         // 1: gradients are stored as fp16
  int fpart;            // which part of the feature columns this launch accumulates (FSPLIT > 1)
  int phase;            // always 0 here: the backward works on whole windows (the shared iterator reads it)
  const int *phase_split;
};

template <int D, int NT8, int STAGES, int WARPS>
struct BwdCfg {
  static constexpr int ROWS = NT8 * 8;
  static constexpr int TILE_BYTES = ROWS * D * 2;
  static constexpr int BM_BYTES = 128;
  static constexpr int ST_BYTES = ROWS * 8;  // {lse, delta} of every gathered row
  static constexpr int STAGE_BYTES = 2 * TILE_BYTES + BM_BYTES + ST_BYTES;
  static constexpr int A_BYTES = 16 * D * 2;
  static constexpr int WARP_BYTES = 2 * A_BYTES + STAGES * STAGE_BYTES;
  static constexpr int SMEM_BYTES = WARPS * WARP_BYTES;
  static_assert(NT8 * 16 <= BM_BYTES, "bitmap slot too small");
  static_assert(NT8 % 2 == 0 && ROWS <= 32, "a step is 16 or 32 gathered rows");
  static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB of shared memory a CTA can have");
};

// A fragments of a 16 x D operand tile in (swizzled) shared memory.
template <int D>
__device__ __forceinline__ void load_a_frags(uint32_t a_s, uint32_t (&af)[D / 16][4], int lane) {
  using T = Tile<D>;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const int m = lane >> 3;
    ldmatrix_x4(af[ks], T::addr(a_s, (m & 1) * 8 + (lane & 7), ks * 2 + (m >> 1)));
  }
}

// acc(16 x 8*NFA) += X(16 x 8*NT8, fp32 -> fp16) * G[:, f0*8 ...] for the gathered tile at tile_s.
template <int D, int NT8, int NFA>
__device__ __forceinline__ void accumulate_tiles(const float (&x)[NT8][4], uint32_t tile_s, int f0,
                                                 float (&acc)[NFA][4], int lane) {
  using T = Tile<D>;
#pragma unroll
  for (int j = 0; j < NT8 / 2; ++j) {
    uint32_t xa[4];
    xa[0] = pack_half2(x[2 * j][0], x[2 * j][1]);
    xa[1] = pack_half2(x[2 * j][2], x[2 * j][3]);
    xa[2] = pack_half2(x[2 * j + 1][0], x[2 * j + 1][1]);
    xa[3] = pack_half2(x[2 * j + 1][2], x[2 * j + 1][3]);
#pragma unroll
    for (int fp = 0; fp < NFA / 2; ++fp) {
      uint32_t b[4];
      const int m = lane >> 3;
      ldmatrix_x4_trans(b, T::addr(tile_s, j * 16 + (m & 1) * 8 + (lane & 7), f0 + 2 * fp + (m >> 1)));
      mma_16816(acc[2 * fp], xa, b[0], b[1]);
      mma_16816(acc[2 * fp + 1], xa, b[2], b[3]);
    }
  }
}

// Store feature tile f (8 columns) of rows g and g+8 of a window of a gradient tensor.
__device__ __forceinline__ void store_grad_tile(void *out, int out_half, const BwdParams &p, int head, int window,
                                                int f, float v0, float v1, float v2, float v3, int lane) {
  if (f * 8 >= p.d_real) return;  // feature tiles that only exist as zero padding
  const int g = lane >> 2, qd = lane & 3;
  const int r0 = window * 16 + g, r1 = r0 + 8;
  const size_t ldo = (size_t)p.heads * p.d_real;
  const size_t off0 = (size_t)r0 * ldo + (size_t)head * p.d_real + 2 * qd + f * 8;
  const size_t off1 = (size_t)r1 * ldo + (size_t)head * p.d_real + 2 * qd + f * 8;
  if (!out_half) {
    float *o = static_cast<float *>(out);
    if (r0 < p.n_nodes) *reinterpret_cast<float2 *>(o + off0) = make_float2(v0, v1);
    if (r1 < p.n_nodes) *reinterpret_cast<float2 *>(o + off1) = make_float2(v2, v3);
  } else {
    __half *o = static_cast<__half *>(out);
    if (r0 < p.n_nodes) *reinterpret_cast<__half2 *>(o + off0) = __floats2half2_rn(v0, v1);
    if (r1 < p.n_nodes) *reinterpret_cast<__half2 *>(o + off1) = __floats2half2_rn(v2, v3);
  }
}

// DKV = false: dQ launch.  DKV = true: dK/dV launch on the transposed graph.
// FSPLIT: the launch accumulates D / FSPLIT feature columns (part p.fpart).
template <int D, int NT8, int STAGES, int WARPS, bool DKV, int FSPLIT>
__global__ void __launch_bounds__(WARPS * 32, 1) bwd_kernel(const BwdParams p) {
  using C = BwdCfg<D, NT8, STAGES, WARPS>;
  using T = Tile<D>;
  constexpr int KS = D / 16;
  constexpr int NFA = D / 8 / FSPLIT;  // feature tiles per accumulator
  constexpr int NACC = DKV ? 2 : 1;
  constexpr int ROWS = C::ROWS;
  constexpr int CPL = ROWS * T::CHUNKS / 32;  // 16-byte copies per lane per operand tile
  constexpr int PARTIAL_FLOATS = NACC * NFA * 4 * 32;
  static_assert(NFA % 2 == 0, "accumulators are filled two feature tiles at a time");
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, qd = lane & 3;
  unsigned char *wsm = smem_raw + warp * C::WARP_BYTES;
  const uint32_t a1_s = smem_u32(wsm), a2_s = a1_s + C::A_BYTES, stage0_s = a2_s + C::A_BYTES;
  const unsigned char *stage0_g = wsm + 2 * C::A_BYTES;
  const int bm_half = (g < 4) ? 1 : 0;  // this lane's rows sit in one 32-bit half of each 64-bit bitmap word
  const int bm_shift = 8 * (g & 3) + 2 * qd;
  const int f0 = p.fpart * NFA;

  UnitSource src;
  src.init(p, blockIdx.x * WARPS + warp, gridDim.x * WARPS);
  Unit u;
  while (src.next(p, lane, u)) {
    float acc1[NFA][4], acc2[DKV ? NFA : 1][4];
#pragma unroll
    for (int f = 0; f < NFA; ++f) acc1[f][0] = acc1[f][1] = acc1[f][2] = acc1[f][3] = 0.f;
#pragma unroll
    for (int f = 0; f < (DKV ? NFA : 1); ++f) acc2[f][0] = acc2[f][1] = acc2[f][2] = acc2[f][3] = 0.f;
    const int t8b = u.t8b, t8e = u.t8e;
    const int nsteps = (t8e - t8b + NT8 - 1) / NT8;
    if (nsteps > 0) {
      const size_t hoff = (size_t)u.head * p.d_real;
      {  // window operands -> shared (join the first copy group); rows past the last node read as 0
        const int row0 = u.window * 16;
#pragma unroll
        for (int c = lane; c < 16 * T::CHUNKS; c += 32) {
          const int r = c / T::CHUNKS, ch = c % T::CHUNKS;
          const int gr = row0 + r;
          const bool ok = gr < p.n_nodes && ch * 8 < p.d_real;
          const size_t row = ok ? gr : 0, col = ok ? ch * 8 : 0;
          cp_async16(T::addr(a1_s, r, ch), p.a1 + row * p.ld_a1 + hoff + col, ok ? 16 : 0);
          cp_async16(T::addr(a2_s, r, ch), p.a2 + row * p.ld_a2 + hoff + col, ok ? 16 : 0);
        }
      }
      float lse_r[2] = {0.f, 0.f}, del_r[2] = {0.f, 0.f};  // dQ launch: statistics of rows g and g+8
      if (!DKV) {
        const int r0 = u.window * 16 + g, r1 = r0 + 8;
        if (r0 < p.n_nodes) {
          const float2 st = __ldg(p.stats + (size_t)r0 * p.heads + u.head);
          lse_r[0] = st.x; del_r[0] = st.y;
        }
        if (r1 < p.n_nodes) {
          const float2 st = __ldg(p.stats + (size_t)r1 * p.heads + u.head);
          lse_r[1] = st.x; del_r[1] = st.y;
        }
      }
      int idx_next = 0;  // id of gathered row `lane` of the next step to be issued
      {
        const int lim = (t8e - t8b) * 8;
        if (lane < ROWS && lane < lim) idx_next = __ldg(p.atox + (size_t)t8b * 8 + lane);
      }
      auto issue = [&](int step) {
        const int t8 = t8b + step * NT8;
        const int st = step % STAGES;
        const uint32_t g1s = stage0_s + st * C::STAGE_BYTES;
        const uint32_t g2s = g1s + C::TILE_BYTES;
        const uint32_t bs = g2s + C::TILE_BYTES;
        const uint32_t ss = bs + C::BM_BYTES;
        const int lim = (t8e - t8) * 8;  // rows at or beyond lim lie outside the unit
        const int idx_cur = idx_next;
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
          const size_t col = real ? ch * 8 : 0;
          cp_async16(T::addr(g1s, r, ch), p.g1 + (size_t)idx * p.ld_g1 + hoff + col, nbytes);
          cp_async16(T::addr(g2s, r, ch), p.g2 + (size_t)idx * p.ld_g2 + hoff + col, nbytes);
        }
        if (lane < NT8) {
          const bool ok = (t8 + lane) < t8e;
          cp_async16(bs + lane * 16, p.bitmap + (ok ? (size_t)(t8 + lane) * 2 : 0), ok ? 16 : 0);
        }
        if (DKV && lane < ROWS)
          cp_async8(ss + lane * 8, p.stats + (size_t)idx_cur * p.heads + u.head, lane < lim ? 8 : 0);
      };
#pragma unroll
      for (int s = 0; s < STAGES - 1; ++s) {
        if (s < nsteps) issue(s);
        cp_async_commit();
      }
      uint32_t a1f[KS][4], a2f[KS][4];
      for (int step = 0; step < nsteps; ++step) {
        if (step + STAGES - 1 < nsteps) issue(step + STAGES - 1);
        cp_async_commit();
        cp_async_wait<STAGES - 1>();
        __syncwarp();
        if (step == 0) {
          load_a_frags<D>(a1_s, a1f, lane);
          load_a_frags<D>(a2_s, a2f, lane);
        }
        const int st = step % STAGES;
        const uint32_t g1s = stage0_s + st * C::STAGE_BYTES;
        const uint32_t g2s = g1s + C::TILE_BYTES;
        const unsigned char *stage_g = stage0_g + st * C::STAGE_BYTES;
        const uint32_t *bm32 = reinterpret_cast<const uint32_t *>(stage_g + 2 * C::TILE_BYTES) + bm_half;
        const float4 *st4 = reinterpret_cast<const float4 *>(stage_g + 2 * C::TILE_BYTES + C::BM_BYTES);

        float s[NT8][4], dp[NT8][4];
        score_tiles<D, NT8>(g1s, a1f, s, lane);   // S (or S^T)
        score_tiles<D, NT8>(g2s, a2f, dp, lane);  // dP (or dP^T)
#pragma unroll
        for (int nt = 0; nt < NT8; ++nt) {
          // tiles past the end of the unit have zero-filled bitmap words: everything masked
          const uint32_t h0 = bm32[nt * 4] << bm_shift, h1 = bm32[nt * 4 + 2] << bm_shift;
          const bool v0 = (int)h0 < 0, v1 = (int)(h0 << 1) < 0, v2 = (int)h1 < 0, v3 = (int)(h1 << 1) < 0;
          float l0, l1, l2, l3, d0, d1, d2, d3;
          if (DKV) {  // statistics belong to the gathered rows = this lane's two columns
            const float4 sv = st4[nt * 4 + qd];
            l0 = l2 = sv.x; d0 = d2 = sv.y;
            l1 = l3 = sv.z; d1 = d3 = sv.w;
          } else {
            l0 = l1 = lse_r[0]; d0 = d1 = del_r[0];
            l2 = l3 = lse_r[1]; d2 = d3 = del_r[1];
          }
          const float p0 = v0 ? fast_exp2(fmaf(s[nt][0], p.scale, -l0)) : 0.f;
          const float p1 = v1 ? fast_exp2(fmaf(s[nt][1], p.scale, -l1)) : 0.f;
          const float p2 = v2 ? fast_exp2(fmaf(s[nt][2], p.scale, -l2)) : 0.f;
          const float p3 = v3 ? fast_exp2(fmaf(s[nt][3], p.scale, -l3)) : 0.f;
          s[nt][0] = p0; s[nt][1] = p1; s[nt][2] = p2; s[nt][3] = p3;
          dp[nt][0] = p0 * (dp[nt][0] - d0);
          dp[nt][1] = p1 * (dp[nt][1] - d1);
          dp[nt][2] = p2 * (dp[nt][2] - d2);
          dp[nt][3] = p3 * (dp[nt][3] - d3);
        }
        accumulate_tiles<D, NT8, NFA>(dp, g1s, f0, acc1, lane);           // dQ += dS K   |  dK += dS^T Q
        if constexpr (DKV) accumulate_tiles<D, NT8, NFA>(s, g2s, f0, acc2, lane);   //                 dV += P^T dO
        __syncwarp();  // every lane is done with this stage before it is refilled
      }
      cp_async_wait<0>();
    }

    // ---- end of the unit: publish / merge the partial sums of a split window, store ----
    bool write_out = true;
    if (u.slot_base >= 0) {
      float *mine = p.partial + ((size_t)u.head * p.max_slots + u.slot_base + u.chunk) * PARTIAL_FLOATS;
#pragma unroll
      for (int f = 0; f < NFA; ++f)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          __stcg(mine + (f * 4 + e) * 32 + lane, acc1[f][e]);
          if constexpr (DKV) __stcg(mine + ((NFA + f) * 4 + e) * 32 + lane, acc2[f][e]);
        }
      __threadfence();
      __syncwarp();
      int prev = 0;
      if (lane == 0) prev = atomicAdd(&p.arrive[(size_t)u.head * p.max_slots + u.slot_base], 1);
      prev = __shfl_sync(FULL, prev, 0);
      write_out = (prev == u.n_chunks - 1);
      if (write_out) {  // last chunk to arrive: sum all chunks in chunk order
        __threadfence();
        const float *base = p.partial + ((size_t)u.head * p.max_slots + u.slot_base) * PARTIAL_FLOATS;
#pragma unroll
        for (int f = 0; f < NFA; ++f) acc1[f][0] = acc1[f][1] = acc1[f][2] = acc1[f][3] = 0.f;
#pragma unroll
        for (int f = 0; f < (DKV ? NFA : 1); ++f) acc2[f][0] = acc2[f][1] = acc2[f][2] = acc2[f][3] = 0.f;
        for (int c = 0; c < u.n_chunks; ++c) {
          const float *pc = base + (size_t)c * PARTIAL_FLOATS;
#pragma unroll
          for (int f = 0; f < NFA; ++f)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              acc1[f][e] += __ldcg(pc + (f * 4 + e) * 32 + lane);
              if constexpr (DKV) acc2[f][e] += __ldcg(pc + ((NFA + f) * 4 + e) * 32 + lane);
            }
        }
      }
    }
    if (write_out) {
#pragma unroll
      for (int f = 0; f < NFA; ++f) {
        store_grad_tile(p.out1, p.out_half, p, u.head, u.window, f0 + f, acc1[f][0] * p.out_scale,
                        acc1[f][1] * p.out_scale, acc1[f][2] * p.out_scale, acc1[f][3] * p.out_scale, lane);
        if constexpr (DKV)
          store_grad_tile(p.out2, p.out_half, p, u.head, u.window, f0 + f, acc2[f][0], acc2[f][1], acc2[f][2],
                          acc2[f][3], lane);
      }
    }
  }
}

// One warp per (row, head): delta = dO . O, fp16 copy of dO, {lse, delta} pairs.
__global__ void __launch_bounds__(256) bwd_prepare_kernel(const float *__restrict__ out,
                                                          const float *__restrict__ d_out,
                                                          const float *__restrict__ lse, __half *__restrict__ do_h,
                                                          float2 *__restrict__ stats, long long pairs, int d) {
  const int lane = threadIdx.x & 31;
  const long long x = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (x >= pairs) return;
  const float *o = out + x * d, *g = d_out + x * d;
  __half *gh = do_h + x * d;
  float acc = 0.f;
  for (int e = lane * 2; e < d; e += 64) {
    const float2 ov = *reinterpret_cast<const float2 *>(o + e);
    const float2 gv = *reinterpret_cast<const float2 *>(g + e);
    acc = fmaf(ov.x, gv.x, fmaf(ov.y, gv.y, acc));
    *reinterpret_cast<__half2 *>(gh + e) = __floats2half2_rn(gv.x, gv.y);
  }
#pragma unroll
  for (int o2 = 16; o2 > 0; o2 >>= 1) acc += __shfl_xor_sync(FULL, acc, o2);
  if (lane == 0) stats[x] = make_float2(lse[x], acc);
}

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
struct BwdKernelCfg {
  int d_pad, nt8, stages, warps_dq, warps_dkv, fsplit;
};

static bool bwd_dim_supported(int d) { return d >= 16 && d <= 128 && d % 16 == 0; }

static BwdKernelCfg bwd_cfg(int d) {
  if (d <= 32) return {32, 4, 3, 8, 8, 1};
  if (d <= 64) return {64, 4, 2, 10, 8, 1};
  return {128, 2, 2, 8, 8, 2};
}

// Scratch of one launch: header, arrival counters, unit list, partial sums of split windows.
struct BwdSched {
  int direct, ch8, max_slots;
  size_t off_hdr, off_arrive, off_units, off_partial, zero_bytes, bytes;
};

constexpr int BWD_UNITS_PER_WARP = 6;
constexpr int BWD_MIN_CH8 = 64;
constexpr int BWD_DIRECT_TILES_PER_WARP = 32;

static BwdSched bwd_sched(long long n_tcb, int block_w, int heads, int warps, int nt8, size_t partial_floats) {
  BwdSched sc;
  const long long total_t8 = n_tcb * (block_w / 8);
  const long long total_warps = (long long)sm_count() * warps;
  sc.direct = (total_t8 * heads <= total_warps * BWD_DIRECT_TILES_PER_WARP) ? 1 : 0;
  long long ch = (total_t8 * heads) / (total_warps * BWD_UNITS_PER_WARP);
  ch = (ch + nt8 - 1) / nt8 * nt8;
  if (ch < BWD_MIN_CH8) ch = BWD_MIN_CH8;
  if (ch > (1 << 28)) ch = 1 << 28;
  sc.ch8 = (int)ch;
  sc.max_slots = sc.direct ? 0 : (int)(2 * total_t8 / sc.ch8 + 2);
  size_t off = 0;
  sc.off_hdr = off; off += HDR_INTS * sizeof(int);
  sc.off_arrive = off; off += (size_t)sc.max_slots * heads * sizeof(int);
  sc.zero_bytes = off;
  off = align_up(off, 256);
  sc.off_units = off; off = align_up(off + (size_t)sc.max_slots * sizeof(UnitDesc), 256);
  sc.off_partial = off; off = align_up(off + (size_t)sc.max_slots * heads * partial_floats * sizeof(float), 256);
  sc.bytes = off;
  return sc;
}

struct BwdLayout {
  BwdKernelCfg kc;
  BwdSched dq, dkv;
  size_t off_doh, off_stats, off_dq, off_dkv, bytes;
};

static BwdLayout bwd_layout(int num_nodes, long long n_tcb, long long n_tcb_t, int block_w, int heads, int d) {
  BwdLayout L;
  L.kc = bwd_cfg(d);
  const int nfa_dq = L.kc.d_pad / 8, nfa_dkv = L.kc.d_pad / 8 / L.kc.fsplit;
  L.dq = bwd_sched(n_tcb, block_w, heads, L.kc.warps_dq, L.kc.nt8, (size_t)nfa_dq * 4 * 32);
  L.dkv = bwd_sched(n_tcb_t, block_w, heads, L.kc.warps_dkv, L.kc.nt8, (size_t)2 * nfa_dkv * 4 * 32);
  size_t off = 0;
  L.off_doh = off; off = align_up(off + (size_t)num_nodes * heads * d * sizeof(__half), 256);
  L.off_stats = off; off = align_up(off + (size_t)num_nodes * heads * sizeof(float2), 256);
  L.off_dq = off; off += L.dq.bytes;
  L.off_dkv = off; off += L.dkv.bytes;
  L.bytes = off;
  return L;
}

template <int D, int NT8, int STAGES, int WARPS, bool DKV, int FSPLIT>
static int launch_bwd(const BwdParams &p, int grid, cudaStream_t stream) {
  using C = BwdCfg<D, NT8, STAGES, WARPS>;
  auto kern = bwd_kernel<D, NT8, STAGES, WARPS, DKV, FSPLIT>;
  F3S_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
  kern<<<grid, WARPS * 32, C::SMEM_BYTES, stream>>>(p);
  F3S_CHECK_LAUNCH();
  return F3S_OK;
}

// Schedule (unless direct) + the launch(es) of one of the two gradient kernels.
static int run_bwd(BwdParams p, const BwdSched &sc, unsigned char *ws, const BwdKernelCfg &kc, bool dkv,
                   cudaStream_t stream) {
  p.direct = sc.direct;
  p.ch8 = sc.direct ? INT_MAX : sc.ch8;
  p.hdr = reinterpret_cast<int *>(ws + sc.off_hdr);
  p.units = reinterpret_cast<const UnitDesc *>(ws + sc.off_units);
  p.arrive = reinterpret_cast<int *>(ws + sc.off_arrive);
  p.partial = reinterpret_cast<float *>(ws + sc.off_partial);
  p.max_slots = sc.max_slots;
  p.phase = 0;
  p.phase_split = nullptr;
  const int warps = dkv ? kc.warps_dkv : kc.warps_dq;
  const int parts = dkv ? kc.fsplit : 1;
  for (int part = 0; part < parts; ++part) {
    p.fpart = part;
    int grid = sm_count();
    if (sc.direct) {
      const long long units = (long long)p.n_rw * p.heads;
      const long long need = (units + warps - 1) / warps;
      if (need < grid) grid = (int)(need > 0 ? need : 1);
    } else {
      F3S_CUDA_TRY(cudaMemsetAsync(ws + sc.off_hdr, 0, sc.zero_bytes, stream));
      plan_kernel<<<(p.n_rw + PLAN_THREADS - 1) / PLAN_THREADS, PLAN_THREADS, 0, stream>>>(
          PlanArgs{p.rwo, 0, nullptr}, p.sorted, p.n_rw, p.t8_per_tcb, sc.ch8, kc.nt8, p.hdr, reinterpret_cast<UnitDesc *>(ws + sc.off_units),
          sc.max_slots);
      F3S_CHECK_LAUNCH();
    }
    int rc = F3S_ERR_UNSUPPORTED;
    if (kc.d_pad == 32) rc = dkv ? launch_bwd<32, 4, 3, 8, true, 1>(p, grid, stream) : launch_bwd<32, 4, 3, 8, false, 1>(p, grid, stream);
    if (kc.d_pad == 64) rc = dkv ? launch_bwd<64, 4, 2, 8, true, 1>(p, grid, stream) : launch_bwd<64, 4, 2, 10, false, 1>(p, grid, stream);
    if (kc.d_pad == 128) rc = dkv ? launch_bwd<128, 2, 2, 8, true, 2>(p, grid, stream) : launch_bwd<128, 2, 2, 8, false, 1>(p, grid, stream);
    if (rc != F3S_OK) return rc;
  }
  return F3S_OK;
}

}  // namespace f3s

using namespace f3s;

extern "C" size_t f3s_backward_workspace_bytes(int32_t num_nodes, int64_t n_tcb, int64_t n_tcb_t, int32_t block_w,
                                               int32_t heads, int32_t head_dim) {
  if (num_nodes < 0 || n_tcb < 0 || n_tcb_t < 0 || heads < 1 || (block_w != 8 && block_w != 16)) return 0;
  if (!bwd_dim_supported(head_dim)) return 0;
  return bwd_layout(num_nodes, n_tcb, n_tcb_t, block_w, heads, head_dim).bytes;
}

extern "C" int f3s_backward(const int32_t *row_window_offset, const int32_t *sorted_row_windows,
                            const int32_t *sparse_a_to_x_idx, const uint64_t *tcb_bitmap, int64_t n_tcb,
                            const int32_t *row_window_offset_t, const int32_t *sorted_row_windows_t,
                            const int32_t *sparse_a_to_x_idx_t, const uint64_t *tcb_bitmap_t, int64_t n_tcb_t,
                            int32_t num_nodes, int32_t n_row_windows, int32_t block_w, int32_t heads,
                            int32_t head_dim, int64_t ld, const void *q, const void *k, const void *v,
                            float scale_divisor, const float *out, const float *lse, const float *d_out, void *dq,
                            void *dk, void *dv, int32_t grads_are_half, void *workspace, size_t workspace_bytes,
                            f3s_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  F3S_REQUIRE(num_nodes >= 0 && n_row_windows >= 0 && n_tcb >= 0 && n_tcb_t >= 0, F3S_ERR_INVALID_ARG,
              "negative size");
  F3S_REQUIRE(n_row_windows == (num_nodes + 15) / 16, F3S_ERR_INVALID_ARG,
              "n_row_windows (%d) must be ceil(num_nodes/16) (%d)", n_row_windows, (num_nodes + 15) / 16);
  F3S_REQUIRE(block_w == 8 || block_w == 16, F3S_ERR_UNSUPPORTED, "block_w must be 8 or 16, got %d", block_w);
  F3S_REQUIRE(bwd_dim_supported(head_dim), F3S_ERR_UNSUPPORTED,
              "head_dim must be a multiple of 16 between 16 and 128, got %d", head_dim);
  F3S_REQUIRE(heads >= 1, F3S_ERR_INVALID_ARG, "heads must be >= 1");
  F3S_REQUIRE(ld >= (int64_t)heads * head_dim && ld % 8 == 0, F3S_ERR_INVALID_ARG,
              "ld (%lld) must be >= heads*head_dim and a multiple of 8", (long long)ld);
  F3S_REQUIRE(scale_divisor != 0.f && isfinite(scale_divisor), F3S_ERR_INVALID_ARG,
              "scale_divisor must be finite and non-zero");
  F3S_REQUIRE(n_tcb * block_w < (1ll << 31) && n_tcb_t * block_w < (1ll << 31), F3S_ERR_UNSUPPORTED,
              "n_tcb*block_w exceeds int32");
  if (num_nodes == 0) return F3S_OK;
  F3S_REQUIRE(row_window_offset && row_window_offset_t && q && k && v && out && lse && d_out && dq && dk && dv,
              F3S_ERR_INVALID_ARG, "null pointer argument");
  F3S_REQUIRE(n_tcb == 0 || (sparse_a_to_x_idx && tcb_bitmap), F3S_ERR_INVALID_ARG, "null TCB array");
  F3S_REQUIRE(n_tcb_t == 0 || (sparse_a_to_x_idx_t && tcb_bitmap_t), F3S_ERR_INVALID_ARG,
              "null TCB array of the transposed graph");
  auto misaligned = [](const void *ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) != 0; };
  F3S_REQUIRE(!misaligned(q) && !misaligned(k) && !misaligned(v) && !misaligned(out) && !misaligned(d_out) &&
                  !misaligned(dq) && !misaligned(dk) && !misaligned(dv) && !misaligned(tcb_bitmap) &&
                  !misaligned(tcb_bitmap_t),
              F3S_ERR_INVALID_ARG, "tensors and bitmaps must be 16-byte aligned");
  const BwdLayout L = bwd_layout(num_nodes, n_tcb, n_tcb_t, block_w, heads, head_dim);
  F3S_REQUIRE(workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 255) == 0, F3S_ERR_WORKSPACE,
              "workspace must be non-null and 256-byte aligned");
  F3S_REQUIRE(workspace_bytes >= L.bytes, F3S_ERR_WORKSPACE, "workspace too small: %zu < %zu", workspace_bytes,
              L.bytes);

  unsigned char *ws = static_cast<unsigned char *>(workspace);
  __half *do_h = reinterpret_cast<__half *>(ws + L.off_doh);
  float2 *stats = reinterpret_cast<float2 *>(ws + L.off_stats);
  const long long pairs = (long long)num_nodes * heads;
  bwd_prepare_kernel<<<(unsigned)((pairs + 7) / 8), 256, 0, stream>>>(out, d_out, lse, do_h, stats, pairs, head_dim);
  F3S_CHECK_LAUNCH();

  BwdParams p;
  p.n_nodes = num_nodes;
  p.n_rw = n_row_windows;
  p.heads = heads;
  p.d_real = head_dim;
  p.t8_per_tcb = block_w / 8;
  p.stats = stats;
  p.scale = 1.4426950408889634f / scale_divisor;
  p.out_scale = 1.f / scale_divisor;
  p.out_half = grads_are_half ? 1 : 0;
  p.fpart = 0;
  const long long ld_do = (long long)heads * head_dim;

  // dQ: TC blocks of the graph; window operands (Q, dO), gathered (K, V)
  p.rwo = row_window_offset; p.sorted = sorted_row_windows; p.atox = sparse_a_to_x_idx;
  p.bitmap = reinterpret_cast<const unsigned long long *>(tcb_bitmap);
  p.a1 = static_cast<const __half *>(q); p.ld_a1 = ld;
  p.a2 = do_h; p.ld_a2 = ld_do;
  p.g1 = static_cast<const __half *>(k); p.ld_g1 = ld;
  p.g2 = static_cast<const __half *>(v); p.ld_g2 = ld;
  p.out1 = dq; p.out2 = nullptr;
  if (int rc = run_bwd(p, L.dq, ws + L.off_dq, L.kc, false, stream)) return rc;

  // dK, dV: TC blocks of the transposed graph; window operands (K, V), gathered (Q, dO)
  p.rwo = row_window_offset_t; p.sorted = sorted_row_windows_t; p.atox = sparse_a_to_x_idx_t;
  p.bitmap = reinterpret_cast<const unsigned long long *>(tcb_bitmap_t);
  p.a1 = static_cast<const __half *>(k); p.ld_a1 = ld;
  p.a2 = static_cast<const __half *>(v); p.ld_a2 = ld;
  p.g1 = static_cast<const __half *>(q); p.ld_g1 = ld;
  p.g2 = do_h; p.ld_g2 = ld_do;
  p.out1 = dk; p.out2 = dv;
  return run_bwd(p, L.dkv, ws + L.off_dkv, L.kc, true, stream);
}

// ---------------------------------------------------------------------------------------
// The three stages of f3s_backward as separate entry points, for row-sharded training: a rank
// owns a block of rows (queries, and the same block of keys / values); gathered operands then
// have more rows than the rank's windows and sit in whatever layout the plan's column ids
// index (the caller all-gathers them).
// ---------------------------------------------------------------------------------------
static int check_stage_args(int32_t num_rows, int32_t n_row_windows, int64_t n_tcb, int32_t block_w, int32_t heads,
                            int32_t head_dim, float scale_divisor) {
  F3S_REQUIRE(num_rows >= 0 && n_row_windows >= 0 && n_tcb >= 0, F3S_ERR_INVALID_ARG, "negative size");
  F3S_REQUIRE(n_row_windows == (num_rows + 15) / 16, F3S_ERR_INVALID_ARG,
              "n_row_windows (%d) must be ceil(num_rows/16) (%d)", n_row_windows, (num_rows + 15) / 16);
  F3S_REQUIRE(block_w == 8 || block_w == 16, F3S_ERR_UNSUPPORTED, "block_w must be 8 or 16, got %d", block_w);
  F3S_REQUIRE(bwd_dim_supported(head_dim), F3S_ERR_UNSUPPORTED,
              "head_dim must be a multiple of 16 between 16 and 128, got %d", head_dim);
  F3S_REQUIRE(heads >= 1, F3S_ERR_INVALID_ARG, "heads must be >= 1");
  F3S_REQUIRE(scale_divisor != 0.f && isfinite(scale_divisor), F3S_ERR_INVALID_ARG,
              "scale_divisor must be finite and non-zero");
  F3S_REQUIRE(n_tcb * block_w < (1ll << 31), F3S_ERR_UNSUPPORTED, "n_tcb*block_w exceeds int32");
  return F3S_OK;
}

static bool misaligned16(const void *ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) != 0; }

extern "C" int f3s_backward_prepare(const float *out, const float *d_out, const float *lse, int32_t num_rows,
                                    int32_t heads, int32_t head_dim, void *d_out_f16, float *stats,
                                    f3s_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  F3S_REQUIRE(num_rows >= 0 && heads >= 1, F3S_ERR_INVALID_ARG, "negative size");
  F3S_REQUIRE(bwd_dim_supported(head_dim), F3S_ERR_UNSUPPORTED,
              "head_dim must be a multiple of 16 between 16 and 128, got %d", head_dim);
  if (num_rows == 0) return F3S_OK;
  F3S_REQUIRE(out && d_out && lse && d_out_f16 && stats, F3S_ERR_INVALID_ARG, "null pointer argument");
  F3S_REQUIRE(!misaligned16(out) && !misaligned16(d_out) && !misaligned16(d_out_f16) && !misaligned16(stats),
              F3S_ERR_INVALID_ARG, "tensors must be 16-byte aligned");
  const long long pairs = (long long)num_rows * heads;
  bwd_prepare_kernel<<<(unsigned)((pairs + 7) / 8), 256, 0, stream>>>(out, d_out, lse, static_cast<__half *>(d_out_f16),
                                                                      reinterpret_cast<float2 *>(stats), pairs, head_dim);
  F3S_CHECK_LAUNCH();
  return F3S_OK;
}

extern "C" size_t f3s_backward_stage_workspace_bytes(int64_t n_tcb, int32_t block_w, int32_t heads, int32_t head_dim,
                                                     int32_t dkv) {
  if (n_tcb < 0 || heads < 1 || (block_w != 8 && block_w != 16) || !bwd_dim_supported(head_dim)) return 0;
  const BwdKernelCfg kc = bwd_cfg(head_dim);
  const int nfa = kc.d_pad / 8 / (dkv ? kc.fsplit : 1);
  return bwd_sched(n_tcb, block_w, heads, dkv ? kc.warps_dkv : kc.warps_dq, kc.nt8,
                   (size_t)(dkv ? 2 : 1) * nfa * 4 * 32)
      .bytes;
}

// dQ of a block of rows.  q: the block's rows (row stride ld_q); k, v: gathered operands indexed by the
// plan's column ids (row stride ld_kv); d_out_f16 / stats: f3s_backward_prepare's outputs for the block.
extern "C" int f3s_backward_dq(const int32_t *row_window_offset, const int32_t *sorted_row_windows,
                               const int32_t *sparse_a_to_x_idx, const uint64_t *tcb_bitmap, int64_t n_tcb,
                               int32_t num_rows, int32_t n_row_windows, int32_t block_w, int32_t heads,
                               int32_t head_dim, int64_t ld_q, const void *q, int64_t ld_kv, const void *k,
                               const void *v, float scale_divisor, const void *d_out_f16, const float *stats,
                               void *dq, int32_t grads_are_half, void *workspace, size_t workspace_bytes,
                               f3s_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (int rc = check_stage_args(num_rows, n_row_windows, n_tcb, block_w, heads, head_dim, scale_divisor)) return rc;
  const int64_t hd = (int64_t)heads * head_dim;
  F3S_REQUIRE(ld_q >= hd && ld_q % 8 == 0 && ld_kv >= hd && ld_kv % 8 == 0, F3S_ERR_INVALID_ARG,
              "row strides must be >= heads*head_dim and multiples of 8");
  if (num_rows == 0) return F3S_OK;
  F3S_REQUIRE(row_window_offset && q && k && v && d_out_f16 && stats && dq, F3S_ERR_INVALID_ARG,
              "null pointer argument");
  F3S_REQUIRE(n_tcb == 0 || (sparse_a_to_x_idx && tcb_bitmap), F3S_ERR_INVALID_ARG, "null TCB array");
  F3S_REQUIRE(!misaligned16(q) && !misaligned16(k) && !misaligned16(v) && !misaligned16(d_out_f16) &&
                  !misaligned16(dq) && !misaligned16(tcb_bitmap) && (reinterpret_cast<uintptr_t>(stats) & 7) == 0,
              F3S_ERR_INVALID_ARG, "tensors and bitmaps must be 16-byte aligned");
  const BwdKernelCfg kc = bwd_cfg(head_dim);
  const BwdSched sc = bwd_sched(n_tcb, block_w, heads, kc.warps_dq, kc.nt8, (size_t)(kc.d_pad / 8) * 4 * 32);
  F3S_REQUIRE(workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 255) == 0, F3S_ERR_WORKSPACE,
              "workspace must be non-null and 256-byte aligned");
  F3S_REQUIRE(workspace_bytes >= sc.bytes, F3S_ERR_WORKSPACE, "workspace too small: %zu < %zu", workspace_bytes,
              sc.bytes);
  BwdParams p;
  p.n_nodes = num_rows; p.n_rw = n_row_windows; p.heads = heads; p.d_real = head_dim;
  p.t8_per_tcb = block_w / 8;
  p.stats = reinterpret_cast<const float2 *>(stats);
  p.scale = 1.4426950408889634f / scale_divisor;
  p.out_scale = 1.f / scale_divisor;
  p.out_half = grads_are_half ? 1 : 0;
  p.fpart = 0;
  p.rwo = row_window_offset; p.sorted = sorted_row_windows; p.atox = sparse_a_to_x_idx;
  p.bitmap = reinterpret_cast<const unsigned long long *>(tcb_bitmap);
  p.a1 = static_cast<const __half *>(q); p.ld_a1 = ld_q;
  p.a2 = static_cast<const __half *>(d_out_f16); p.ld_a2 = hd;
  p.g1 = static_cast<const __half *>(k); p.ld_g1 = ld_kv;
  p.g2 = static_cast<const __half *>(v); p.ld_g2 = ld_kv;
  p.out1 = dq; p.out2 = nullptr;
  return run_bwd(p, sc, static_cast<unsigned char *>(workspace), kc, false, stream);
}

// dK and dV of a block of key/value rows from the TC blocks of the transposed graph's rows of that
// block.  k, v: the block's rows; q_g, d_out_f16_g, stats_g: gathered operands of ALL query rows,
// indexed by that plan's column ids (row strides ld_q, heads*head_dim, heads pairs).
extern "C" int f3s_backward_dkv(const int32_t *row_window_offset_t, const int32_t *sorted_row_windows_t,
                                const int32_t *sparse_a_to_x_idx_t, const uint64_t *tcb_bitmap_t, int64_t n_tcb_t,
                                int32_t num_rows, int32_t n_row_windows, int32_t block_w, int32_t heads,
                                int32_t head_dim, int64_t ld_kv, const void *k, const void *v, int64_t ld_q,
                                const void *q_g, const void *d_out_f16_g, const float *stats_g, float scale_divisor,
                                void *dk, void *dv, int32_t grads_are_half, void *workspace, size_t workspace_bytes,
                                f3s_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (int rc = check_stage_args(num_rows, n_row_windows, n_tcb_t, block_w, heads, head_dim, scale_divisor)) return rc;
  const int64_t hd = (int64_t)heads * head_dim;
  F3S_REQUIRE(ld_q >= hd && ld_q % 8 == 0 && ld_kv >= hd && ld_kv % 8 == 0, F3S_ERR_INVALID_ARG,
              "row strides must be >= heads*head_dim and multiples of 8");
  if (num_rows == 0) return F3S_OK;
  F3S_REQUIRE(row_window_offset_t && k && v && q_g && d_out_f16_g && stats_g && dk && dv, F3S_ERR_INVALID_ARG,
              "null pointer argument");
  F3S_REQUIRE(n_tcb_t == 0 || (sparse_a_to_x_idx_t && tcb_bitmap_t), F3S_ERR_INVALID_ARG, "null TCB array");
  F3S_REQUIRE(!misaligned16(k) && !misaligned16(v) && !misaligned16(q_g) && !misaligned16(d_out_f16_g) &&
                  !misaligned16(dk) && !misaligned16(dv) && !misaligned16(tcb_bitmap_t) &&
                  (reinterpret_cast<uintptr_t>(stats_g) & 7) == 0,
              F3S_ERR_INVALID_ARG, "tensors and bitmaps must be 16-byte aligned");
  const BwdKernelCfg kc = bwd_cfg(head_dim);
  const BwdSched sc = bwd_sched(n_tcb_t, block_w, heads, kc.warps_dkv, kc.nt8,
                                (size_t)2 * (kc.d_pad / 8 / kc.fsplit) * 4 * 32);
  F3S_REQUIRE(workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 255) == 0, F3S_ERR_WORKSPACE,
              "workspace must be non-null and 256-byte aligned");
  F3S_REQUIRE(workspace_bytes >= sc.bytes, F3S_ERR_WORKSPACE, "workspace too small: %zu < %zu", workspace_bytes,
              sc.bytes);
  BwdParams p;
  p.n_nodes = num_rows; p.n_rw = n_row_windows; p.heads = heads; p.d_real = head_dim;
  p.t8_per_tcb = block_w / 8;
  p.stats = reinterpret_cast<const float2 *>(stats_g);
  p.scale = 1.4426950408889634f / scale_divisor;
  p.out_scale = 1.f / scale_divisor;
  p.out_half = grads_are_half ? 1 : 0;
  p.fpart = 0;
  p.rwo = row_window_offset_t; p.sorted = sorted_row_windows_t; p.atox = sparse_a_to_x_idx_t;
  p.bitmap = reinterpret_cast<const unsigned long long *>(tcb_bitmap_t);
  p.a1 = static_cast<const __half *>(k); p.ld_a1 = ld_kv;
  p.a2 = static_cast<const __half *>(v); p.ld_a2 = ld_kv;
  p.g1 = static_cast<const __half *>(q_g); p.ld_g1 = ld_q;
  p.g2 = static_cast<const __half *>(d_out_f16_g); p.ld_g2 = hd;
  p.out1 = dk; p.out2 = dv;
  return run_bwd(p, sc, static_cast<unsigned char *>(workspace), kc, true, stream);
}
