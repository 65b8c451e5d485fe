// The score stage (SDDMM) of the fused path on the 5th-generation tensor cores: tcgen05.mma with the
// accumulator in tensor memory (TMEM).
//
// A row window has 16 query rows, below the smallest M (64) a tcgen05.mma accepts, so the product is
// taken in its transposed form: S^T = K_g Q^T with M = 128 gathered key rows, N = 16 query rows,
// K = 64 features.  One CTA of four warps owns one row window at a time:
//   * every thread holds the id of one key row of the step; eight lanes copy a row together (one 128-byte
//     request, 16-byte cp.async each) into a tile in the
//     canonical K-major layout with 128-byte swizzle (row pitch 128 B, groups of eight rows 1024 B apart);
//     three tiles rotate, so two gathers are in flight while a step is multiplied;
//   * one thread issues four tcgen05.mma (K = 16 each; A = key tile, B = Q window, both read from shared
//     memory through matrix descriptors) into a 128-lane x 16-column fp32 accumulator in TMEM and commits
//     them to an mbarrier; two accumulators alternate, so the product of step i runs while step i-1 is
//     read back and stored;
//   * every warp reads its 32 lanes of the accumulator with tcgen05.ld (thread = gathered column, 16
//     registers = the 16 query rows), masks by the TC-block occupancy words, transposes through a small
//     staging area and stores the scores with 16-byte coalesced writes in the layout of the reference's
//     score dump (src/F3S_kernel.cu:99-115).
// Every wait is bounded; a wait that runs out sets the status word and the CTA leaves after freeing its TMEM.
//
// This is the stage a tensor-memory version of the fused kernel would start from; it exists as an entry
// point of its own (a score dump for 16-wide or 8-wide TC blocks, d = 64) so that the tcgen05 data path
// can be checked against the oracle and timed against the mma.sync kernels on the same arrays.
#include "attn_common.cuh"

namespace f3s {
namespace umma {

constexpr int THREADS = 128;
constexpr int D = 64;
constexpr int STEP_COLS = 128;                 // gathered key rows per product (M)
constexpr int TILE_BYTES = STEP_COLS * D * 2;  // 16 KB
constexpr int Q_BYTES = 16 * D * 2;            // 2 KB
constexpr int STAGES = 3;                      // key tiles in flight
constexpr int OUT_STRIDE = 17;                 // floats per staged column (16 rows + 1: conflict-free transposition)
constexpr int OUT_BYTES = 4 * 32 * OUT_STRIDE * 4;  // per warp 32 columns x 16 rows, staged for coalesced stores
constexpr int SMEM_BYTES = STAGES * TILE_BYTES + Q_BYTES + OUT_BYTES + 1024;  // + alignment slack
constexpr int TMEM_COLS = 32;                  // smallest allocation: two accumulators of 16 columns
constexpr int WAIT_LIMIT = 1 << 22;

__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
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
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
  for (int it = 0; it < WAIT_LIMIT; ++it)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows 128 bytes apart, groups of
// eight rows 1024 bytes apart; the tile starts on a 1024-byte boundary.  byte_offset selects the K slice
// (32 bytes per 16 fp16 features) inside the swizzle atom.
__device__ __forceinline__ uint64_t smem_desc(uint32_t tile_addr, uint32_t byte_offset) {
  uint64_t d = 0;
  d |= (uint64_t)(((tile_addr + byte_offset) & 0x3FFFFu) >> 4);  // start address, bits [0,14)
  d |= (uint64_t)1 << 16;                                        // leading byte offset (unused with swizzle), bits [16,30)
  d |= (uint64_t)(1024 >> 4) << 32;                              // stride byte offset, bits [32,46)
  d |= (uint64_t)1 << 46;                                        // descriptor version of sm_100
  d |= (uint64_t)2 << 61;                                        // layout type: SWIZZLE_128B
  return d;
}

// Instruction descriptor: fp16 x fp16 -> fp32, A and B K-major, M = 128, N = 16.
constexpr uint32_t IDESC = (1u << 4) | ((16u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void mma_f16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(IDESC), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)  // no output lane disabled
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

struct Params {
  const int *rwo;
  const int *atox;
  const unsigned long long *bitmap;
  const __half *q, *k;
  float *sddmm;
  int *status;
  int n_nodes, n_rw, t8_per_tcb;
  long long ld_q, ld_k;
};

static __global__ void __launch_bounds__(THREADS) sddmm_umma_kernel(const Params p) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long mbar_storage[2];
  __shared__ uint32_t tmem_base_s;
  const int tid = threadIdx.x, warp = tid >> 5;
  const uint32_t base_s = (smem_u32(smem_raw) + 1023u) & ~1023u;  // tiles sit on 1024-byte boundaries
  const uint32_t q_s = base_s + STAGES * TILE_BYTES;
  float *stage = reinterpret_cast<float *>(smem_raw + (base_s - smem_u32(smem_raw)) + STAGES * TILE_BYTES + Q_BYTES) +
                 warp * 32 * OUT_STRIDE;
  const int lane = tid & 31;
  const uint32_t bar0 = smem_u32(&mbar_storage[0]);

  if (tid == 0) {
    mbar_init(bar0, 1);
    mbar_init(bar0 + 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {  // one warp allocates the CTA's tensor memory and gives up the right to allocate more
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_d = tmem_base_s;  // two accumulators: columns [0,16) and [16,32)
  const uint32_t my_lanes = (uint32_t)(warp * 32) << 16;
  bool ok = true;
  // g counts the products this CTA has issued: key tile g % STAGES, accumulator and barrier g & 1, and the
  // barrier's phase (g >> 1) & 1 follow from it, across row windows
  uint32_t g = 0;

  for (int w = blockIdx.x; w < p.n_rw && ok; w += gridDim.x) {
    const int t8b = p.rwo[w] * p.t8_per_tcb, t8e = p.rwo[w + 1] * p.t8_per_tcb;
    const int nsteps = (t8e - t8b + 15) / 16;  // 16 tiles of 8 columns per product
    if (nsteps == 0) continue;
    const uint32_t g0 = g;  // product number of this window's step 0
    const long long slots_end = (long long)t8e * 8;
    // column id of this thread's key row, loaded one gather ahead of its use
    long long next_slot = (long long)t8b * 8 + tid;
    int next_col = next_slot < slots_end ? __ldg(p.atox + next_slot) : 0;
    auto gather = [&](int step) {  // steps are gathered in order: 0, 1, 2, ...
      const bool real = next_slot < slots_end;
      const int col = next_col;
      next_slot += STEP_COLS;
      next_col = next_slot < slots_end ? __ldg(p.atox + next_slot) : 0;
      // Eight consecutive lanes copy one key row (one 128-byte request), a warp the 32 rows whose ids its
      // lanes hold: lane l copies piece l % 8 of rows l / 8 + 4 i, i = 0..7, of the warp's quarter of the tile.
      const uint32_t tile = base_s + ((g0 + (uint32_t)step) % STAGES) * TILE_BYTES;
      const int piece = lane & 7;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int rl = (lane >> 3) + 4 * i;
        const int idx = __shfl_sync(FULL, col, rl);
        const int ok_row = __shfl_sync(FULL, (int)real, rl);
        const int r = warp * 32 + rl;
        cp_async16(tile + (uint32_t)r * 128u + (((uint32_t)piece ^ (uint32_t)(r & 7)) << 4),
                   reinterpret_cast<const char *>(p.k + (size_t)idx * p.ld_k) + piece * 16, ok_row ? 16 : 0);
      }
    };
    // Wait for the product of `step`, read this warp's 32 lanes of its accumulator, mask, store.
    auto finish = [&](int step) {
      const uint32_t gs = g0 + (uint32_t)step;
      const int t8 = t8b + step * 16 + (tid >> 3);
      unsigned long long w0 = 0, w1 = 0;
      if (t8 < t8e) {  // occupancy words of this thread's 8-column tile, fetched while the product runs
        w0 = __ldg(p.bitmap + (size_t)t8 * 2);
        w1 = __ldg(p.bitmap + (size_t)t8 * 2 + 1);
      }
      bool mine = mbar_wait_bounded(bar0 + (gs & 1u) * 8, (gs >> 1) & 1u);
      if (!mine) atomicExch(p.status, STATUS_WAIT_TIMEOUT);
      if (!__syncthreads_and(mine)) {  // some thread gave up: everybody leaves
        ok = false;
        return;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      uint32_t acc[16];
      tmem_ld16(tmem_d + my_lanes + (gs & 1u) * 16u, acc);
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");  // ordered before the next barrier
      {  // mask (row i of the window, column c of the tile: bit 63 - (i % 8) * 8 - c of word i / 8) and stage
        const int c = tid & 7;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const unsigned long long word = i < 8 ? w0 : w1;
          const bool set = (word >> (63 - (i & 7) * 8 - c)) & 1ull;
          stage[lane * OUT_STRIDE + i] = set ? __uint_as_float(acc[i]) : 0.f;
        }
      }
      __syncwarp();
      // the warp's four tiles are 2 KB of consecutive floats in the dump ([tile][row][column]): lane l
      // writes floats 4 l .. 4 l + 3 of every tile = row l / 2, columns 4 (l % 2) .. + 3
      const int t8w = t8b + step * 16 + warp * 4;  // first tile of this warp
      const int row = lane >> 1, c0 = (lane & 1) * 4;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (t8w + k < t8e) {
          const float *src = stage + (k * 8 + c0) * OUT_STRIDE + row;
          const float4 v = make_float4(src[0], src[OUT_STRIDE], src[2 * OUT_STRIDE], src[3 * OUT_STRIDE]);
          __stcs(reinterpret_cast<float4 *>(p.sddmm + (size_t)(t8w + k) * 128 + lane * 4), v);
        }
      }
      __syncwarp();  // the staging area is rewritten by the next step
    };
    {  // Q window (rows past the last node read as zero) joins the first copy group
      const int r = tid >> 3, c = tid & 7;
      const int gr = w * 16 + r;
      const bool in = gr < p.n_nodes;
      cp_async16(q_s + r * 128 + ((c ^ (r & 7)) << 4), p.q + (size_t)(in ? gr : 0) * p.ld_q + c * 8, in ? 16 : 0);
    }
    gather(0);
    cp_async_commit();
    if (nsteps > 1) gather(1);
    cp_async_commit();
    for (int step = 0; step < nsteps && ok; ++step) {
      cp_async_wait<1>();  // every group but the newest has landed: this step's tile (and Q) are there
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // visible to the tensor core's reads
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncthreads();  // also: every warp has read the accumulator this product is about to overwrite
      if (tid == 0) {
        const uint32_t gs = g0 + (uint32_t)step;
        const uint32_t tile = base_s + (gs % STAGES) * TILE_BYTES;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          mma_f16_ss(tmem_d + (gs & 1u) * 16u, smem_desc(tile, ks * 32), smem_desc(q_s, ks * 32), ks > 0 ? 1u : 0u);
        mma_commit(bar0 + (gs & 1u) * 8);
      }
      if (step > 0) finish(step - 1);  // runs beside the product just issued
      // the tile of step-1 has been multiplied (its product was waited for): it takes the gather of step+2
      if (ok && step + 2 < nsteps) gather(step + 2);
      cp_async_commit();
    }
    if (ok) finish(nsteps - 1);
    g = g0 + (uint32_t)nsteps;
    cp_async_wait<0>();
    __syncthreads();  // the Q tile is free for the next window
  }
  cp_async_wait<0>();
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"((uint32_t)TMEM_COLS) : "memory");
}

}  // namespace umma
}  // namespace f3s

using namespace f3s;

extern "C" int f3s_sddmm_umma(const int32_t *row_window_offset, const int32_t *sparse_a_to_x_idx,
                              const uint64_t *tcb_bitmap, int32_t num_nodes, int32_t n_row_windows, int64_t n_tcb,
                              int32_t block_w, int32_t head_dim, int64_t ld_q, const void *q, int64_t ld_k,
                              const void *k, float *sddmm_out, void *workspace, size_t workspace_bytes,
                              f3s_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  F3S_REQUIRE(num_nodes >= 0 && n_row_windows == (num_nodes + 15) / 16 && n_tcb >= 0, F3S_ERR_INVALID_ARG, "bad size");
  F3S_REQUIRE(block_w == 8 || block_w == 16, F3S_ERR_UNSUPPORTED, "block_w must be 8 or 16, got %d", block_w);
  F3S_REQUIRE(head_dim == 64, F3S_ERR_UNSUPPORTED, "the tensor-memory score kernel is built for head_dim 64");
  F3S_REQUIRE(ld_q >= 64 && ld_k >= 64 && ld_q % 8 == 0 && ld_k % 8 == 0, F3S_ERR_INVALID_ARG, "bad row stride");
  F3S_REQUIRE(n_tcb * block_w < (1ll << 31), F3S_ERR_UNSUPPORTED, "n_tcb*block_w exceeds int32");
  F3S_REQUIRE(workspace != nullptr && workspace_bytes >= 64 && (reinterpret_cast<uintptr_t>(workspace) & 15) == 0,
              F3S_ERR_WORKSPACE, "64 bytes of 16-byte aligned device scratch are needed for the status word");
  if (num_nodes == 0 || n_tcb == 0) return F3S_OK;
  F3S_REQUIRE(row_window_offset && sparse_a_to_x_idx && tcb_bitmap && q && k && sddmm_out, F3S_ERR_INVALID_ARG,
              "null pointer argument");
  F3S_REQUIRE(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k)) & 15) == 0, F3S_ERR_INVALID_ARG,
              "q and k must be 16-byte aligned");
  umma::Params p;
  p.rwo = row_window_offset;
  p.atox = sparse_a_to_x_idx;
  p.bitmap = reinterpret_cast<const unsigned long long *>(tcb_bitmap);
  p.q = static_cast<const __half *>(q);
  p.k = static_cast<const __half *>(k);
  p.sddmm = sddmm_out;
  p.status = static_cast<int *>(workspace) + HDR_STATUS;  // where f3s_forward_status looks
  p.n_nodes = num_nodes;
  p.n_rw = n_row_windows;
  p.t8_per_tcb = block_w / 8;
  p.ld_q = ld_q;
  p.ld_k = ld_k;
  F3S_CUDA_TRY(cudaMemsetAsync(workspace, 0, 64, stream));
  F3S_CUDA_TRY(cudaFuncSetAttribute(umma::sddmm_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    umma::SMEM_BYTES));
  const long long want = (long long)sm_count() * 3;  // three CTAs per SM: 61 KB of shared memory, 32 TMEM columns each
  const int grid = (int)(n_row_windows < want ? n_row_windows : want);
  umma::sddmm_umma_kernel<<<grid, umma::THREADS, umma::SMEM_BYTES, stream>>>(p);
  F3S_CHECK_LAUNCH();
  return F3S_OK;
}
