// Measurement aid: how fast can this GPU gather 128-byte rows from a table at random row ids?
// The fused attention kernel is a gather of exactly that shape (one fp16 K or V row of 64 features per
// gathered column), so this rate -- with the table smaller than the L2 cache, or larger -- is the
// ceiling that its achieved gather rate is compared with.  Nothing but loads: each group of eight lanes
// reads one row in 16-byte pieces, eight rows per lane in flight, folded into a register that is stored
// only under a condition that never holds (it keeps the loads alive).
#include "common.cuh"

namespace f3s {

constexpr int PROBE_THREADS = 512;
constexpr int PROBE_UNROLL = 8;

static __global__ void __launch_bounds__(PROBE_THREADS)
gather_probe_kernel(const uint4 *__restrict__ table, const int *__restrict__ idx, long long n_idx, unsigned *sink) {
  const int lane = threadIdx.x & 31;
  const int rl = lane >> 3, ch = lane & 7;  // row within a group of four, 16-byte piece of the row
  const long long warp = ((long long)blockIdx.x * PROBE_THREADS + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * PROBE_THREADS) >> 5;
  constexpr int ROWS_PER_ITER = 4 * PROBE_UNROLL;
  unsigned acc = 0;
  for (long long base = warp * ROWS_PER_ITER; base + ROWS_PER_ITER <= n_idx; base += n_warps * ROWS_PER_ITER) {
    int id[PROBE_UNROLL];
#pragma unroll
    for (int i = 0; i < PROBE_UNROLL; ++i) id[i] = __ldg(idx + base + i * 4 + rl);
    uint4 v[PROBE_UNROLL];
#pragma unroll
    for (int i = 0; i < PROBE_UNROLL; ++i) v[i] = __ldcg(table + (size_t)id[i] * 8 + ch);
#pragma unroll
    for (int i = 0; i < PROBE_UNROLL; ++i) acc ^= v[i].x ^ v[i].y ^ v[i].z ^ v[i].w;
  }
  if (acc == 0x9e3779b9u) sink[0] = acc;  // the table holds zeros: never true, but the compiler cannot know
}

}  // namespace f3s

extern "C" int f3s_probe_gather_rows(const void *table, int64_t table_rows, const int32_t *row_ids, int64_t n_ids,
                                     void *sink, f3s_stream_t stream_) {
  using namespace f3s;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  F3S_REQUIRE(table && row_ids && sink, F3S_ERR_INVALID_ARG, "null pointer argument");
  F3S_REQUIRE(table_rows > 0 && n_ids >= 0, F3S_ERR_INVALID_ARG, "table_rows > 0 and n_ids >= 0 required");
  F3S_REQUIRE((reinterpret_cast<uintptr_t>(table) & 15) == 0, F3S_ERR_INVALID_ARG, "table must be 16-byte aligned");
  gather_probe_kernel<<<sm_count() * 4, PROBE_THREADS, 0, stream>>>(static_cast<const uint4 *>(table), row_ids, n_ids,
                                                                    static_cast<unsigned *>(sink));
  F3S_CHECK_LAUNCH();
  return F3S_OK;
}
