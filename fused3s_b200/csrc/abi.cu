// Library-wide pieces of the C ABI: version, error text, device queries, host-side partition.
#include <stdarg.h>
#include <string.h>

#include "common.cuh"

namespace f3s {

static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

static unsigned long long g_launches = 0;  // kernels launched by this library in this process
void note_launches(int n) { __atomic_fetch_add(&g_launches, (unsigned long long)n, __ATOMIC_RELAXED); }

// Number of SMs of the current device.  A failed query is not papered over: the last CUDA error stays
// pending for the launch that follows (which reports it), and the grid falls back to one B200's worth
// of CTAs, which is correct on any device because the kernels are persistent.
int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
      set_error("cudaDeviceGetAttribute(multiProcessorCount) failed on device %d; using 148", dev);
      return 148;  // not cached: asked again on the next call
    }
    cached[dev] = n;
  }
  return cached[dev];
}

// Plan validation: every index a forward / backward kernel would dereference without a check.
// result[0] = number of violations, result[1] = kind of the first one seen, result[2] = its position,
// result[3] = its value.
enum { BAD_RWO_START = 1, BAD_RWO_ORDER = 2, BAD_RWO_END = 3, BAD_COLUMN = 4, BAD_WINDOW_ID = 5 };

__device__ __forceinline__ void report(int *result, int kind, long long pos, int value) {
  if (atomicAdd(&result[0], 1) == 0) {
    result[1] = kind;
    result[2] = (int)(pos > 0x7fffffff ? 0x7fffffff : pos);
    result[3] = value;
  }
}

static __global__ void validate_plan_kernel(const int *__restrict__ rwo, const int *__restrict__ sorted,
                                            const int *__restrict__ atox, int n_rw, long long n_tcb, int block_w,
                                            int num_kv_rows, int *result) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long t0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (long long i = t0; i <= n_rw; i += stride) {
    const int a = rwo[i];
    if (i == 0 && a != 0) report(result, BAD_RWO_START, 0, a);
    if (i == n_rw && (long long)a != n_tcb) report(result, BAD_RWO_END, i, a);
    if (i < n_rw && rwo[i + 1] < a) report(result, BAD_RWO_ORDER, i, a);
    if (i < n_rw && sorted != nullptr) {
      const int w = sorted[i];
      if (w < 0 || w >= n_rw) report(result, BAD_WINDOW_ID, i, w);
    }
  }
  const long long n_idx = n_tcb * block_w;
  for (long long i = t0; i < n_idx; i += stride) {
    const int c = atox[i];
    if (c < 0 || c >= num_kv_rows) report(result, BAD_COLUMN, i, c);
  }
}

}  // namespace f3s

extern "C" int f3s_validate_plan(const int32_t *row_window_offset, const int32_t *sorted_row_windows,
                                 const int32_t *sparse_a_to_x_idx, int32_t n_row_windows, int64_t n_tcb,
                                 int32_t block_w, int32_t num_kv_rows, void *workspace, size_t workspace_bytes,
                                 f3s_stream_t stream_) {
  using namespace f3s;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  F3S_REQUIRE(n_row_windows >= 0 && n_tcb >= 0 && num_kv_rows >= 0, F3S_ERR_INVALID_ARG, "negative size");
  F3S_REQUIRE(block_w == 8 || block_w == 16, F3S_ERR_UNSUPPORTED, "block_w must be 8 or 16, got %d", block_w);
  F3S_REQUIRE(row_window_offset != nullptr && (n_tcb == 0 || sparse_a_to_x_idx != nullptr), F3S_ERR_INVALID_ARG,
              "null plan array");
  F3S_REQUIRE(workspace != nullptr && workspace_bytes >= 16 && (reinterpret_cast<uintptr_t>(workspace) & 15) == 0,
              F3S_ERR_WORKSPACE, "validation needs 16 bytes of 16-byte aligned device scratch");
  int *result = static_cast<int *>(workspace);
  F3S_CUDA_TRY(cudaMemsetAsync(result, 0, 16, stream));
  const long long work = n_tcb * block_w > n_row_windows ? n_tcb * block_w : (long long)n_row_windows + 1;
  long long blocks = (work + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  validate_plan_kernel<<<(int)blocks, 256, 0, stream>>>(row_window_offset, sorted_row_windows, sparse_a_to_x_idx,
                                                        n_row_windows, n_tcb, block_w, num_kv_rows, result);
  F3S_CHECK_LAUNCH();
  int host[4] = {0, 0, 0, 0};
  F3S_CUDA_TRY(cudaMemcpyAsync(host, result, 16, cudaMemcpyDeviceToHost, stream));
  F3S_CUDA_TRY(cudaStreamSynchronize(stream));
  if (host[0] == 0) return F3S_OK;
  static const char *kinds[] = {"?", "row_window_offset[0] is not 0", "row_window_offset decreases",
                                "row_window_offset[n_row_windows] differs from n_tcb",
                                "column id outside [0, num_kv_rows)", "window id outside [0, n_row_windows)"};
  const int kind = host[1] >= 1 && host[1] <= 5 ? host[1] : 0;
  set_error("plan invalid: %d violation(s); first seen: %s at position %d (value %d)", host[0], kinds[kind], host[2],
            host[3]);
  return F3S_ERR_INVALID_ARG;
}

extern "C" int f3s_version(void) { return 200; }

extern "C" uint64_t f3s_kernel_launch_count(void) { return __atomic_load_n(&f3s::g_launches, __ATOMIC_RELAXED); }

extern "C" const char *f3s_last_error_string(void) { return f3s::g_error; }

// Contiguous window ranges with near-equal TCB counts: cut k is the first window whose
// TCB prefix reaches k/n_parts of the total.  Host only.
extern "C" int f3s_partition_row_windows(const int32_t *rwo, int32_t n_rw, int32_t n_parts, int32_t *cuts) {
  F3S_REQUIRE(rwo && cuts, F3S_ERR_INVALID_ARG, "null pointer argument");
  F3S_REQUIRE(n_rw >= 0 && n_parts >= 1, F3S_ERR_INVALID_ARG, "n_row_windows >= 0 and n_parts >= 1 required");
  const long long total = rwo[n_rw] - rwo[0];
  cuts[0] = 0;
  int w = 0;
  for (int k = 1; k < n_parts; ++k) {
    const long long want = rwo[0] + (total * k + n_parts / 2) / n_parts;
    while (w < n_rw && rwo[w] < want) ++w;
    // choose the closer of the two neighbouring boundaries
    if (w > cuts[k - 1] && w <= n_rw && (want - rwo[w - 1]) < (rwo[w < n_rw ? w : n_rw] - want)) --w;
    if (w < cuts[k - 1]) w = cuts[k - 1];
    cuts[k] = w;
  }
  cuts[n_parts] = n_rw;
  return F3S_OK;
}
