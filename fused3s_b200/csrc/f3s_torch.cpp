// PyTorch extension module "F3S": the reference's operator surface (src/F3S.cpp:298-305,
// same op names, positional arguments and return tuples) on top of the f3s_b200 C ABI.
// Tensors are allocated here; every computation happens behind the C ABI.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cstdlib>
#include <tuple>
#include <vector>

#include "../../include/f3s_b200.h"

namespace {

#define CHECK_CUDA(x) TORCH_CHECK(x.device().is_cuda(), #x " must be a CUDA tensor")
#define CHECK_CONTIGUOUS(x) TORCH_CHECK(x.is_contiguous(), #x " must be contiguous")
#define CHECK_INPUT(x) \
  CHECK_CUDA(x);       \
  CHECK_CONTIGUOUS(x)

void check_status(int rc, const char *what) {
  TORCH_CHECK(rc == F3S_OK, what, " failed (status ", rc, "): ", f3s_last_error_string());
}

bool verbose() {
  static const bool v = std::getenv("F3S_VERBOSE") != nullptr;
  return v;
}

torch::Tensor workspace(size_t bytes, const torch::Device &dev) {
  return torch::empty({static_cast<int64_t>(bytes > 0 ? bytes : 1)},
                      torch::TensorOptions().dtype(torch::kUInt8).device(dev));
}

// preprocess_gpu (src/F3S.cpp:40-87): same arguments, same 8-tuple, the three caller
// tensors are filled in place.  The window count is taken from blockPartition.size(0)
// exactly as the reference does (src/F3S.cpp:55).
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, int>
preprocess_gpu(torch::Tensor colIdx, torch::Tensor rowPtr, int num_nodes, int blockSize_h, int blockSize_w,
               torch::Tensor blockPartition, torch::Tensor edgeToColumn, torch::Tensor edgeToRow) {
  CHECK_INPUT(colIdx);
  CHECK_INPUT(rowPtr);
  CHECK_INPUT(blockPartition);
  CHECK_INPUT(edgeToColumn);
  CHECK_INPUT(edgeToRow);
  TORCH_CHECK(colIdx.scalar_type() == torch::kInt32 && rowPtr.scalar_type() == torch::kInt32 &&
                  blockPartition.scalar_type() == torch::kInt32 && edgeToColumn.scalar_type() == torch::kInt32 &&
                  edgeToRow.scalar_type() == torch::kInt32,
              "preprocess_gpu takes int32 tensors");
  const int64_t nnz = colIdx.size(0);
  const int64_t n_rw = (static_cast<int64_t>(num_nodes) + 15) / 16;
  TORCH_CHECK(rowPtr.size(0) == static_cast<int64_t>(num_nodes) + 1, "rowPtr must have num_nodes+1 entries");
  TORCH_CHECK(blockPartition.size(0) == n_rw, "blockPartition must have ceil(num_nodes/16) entries");
  TORCH_CHECK(edgeToColumn.size(0) == nnz && edgeToRow.size(0) == nnz, "edgeToColumn/edgeToRow must have nnz entries");
  c10::cuda::CUDAGuard guard(colIdx.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  auto i32 = torch::TensorOptions().dtype(torch::kInt32).device(colIdx.device());
  auto rwo = torch::empty({n_rw + 1}, i32);
  const size_t ws_bytes = f3s_preprocess_workspace_bytes(num_nodes, nnz, blockSize_w);
  auto ws = workspace(ws_bytes, colIdx.device());
  int n_tcb = 0, max_tcb = 0;
  check_status(f3s_preprocess_count(colIdx.data_ptr<int>(), rowPtr.data_ptr<int>(), num_nodes, nnz, blockSize_h,
                                    blockSize_w, blockPartition.data_ptr<int>(), edgeToColumn.data_ptr<int>(),
                                    edgeToRow.data_ptr<int>(), rwo.data_ptr<int>(), ws.data_ptr(), ws_bytes, &n_tcb,
                                    &max_tcb, stream.stream()),
               "f3s_preprocess_count");
  auto sorted_rw = torch::empty({n_rw}, i32);
  auto rowid = torch::empty({n_tcb}, i32);
  auto tile_id = torch::empty({nnz}, torch::TensorOptions().dtype(torch::kUInt8).device(colIdx.device()));
  auto tcb_off = torch::empty({static_cast<int64_t>(n_tcb) + 1}, i32);
  auto atox = torch::empty({static_cast<int64_t>(n_tcb) * blockSize_w}, i32);
  const int64_t wpt = 16 * blockSize_w / 64;
  auto bitmap = torch::empty({static_cast<int64_t>(n_tcb) * wpt},
                             torch::TensorOptions().dtype(torch::kUInt64).device(colIdx.device()));
  check_status(f3s_preprocess_fill(colIdx.data_ptr<int>(), rowPtr.data_ptr<int>(), num_nodes, nnz, blockSize_h,
                                   blockSize_w, edgeToColumn.data_ptr<int>(), edgeToRow.data_ptr<int>(),
                                   rwo.data_ptr<int>(), n_tcb, sorted_rw.data_ptr<int>(), rowid.data_ptr<int>(),
                                   tile_id.data_ptr<uint8_t>(), tcb_off.data_ptr<int>(), atox.data_ptr<int>(),
                                   reinterpret_cast<uint64_t *>(bitmap.data_ptr()), ws.data_ptr(), ws_bytes,
                                   stream.stream()),
               "f3s_preprocess_fill");
  if (verbose()) printf("TC_Blocks:\t%d (max per window %d)\n", n_tcb, max_tcb);
  return std::make_tuple(rwo, sorted_rw, rowid, tile_id, tcb_off, atox, bitmap, n_tcb);
}

struct FwdOpts {
  int block_w = 16;
  bool softmax = true;
  float scale_divisor = 1.0f;
  bool save_sddmm = false;
  bool timed = true;  // the reference ops return the kernel time and block until it is known
  const char *sm_time_file = nullptr;  // checkSMActiveTime: write per-SM start/end times to this file
};

// One line per SM that took part: "start_ms end_ms" of its busy interval, the format of the
// reference's printSMTime (src/F3S_kernel.cu:43-75; its array is sized for 56 SMs, this one for
// every SM id the hardware can report).
void write_sm_times(const torch::Tensor &trace_cpu, const char *path) {
  FILE *f = fopen(path, "w");
  TORCH_CHECK(f != nullptr, "cannot open ", path);
  const int64_t *t = trace_cpu.data_ptr<int64_t>();
  for (int s = 0; s < F3S_SM_TRACE_SLOTS; ++s) {
    const uint64_t a = static_cast<uint64_t>(t[2 * s]), b = static_cast<uint64_t>(t[2 * s + 1]);
    if (b == 0) continue;  // SM not used by this launch
    fprintf(f, "%.15f %.15f\n", static_cast<double>(a) / 1e6, static_cast<double>(b) / 1e6);
  }
  fclose(f);
}

// Common body of the forward ops.  Q/K/V are [N, d] (the reference's layout) or [N, H, d].
std::vector<torch::Tensor> run_forward(const torch::Tensor &rwo, const c10::optional<torch::Tensor> &sortedRW,
                                       const torch::Tensor &atox, const torch::Tensor &bitmap, int nNodes,
                                       const torch::Tensor &Q, const torch::Tensor &K, const torch::Tensor &V,
                                       const FwdOpts &opt) {
  CHECK_INPUT(rwo);
  CHECK_INPUT(atox);
  CHECK_INPUT(bitmap);
  CHECK_INPUT(Q);
  CHECK_INPUT(K);
  CHECK_INPUT(V);
  if (sortedRW.has_value()) { CHECK_INPUT((*sortedRW)); }
  TORCH_CHECK(Q.scalar_type() == torch::kFloat16 && K.scalar_type() == torch::kFloat16 &&
                  V.scalar_type() == torch::kFloat16, "Q, K, V must be float16");
  TORCH_CHECK(Q.dim() == 2 || Q.dim() == 3, "Q must be [N, d] or [N, H, d]");
  // K and V may hold more rows than Q: a rank that owns a block of query rows still needs every key row
  TORCH_CHECK(K.sizes() == V.sizes() && K.dim() == Q.dim() && K.size(-1) == Q.size(-1) &&
                  (Q.dim() == 2 || K.size(1) == Q.size(1)),
              "K and V must have the same shape, and the same head count and head dim as Q");
  TORCH_CHECK(Q.size(0) >= nNodes, "Q has fewer rows than nNodes");
  const int heads = Q.dim() == 3 ? static_cast<int>(Q.size(1)) : 1;
  const int d = static_cast<int>(Q.size(-1));
  const int64_t ld = static_cast<int64_t>(heads) * d;
  const int n_rw = static_cast<int>(rwo.size(0)) - 1;
  const int64_t n_tcb = atox.size(0) / opt.block_w;
  c10::cuda::CUDAGuard guard(Q.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  auto f32 = torch::TensorOptions().dtype(torch::kFloat32).device(Q.device());
  std::vector<int64_t> oshape = Q.dim() == 3 ? std::vector<int64_t>{nNodes, heads, d} : std::vector<int64_t>{nNodes, d};
  auto out = torch::empty(oshape, f32);
  torch::Tensor sddmm = opt.save_sddmm ? torch::zeros({n_tcb * 16 * opt.block_w}, f32) : torch::zeros({0}, f32);
  const size_t ws_bytes = f3s_forward_workspace_bytes(n_rw, n_tcb, opt.block_w, heads, d);
  TORCH_CHECK(ws_bytes > 0, "unsupported shape: head dim ", d, " (supported: multiples of 16 up to 128), block width ", opt.block_w);
  auto ws = workspace(ws_bytes, Q.device());
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  if (opt.timed) {
    C10_CUDA_CHECK(cudaEventCreate(&e0));
    C10_CUDA_CHECK(cudaEventCreate(&e1));
    C10_CUDA_CHECK(cudaEventRecord(e0, stream.stream()));
  }
  torch::Tensor trace;
  int rc;
  if (opt.sm_time_file != nullptr) {
    // [slots][2] = (earliest start, latest end) in ns; int64 bit patterns of UINT64_MAX and 0
    trace = torch::zeros({F3S_SM_TRACE_SLOTS, 2}, torch::TensorOptions().dtype(torch::kInt64).device(Q.device()));
    trace.select(1, 0).fill_(-1);
    rc = f3s_forward_traced(rwo.data_ptr<int>(), sortedRW.has_value() ? sortedRW->data_ptr<int>() : nullptr,
                            atox.data_ptr<int>(), reinterpret_cast<const uint64_t *>(bitmap.data_ptr()), nNodes, n_rw,
                            n_tcb, opt.block_w, heads, d, ld, Q.data_ptr(), K.data_ptr(), V.data_ptr(),
                            opt.scale_divisor, opt.softmax ? 1 : 0, out.data_ptr<float>(), ws.data_ptr(), ws_bytes,
                            reinterpret_cast<uint64_t *>(trace.data_ptr()), stream.stream());
  } else {
    rc = f3s_forward(rwo.data_ptr<int>(), sortedRW.has_value() ? sortedRW->data_ptr<int>() : nullptr,
                     atox.data_ptr<int>(), reinterpret_cast<const uint64_t *>(bitmap.data_ptr()), nNodes, n_rw, n_tcb,
                     opt.block_w, heads, d, ld, Q.data_ptr(), K.data_ptr(), V.data_ptr(), opt.scale_divisor,
                     opt.softmax ? 1 : 0, out.data_ptr<float>(), opt.save_sddmm ? sddmm.data_ptr<float>() : nullptr,
                     ws.data_ptr(), ws_bytes, stream.stream());
  }
  float ms = 0.f;
  if (opt.timed) {
    cudaEventRecord(e1, stream.stream());
    cudaEventSynchronize(e1);
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
  }
  check_status(rc, "f3s_forward");
  // the timed ops have synchronised already, so asking the kernels how they fared costs one small copy
  if (opt.timed) check_status(f3s_forward_status(ws.data_ptr(), nullptr, stream.stream()), "f3s_forward (device status)");
  if (opt.sm_time_file != nullptr) write_sm_times(trace.cpu(), opt.sm_time_file);
  auto time = torch::tensor(ms, torch::TensorOptions().dtype(torch::kFloat32));
  return {time, out, sddmm};
}


// f3s_1tb1tcb (src/F3S.cpp:272-296): TCBs of width 8; optional masked score output.
std::vector<torch::Tensor> f3s_1tb1tcb(torch::Tensor rwo, torch::Tensor atox, torch::Tensor bitmap, int nNodes,
                                       torch::Tensor Q, torch::Tensor K, torch::Tensor V, bool applySoftmax,
                                       bool saveSddmmResult) {
  FwdOpts o;
  o.block_w = 8;
  o.softmax = applySoftmax;
  o.save_sddmm = saveSddmmResult;
  return run_forward(rwo, c10::nullopt, atox, bitmap, nNodes, Q, K, V, o);
}

// f3s_1tb1rw (src/F3S.cpp:145-183)
std::vector<torch::Tensor> f3s_1tb1rw(torch::Tensor rwo, torch::Tensor atox, torch::Tensor bitmap, int nNodes,
                                      torch::Tensor Q, torch::Tensor K, torch::Tensor V, int /*nWarpPerBlock*/,
                                      bool applySoftmax, bool checkSMActiveTime) {
  FwdOpts o;
  o.softmax = applySoftmax;
  if (checkSMActiveTime) o.sm_time_file = "SM_time_f3s1tb1rw.csv";  // file name of src/F3S_kernel.cu:514
  return run_forward(rwo, c10::nullopt, atox, bitmap, nNodes, Q, K, V, o);
}

// f3s_1tb1rw_scheduled (src/F3S.cpp:185-219)
std::vector<torch::Tensor> f3s_1tb1rw_scheduled(torch::Tensor rwo, torch::Tensor sortedRW, torch::Tensor atox,
                                                torch::Tensor bitmap, int nNodes, torch::Tensor Q, torch::Tensor K,
                                                torch::Tensor V, int /*nWarpPerBlock*/, bool checkSMActiveTime) {
  FwdOpts o;
  if (checkSMActiveTime) o.sm_time_file = "SM_time_f3s1tb1rw_scheduled.csv";  // src/F3S_kernel.cu:577
  return run_forward(rwo, sortedRW, atox, bitmap, nNodes, Q, K, V, o);
}

// f3s_1tb1rw_scheduled_permuteV (src/F3S.cpp:222-244)
std::vector<torch::Tensor> f3s_1tb1rw_scheduled_permuteV(torch::Tensor rwo, torch::Tensor sortedRW,
                                                         torch::Tensor atox, torch::Tensor bitmap, int nNodes,
                                                         torch::Tensor Q, torch::Tensor K, torch::Tensor V,
                                                         int /*nWarpPerBlock*/) {
  return run_forward(rwo, sortedRW, atox, bitmap, nNodes, Q, K, V, FwdOpts{});
}

// f3s_1tb1rw_scheduled_permuteV_scaleQK (src/F3S.cpp:247-270): scores are divided by scalingFactor.
std::vector<torch::Tensor> f3s_1tb1rw_scheduled_permuteV_scaleQK(torch::Tensor rwo, torch::Tensor sortedRW,
                                                                 torch::Tensor atox, torch::Tensor bitmap,
                                                                 int nNodes, torch::Tensor Q, torch::Tensor K,
                                                                 torch::Tensor V, float scalingFactor,
                                                                 int /*nWarpPerBlock*/) {
  FwdOpts o;
  o.scale_divisor = scalingFactor;
  return run_forward(rwo, sortedRW, atox, bitmap, nNodes, Q, K, V, o);
}

// Extension (no reference counterpart): the scheduled op without the blocking event timing;
// returns only the output tensor and leaves the work queued on the current stream.
torch::Tensor f3s_forward_async(torch::Tensor rwo, c10::optional<torch::Tensor> sortedRW, torch::Tensor atox,
                                torch::Tensor bitmap, int nNodes, torch::Tensor Q, torch::Tensor K, torch::Tensor V,
                                float scalingFactor, int blockSize_w, bool applySoftmax) {
  FwdOpts o;
  o.block_w = blockSize_w;
  o.scale_divisor = scalingFactor;
  o.softmax = applySoftmax;
  o.timed = false;
  return run_forward(rwo, sortedRW, atox, bitmap, nNodes, Q, K, V, o)[1];
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("preprocess_gpu", &preprocess_gpu, "Preprocess Step on (CUDA)");
  m.def("f3s_1tb1tcb", &f3s_1tb1tcb, "fused3S 1tb1tcb");
  m.def("f3s_1tb1rw", &f3s_1tb1rw, "fused3S 1tb1rw");
  m.def("f3s_1tb1rw_scheduled", &f3s_1tb1rw_scheduled, "fused3S 1tb1rw scheduled");
  m.def("f3s_1tb1rw_scheduled_permuteV", &f3s_1tb1rw_scheduled_permuteV, "fused3S 1tb1rw scheduled permuteV");
  m.def("f3s_1tb1rw_scheduled_permuteV_scaleQK", &f3s_1tb1rw_scheduled_permuteV_scaleQK,
        "fused3S 1tb1rw scheduled permuteV scaleQK");
  m.def("f3s_forward_async", &f3s_forward_async, "fused3S forward, no host synchronisation");
}
