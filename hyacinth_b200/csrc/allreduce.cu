// Exact cross-rank sum of the packed integer Gram over the 1-D row distribution (NCCL).
//
// Contract (reference: src/allreduce_1drow.cu:145-178): every rank ends with the integer sum of all ranks'
// packed Grams, in the same 63-bit-limb format; the column exponents are reduced with an integer minimum.
//
// NCCL can only add machine words, so each multi-limb value is first cut into slices narrow enough that the
// sum over all ranks cannot carry out of a 64-bit word; the slices are summed with ONE ncclAllReduce on one
// contiguous buffer and then re-assembled.  The reference hard-codes twelve slice layouts; here the slice
// width and count are derived from the communicator size (slice_plan) and one pair of kernels handles every
// case.  Integer addition is associative, so the result does not depend on rank order or on the algorithm
// NCCL picks (ring, tree or in-switch reduction).
#include "hyb_internal.h"
#include "slices.cuh"
#include <hyacin_b200.h>

namespace hyb {

// A value of `order` limbs has at most 63 * order + 1 significant bits including its sign.
SlicePlan slice_plan(int order, int ranks) {
  int log_r = 0; while ((int64_t(1) << log_r) < ranks) ++log_r;
  SlicePlan p; p.width = 64 - log_r; if (p.width > 62) p.width = 62;
  const int total = 63 * order + 1;
  p.slices = 2;
  while (total - (p.slices - 1) * p.width + log_r > 64) ++p.slices;
  // with the slice count fixed, use the narrowest width that still fits: keeps magnitudes small and even
  while (p.width > 1 && total - (p.slices - 1) * (p.width - 1) + log_r <= 64) --p.width;
  return p;
}

namespace {

__global__ void __launch_bounds__(256)
limbs_to_slices_kernel(int order, SlicePlan plan, uint64_t count, const uint64_t* __restrict__ A, uint64_t* __restrict__ S) {
  const uint64_t i = uint64_t(blockIdx.x) * 256 + threadIdx.x; if (i >= count) return;
  const uint64_t* src = A + uint64_t(blockIdx.y) * order * count + i;
  uint64_t* dst = S + uint64_t(blockIdx.y) * plan.slices * count + i;
  W192 v = load_value(src, count, order);
  const uint64_t mask = (uint64_t(1) << plan.width) - 1;
  for (int s = 0; s + 1 < plan.slices; ++s) { dst[uint64_t(s) * count] = v.w[0] & mask; sar(v, plan.width); }
  dst[uint64_t(plan.slices - 1) * count] = v.w[0];         // signed remainder (two's complement)
}

__global__ void __launch_bounds__(256)
slices_to_limbs_kernel(int order, SlicePlan plan, uint64_t count, const uint64_t* __restrict__ S, uint64_t* __restrict__ A) {
  const uint64_t i = uint64_t(blockIdx.x) * 256 + threadIdx.x; if (i >= count) return;
  const uint64_t* src = S + uint64_t(blockIdx.y) * plan.slices * count + i;
  uint64_t* dst = A + uint64_t(blockIdx.y) * order * count + i;
  W192 v; v.w[0] = v.w[1] = v.w[2] = 0;
  for (int s = 0; s < plan.slices; ++s) add_shifted(v, src[uint64_t(s) * count], s + 1 == plan.slices, s * plan.width);
  constexpr uint64_t m63 = 0x7fffffffffffffffull;
  for (int l = 0; l + 1 < order; ++l) { dst[uint64_t(l) * count] = v.w[0] & m63; sar(v, 63); }
  dst[uint64_t(order - 1) * count] = v.w[0];
}

}  // namespace

int slice_count(int order, int ranks) { return slice_plan(order, ranks).slices; }
void slice_layout(int order, int ranks, int* slices, int* width) { const SlicePlan p = slice_plan(order, ranks); *slices = p.slices; *width = p.width; }

void launch_limbs_to_slices(cudaStream_t stream, int panels, int order, int ranks, uint64_t count, const uint64_t* A, uint64_t* S) {
  dim3 grid(unsigned((count + 255) / 256), unsigned(panels));
  count_launch();
  limbs_to_slices_kernel<<<grid, 256, 0, stream>>>(order, slice_plan(order, ranks), count, A, S);
  HYB_CUDA(cudaGetLastError());
}
void launch_slices_to_limbs(cudaStream_t stream, int panels, int order, int ranks, uint64_t count, const uint64_t* S, uint64_t* A) {
  dim3 grid(unsigned((count + 255) / 256), unsigned(panels));
  count_launch();
  slices_to_limbs_kernel<<<grid, 256, 0, stream>>>(order, slice_plan(order, ranks), count, S, A);
  HYB_CUDA(cudaGetLastError());
}

}  // namespace hyb

extern "C" void hyacinB200SlicePlan(int32_t orderA, int32_t ranks, int32_t* slices, int32_t* widthBits) {
  int s = 0, w = 0;
  if (orderA >= 1 && orderA <= 3 && ranks >= 1) hyb::slice_layout(orderA, ranks, &s, &w);
  if (slices) *slices = s; if (widthBits) *widthBits = w;
}

#ifdef HYACIN_BUILD_NO_NCCL
namespace hyb { uint64_t* allreduce_to_slices(const hyacinHandle_t*, int, int, uint64_t, const uint64_t*, int*) { return nullptr; } }
extern "C" void hyacinAllReduce1Drow(const hyacinHandle_t*, int32_t, int32_t, uint64_t, uint64_t*) {}
extern "C" void hyacinAllReduceVExp(const hyacinHandle_t*, uint64_t, int32_t*) {}
#else

namespace hyb {
uint64_t* allreduce_to_slices(const hyacinHandle_t* handle, int panels, int order, uint64_t count, const uint64_t* C, int* ranks_out) {
  if (panels <= 0 || order <= 0 || order > 3 || count == 0 || handle->ncclComm == nullptr) return nullptr;
  int ranks = 0;
  if (ncclCommCount(handle->ncclComm, &ranks) != ncclSuccess || ranks <= 1) return nullptr;
  timer_mark(handle, Segment::Comm);
  cudaStream_t stream = handle->cudaStream;
  const uint64_t words = uint64_t(panels) * uint64_t(slice_count(order, ranks)) * count;
  uint64_t* S = nullptr;
  HYB_CUDA(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&S), words * sizeof(uint64_t), handle->mempool, stream));
  if (!S) return nullptr;
  launch_limbs_to_slices(stream, panels, order, ranks, count, C, S);
  ncclResult_t r = ncclAllReduce(S, S, words, ncclUint64, ncclSum, handle->ncclComm, stream);
  if (r != ncclSuccess) std::fprintf(stderr, "hyacin-b200: ncclAllReduce failed: %s\n", ncclGetErrorString(r));
  if (handle->logger) std::fprintf(static_cast<FILE*>(handle->logger), "NCCL-AllReduce [Bytes=%llu]\n", (unsigned long long)(words * sizeof(uint64_t)));
  if (ranks_out) *ranks_out = ranks;
  return S;
}
}  // namespace hyb

extern "C" void hyacinAllReduce1Drow(const hyacinHandle_t* handle, int32_t Complex, int32_t orderA, uint64_t N, uint64_t* A) {
  if (Complex <= 0 || orderA <= 0 || orderA > 3 || N == 0 || handle->ncclComm == nullptr) return;
  int ranks = 0;
  if (ncclCommCount(handle->ncclComm, &ranks) != ncclSuccess || ranks <= 1) return;
  hyb::timer_mark(handle, hyb::Segment::Comm);
  cudaStream_t stream = handle->cudaStream;
  const int slices = hyb::slice_count(orderA, ranks);
  const uint64_t words = uint64_t(Complex) * uint64_t(slices) * N;
  uint64_t* S = nullptr;
  HYB_CUDA(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&S), words * sizeof(uint64_t), handle->mempool, stream));
  if (!S) return;
  hyb::launch_limbs_to_slices(stream, Complex, orderA, ranks, N, A, S);
  ncclResult_t r = ncclAllReduce(S, S, words, ncclUint64, ncclSum, handle->ncclComm, stream);
  if (r != ncclSuccess) std::fprintf(stderr, "hyacin-b200: ncclAllReduce failed: %s\n", ncclGetErrorString(r));
  hyb::launch_slices_to_limbs(stream, Complex, orderA, ranks, N, S, A);
  HYB_CUDA(cudaFreeAsync(S, stream));
  if (handle->logger) std::fprintf(static_cast<FILE*>(handle->logger), "NCCL-AllReduce [Bytes=%llu]\n", (unsigned long long)(words * sizeof(uint64_t)));
}

extern "C" void hyacinAllReduceVExp(const hyacinHandle_t* handle, uint64_t N, int32_t* vexp) {
  if (N == 0 || handle->ncclComm == nullptr) return;
  int ranks = 0;
  if (ncclCommCount(handle->ncclComm, &ranks) != ncclSuccess || ranks <= 1) return;
  hyb::timer_mark(handle, hyb::Segment::Comm);
  ncclResult_t r = ncclAllReduce(vexp, vexp, N, ncclInt32, ncclMin, handle->ncclComm, handle->cudaStream);
  if (r != ncclSuccess) std::fprintf(stderr, "hyacin-b200: ncclAllReduce failed: %s\n", ncclGetErrorString(r));
  if (handle->logger) std::fprintf(static_cast<FILE*>(handle->logger), "NCCL-AllReduce [Bytes=%llu]\n", (unsigned long long)(N * sizeof(int32_t)));
}

#endif
