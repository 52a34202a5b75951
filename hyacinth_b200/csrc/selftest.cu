// Self-test of the bounded waits: the path every kernel of this library takes when an mbarrier never completes.
//
// The product kernels (residue Gram, pivoted Cholesky) wait on mbarriers with a poll limit; when the limit runs
// out the waiting thread raises a flag for the other roles of its block, stores a code in the status word (mapped
// host memory, read by hyacinB200Status) and returns, so the context stays usable.  Nothing in a healthy run ever
// reaches that path.  This kernel reaches it on purpose and harmlessly: it initialises a barrier that nobody
// arrives at, waits on it with a small limit, and leaves.  No copy is in flight, no tensor memory is held.
#include "hyb_internal.h"
#include "ptx_sm100.cuh"
#include <hyacin_b200.h>

namespace hyb {
namespace {
__global__ void wait_expiry_kernel(uint32_t limit, uint32_t code, uint32_t* status, uint32_t* observed) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    ptx::mbar_init(&bar, 1); abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  bool ok = true;
  if (threadIdx.x == 0) ok = ptx::mbar_wait(&bar, 0u, &abort_flag, status, code, limit);       // expires
  __syncthreads();
  // a second role that polls after the first gave up leaves at once through the flag
  if (threadIdx.x == 32) ok = ptx::mbar_wait(&bar, 0u, &abort_flag, status, code + 1000u, ptx::kSpinLimit);
  __syncthreads();
  if (threadIdx.x == 0) observed[0] = ok ? 0u : 1u;
  if (threadIdx.x == 32) observed[1] = ok ? 0u : 1u;
}
}  // namespace
}  // namespace hyb

extern "C" int32_t hyacinB200SelfTestWait(const hyacinHandle_t* handle, uint32_t pollLimit, uint32_t code) {
  using namespace hyb;
  if (pollLimit == 0 || pollLimit > (1u << 16) || code == 0) return -1;
  uint32_t* status = status_word_device(handle->DeviceID);
  uint32_t* observed = nullptr;
  HYB_CUDA(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&observed), 2 * sizeof(uint32_t), handle->mempool, handle->cudaStream));
  HYB_CUDA(cudaMemsetAsync(observed, 0xff, 2 * sizeof(uint32_t), handle->cudaStream));
  count_launch();
  wait_expiry_kernel<<<1, 64, 0, handle->cudaStream>>>(pollLimit, code, status, observed);
  HYB_CUDA(cudaGetLastError());
  uint32_t host[2] = {7u, 7u};
  HYB_CUDA(cudaMemcpyAsync(host, observed, sizeof(host), cudaMemcpyDeviceToHost, handle->cudaStream));
  HYB_CUDA(cudaFreeAsync(observed, handle->cudaStream));
  HYB_CUDA(cudaStreamSynchronize(handle->cudaStream));
  return (host[0] == 1u && host[1] == 1u) ? 0 : -2;       // both roles must have returned "gave up"
}
