// hyacinB200HerkBatchStatic: the integer Gram of hyacinXherkBatch without a single allocation.
//
// Who needs this.  hyacinXherkBatch takes its int8 residue planes and residue accumulators from the handle's
// stream-ordered memory pool.  Some hosts of this library cannot let it do that: a solver that reserved the
// whole device for its own arena at start-up (the pool then has nothing left to grow into and the call fails
// in the middle of a factorisation), or a service that updates many small Gram matrices inside a
// latency-bound loop where an allocator call -- and the device synchronisation a growing pool can imply --
// is not acceptable.  For such callers this entry point keeps all of its scratch in a fixed array that is part
// of the loaded module.
//
// The limit.  The array holds kStaticScratchBytes (64 MiB) on every GPU that loads this library, from the
// moment the module is loaded until the process exits.  A call needs
//     256 B (reserved) + residues: moduli x tiles(N) x 32 KiB (x2 for complex input)
//                         + one row chunk of int8 planes: chunk x N x moduli (x3 for complex), chunk >= 128
// and is refused (return value -2, message on stderr) when that does not fit; N up to about 2000 fits for
// FP64 inputs at eps = 1e-10.  Larger problems must use hyacinXherkBatch.
//
// Rules of use.  The first call on a device looks up the device address of the array (cudaGetSymbolAddress),
// and with CUDA's default lazy module loading that lookup is also what makes the driver load this module and
// reserve the 64 MiB.  A host whose arena is about to take the rest of the device must therefore make one call
// BEFORE it does so (or run with CUDA_MODULE_LOADING=EAGER): a call with zero rows is enough, it binds the array
// and returns 0 without launching anything.  Make that first call outside any stream capture.
// The handle must come from hyacinCreate on the device that is current at the call (the status word of the
// bounded waits is set up there); any other combination is refused with -1 / -3 rather than run on the wrong GPU.
// All calls on a device share the array and it keeps whatever the previous call left in it: everything a call
// reads is written by that call first (padding rows are zero-filled by the quantiser, residues start in overwrite
// mode), so stale contents never matter -- but two calls whose kernels overlap on the GPU (different streams or
// handles on the same device) would race on it; issue them on one stream or order them with events.
// Complex input always takes the three-part schedule here (planes re, im, -re); handle->GramMatrixAlgorithm is
// not consulted.  Results are identical to hyacinXherkBatch: only the schedule differs and the integer Gram is exact.
#include "hyb_internal.h"
#include <hyacin_b200.h>
#include <algorithm>
#include <atomic>

namespace hyb {
namespace {

constexpr size_t kStaticScratchBytes = size_t(64) << 20;
constexpr size_t kStatusBytes = 256;
constexpr int kMaxDevices = 64;

// The scratch itself.  In host code this name is only a handle for the runtime's symbol lookup, never an
// address a kernel could use; device_scratch() below obtains the real device address.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

std::atomic<unsigned char*> g_scratch_addr[kMaxDevices];

// Once per device, with that device current.  Two host threads that make their first call together both look
// the address up and store the same value.
unsigned char* device_scratch(int device) {
  if (device < 0 || device >= kMaxDevices) return nullptr;
  unsigned char* known = g_scratch_addr[device].load(std::memory_order_acquire);
  if (known) return known;
  void* ptr = nullptr;
  const cudaError_t err = cudaGetSymbolAddress(&ptr, g_static_scratch);
  if (err != cudaSuccess || ptr == nullptr) {
    std::fprintf(stderr, "hyacin-b200: cudaGetSymbolAddress for the static scratch failed: %s\n", cudaGetErrorString(err));
    return nullptr;
  }
  g_scratch_addr[device].store(static_cast<unsigned char*>(ptr), std::memory_order_release);
  return static_cast<unsigned char*>(ptr);
}

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace
}  // namespace hyb

extern "C" int32_t hyacinB200HerkBatchStatic(const hyacinHandle_t* handle, int32_t batches, int32_t segM, int32_t lastM, int32_t N,
                                             hyacinPrecision_t Atype, const void* A, int32_t lda, int32_t u, const int32_t* vexp,
                                             int32_t beta, int32_t orderC, uint64_t* C) {
  using namespace hyb;
  if (N <= 0 || orderC <= 0 || orderC > 3 || int(Atype) < 0 || int(Atype) > int(HYACIN_F16_COMPLEX)) return -1;
  cudaStream_t stream = handle->cudaStream;
  const int64_t rows = batches <= 1 ? int64_t(lastM) : int64_t(batches - 1) * segM + lastM;
  const int cplx = is_complex(Atype), parts = cplx ? 3 : 1;
  const int64_t tri = (int64_t(N) * N + N) / 2;
  // bind the array first, so that a call without rows serves as the warm-up that reserves it
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess) return -3;
  if (device != handle->DeviceID) {
    std::fprintf(stderr, "hyacin-b200: hyacinB200HerkBatchStatic: the handle belongs to device %d but device %d is current\n", handle->DeviceID, device);
    return -1;
  }
  unsigned char* scratch = device_scratch(device);
  if (!scratch) return -3;
  // expired waits are reported through the status word that hyacinCreate set up on this device (hyacinB200Status)
  uint32_t* status = status_word_if_ready(device);
  if (!status) {
    std::fprintf(stderr, "hyacin-b200: hyacinB200HerkBatchStatic: no status word on device %d (the handle was not made by hyacinCreate there)\n", device);
    return -3;
  }
  if (rows <= 0 || u < 0) {
    if (beta == 0 && C) HYB_CUDA(cudaMemsetAsync(C, 0, size_t(tri) * orderC * (1 + cplx) * sizeof(uint64_t), stream));
    return 0;
  }
  const CrtPlan plan = make_crt_plan(u, cplx, rows, false);
  if (plan.moduli == 0) return -1;
  const TilePlan tp = make_tile_plan(N);
  const size_t r_bytes = round_up(size_t(plan.moduli) * tp.num_tiles * size_t(kTileY) * kTileX, 256);
  const size_t fixed = kStatusBytes + r_bytes * (cplx ? 2 : 1);
  const size_t per_row = size_t(N) * plan.moduli * parts;
  int64_t chunk = fixed < kStaticScratchBytes ? int64_t((kStaticScratchBytes - fixed) / per_row) / kStageK * kStageK : 0;
  chunk = std::min<int64_t>(chunk, plan.chunk_rows);
  if (chunk < kStageK) {
    std::fprintf(stderr, "hyacin-b200: hyacinB200HerkBatchStatic: N = %d with %d moduli needs %zu bytes of residues plus %zu bytes per "
                         "128-row chunk, more than the %zu-byte static scratch; use hyacinXherkBatch\n",
                 N, plan.moduli, fixed, per_row * kStageK, kStaticScratchBytes);
    return -2;
  }
  timer_mark(handle, Segment::Distributed);
  uint8_t* R = scratch + kStatusBytes;
  int8_t* W = reinterpret_cast<int8_t*>(scratch + fixed);
  const size_t elem = (base_type(Atype) == HYACIN_F64 ? 8 : base_type(Atype) == HYACIN_F32 ? 4 : 2) * size_t(cplx ? 2 : 1);
  int accumulate_c = beta ? 1 : 0;
  for (int64_t row = 0; row < rows; row += plan.group_rows) {
    const int64_t g = std::min<int64_t>(plan.group_rows, rows - row);
    bool first = true;
    for (int64_t c0 = 0; c0 < g; c0 += chunk) {
      const int rc = int(std::min<int64_t>(chunk, g - c0));
      const int64_t ldk = (rc + kStageK - 1) / kStageK * kStageK;
      const char* src = static_cast<const char*>(A) + size_t(row + c0) * elem;
      launch_quantize_crt(stream, Atype, rc, N, src, lda, vexp, plan, W, ldk);
      GramLaunch gl{};
      gl.w = W; gl.ldw = ldk * parts; gl.plane_stride = gl.ldw * N;
      gl.ka0 = 0; gl.kb0 = 0; gl.k_rows = int(ldk) * (cplx ? 2 : 1); gl.n = N; gl.moduli = plan.moduli;
      gl.accumulate = first ? 0 : 1; gl.sm_count = handle->DeviceSMs; gl.residues = R; gl.status = status;
      launch_gram_residues(stream, gl);
      if (cplx) { gl.kb0 = int(ldk); gl.residues = R + r_bytes; launch_gram_residues(stream, gl); }
      first = false;
    }
    launch_reconstruct(stream, N, plan.moduli, R, accumulate_c, orderC, C);
    if (cplx) launch_reconstruct(stream, N, plan.moduli, R + r_bytes, accumulate_c, orderC, C + size_t(orderC) * tri);
    accumulate_c = 1;
  }
  return 0;
}
