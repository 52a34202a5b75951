// Handle life cycle, segment timer and error reporting.
//
// Behaviour mirrors the reference's src/utils.cpp: hyacinCreate (:56-90) fills the tuning fields from the
// environment and creates only the resources whose fields are still zero, recording ownership in
// HandleOwnedResource; hyacinDestroy (:92-101) synchronises the device, frees owned resources and zeroes the
// handle; the timer (:39-43, 103-141) records a CUDA event whenever the class of work changes and
// hyacinSync_TimerSegments reports the milliseconds per class.
#include "hyb_internal.h"
#include <hyacin_b200.h>
#include <atomic>
#include <mutex>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

namespace hyb {

void report_cuda_error(cudaError_t err, const char* what, const char* file, int line) {
  std::fprintf(stderr, "hyacin-b200: CUDA error %d (%s) from %s at %s:%d\n", int(err), cudaGetErrorString(err), what, file, line);
}

namespace {
constexpr uint32_t kOwnsCublas = 0x1, kOwnsCusolver = 0x2, kOwnsMempool = 0x4, kOwnsPinned = 0x8, kOwnsTimer = 0x10;

struct SegmentTimer {
  // events[i].first is the class of the work enqueued BEFORE events[i].second was recorded
  std::vector<std::pair<Segment, cudaEvent_t>> events;
  Segment current = Segment::Untimed;
};

const char* env(const char* key) { return std::getenv(key); }
bool env_true(const char* key) { const char* v = env(key); return v && (!std::strcmp(v, "1") || !std::strcmp(v, "true") || !std::strcmp(v, "True")); }
}  // namespace

// ---- launch counter and optional per-kernel event profile ---------------------------------------------
namespace {
struct ProfileEntry { cudaEvent_t start, stop; KernelKind kind; };
std::atomic<long long> g_launches{0};
std::atomic<int> g_profile_on{0};
std::mutex g_profile_mutex;
std::vector<ProfileEntry> g_profile;
double g_tail_ms[2] = {0., 0.}; int g_tail_n[2] = {0, 0};      // Cholesky / SVD totals carried between the two read calls
}  // namespace

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

ProfileScope::ProfileScope(cudaStream_t s, KernelKind kind) : stream(s), slot(-1) {
  if (!g_profile_on.load(std::memory_order_relaxed)) return;
  ProfileEntry e; e.kind = kind;
  if (cudaEventCreate(&e.start) != cudaSuccess || cudaEventCreate(&e.stop) != cudaSuccess) return;
  cudaEventRecord(e.start, stream);
  std::lock_guard<std::mutex> lock(g_profile_mutex);
  g_profile.push_back(e); slot = int(g_profile.size()) - 1;
}
ProfileScope::~ProfileScope() {
  if (slot < 0) return;
  std::lock_guard<std::mutex> lock(g_profile_mutex);
  cudaEventRecord(g_profile[slot].stop, stream);
}

void timer_mark(const hyacinHandle_t* handle, Segment seg) {
  auto* t = static_cast<SegmentTimer*>(handle->timer);
  if (!t || t->current == seg) return;
  cudaEvent_t e; if (cudaEventCreate(&e) != cudaSuccess) return;
  HYB_CUDA(cudaEventRecord(e, handle->cudaStream));
  t->events.emplace_back(t->current, e); t->current = seg;
}

}  // namespace hyb

using namespace hyb;

extern "C" void hyacinCreate(hyacinHandle_t* handle) {
  HYB_CUDA(cudaGetDevice(&handle->DeviceID));
  int major = 0, minor = 0;
  HYB_CUDA(cudaDeviceGetAttribute(&handle->DeviceSMs, cudaDevAttrMultiProcessorCount, handle->DeviceID));
  HYB_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, handle->DeviceID));
  HYB_CUDA(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, handle->DeviceID));
  const int cc = 10 * major + minor;     // GPUs with full-rate FP64: sm_80, sm_90, sm_100, sm_107
  handle->DeviceIsF64Capable = (cc == 80 || cc == 90 || cc == 100 || cc == 107) ? 1 : 0;

  const char* v;
  handle->GramMatrixAlgorithm = (v = env("HYACIN_GRAM_ALGORITHM")) && v[0] ? v[0] : 'A';
  handle->StrideBatchPerfPenalty = (v = env("HYACIN_STRIDE_BATCH_PERF_PENALTY")) ? std::atof(v) : 1.3;
  handle->GramSegmentK = (v = env("HYACIN_GRAM_SEGMENT_K")) ? std::atoi(v) : 8192;
  handle->TCGemmTargetK = (v = env("HYACIN_TCGEMM_TARGET_K")) ? std::atoi(v) : 8192;
  handle->QuantizeBitCorrection = (v = env("HYACIN_QUANTIZE_BITS_CORR")) ? std::atoi(v) : 7;
  handle->QRCPTruncateRank = (v = env("HYACIN_QRCP_TRUNCATE_RANK")) ? std::atoi(v) : 1;
  handle->JacobiSVDSweeps = (v = env("HYACIN_JACOBI_SVD_SWEEPS")) ? std::atoi(v) : 3;

  if (!handle->cublasHandle) {
    if (cublasCreate(&handle->cublasHandle) == CUBLAS_STATUS_SUCCESS) {
      cublasSetStream(handle->cublasHandle, handle->cudaStream); handle->HandleOwnedResource |= kOwnsCublas;
    } else std::fprintf(stderr, "hyacin-b200: cublasCreate failed\n");
  }
  if (!handle->cusolverHandle) {
    if (cusolverDnCreate(&handle->cusolverHandle) == CUSOLVER_STATUS_SUCCESS) {
      cusolverDnSetStream(handle->cusolverHandle, handle->cudaStream); handle->HandleOwnedResource |= kOwnsCusolver;
    } else std::fprintf(stderr, "hyacin-b200: cusolverDnCreate failed\n");
  }
  if (!handle->mempool) {
    cudaMemPoolProps props{};
    props.allocType = cudaMemAllocationTypePinned; props.location.type = cudaMemLocationTypeDevice; props.location.id = handle->DeviceID;
    HYB_CUDA(cudaMemPoolCreate(&handle->mempool, &props));
    uint64_t keep = ~uint64_t(0);      // never hand memory back to the driver between fits
    HYB_CUDA(cudaMemPoolSetAttribute(handle->mempool, cudaMemPoolAttrReleaseThreshold, &keep));
    handle->HandleOwnedResource |= kOwnsMempool;
  }
  if (!handle->pinnedWorkspace) {
    HYB_CUDA(cudaMallocHost(&handle->pinnedWorkspace, sizeof(int32_t)));
    handle->HandleOwnedResource |= kOwnsPinned;
  }
  if (env_true("HYACIN_CREATE_TIMER") && !handle->timer) { handle->timer = new SegmentTimer(); handle->HandleOwnedResource |= kOwnsTimer; }
  if (env_true("HYACIN_VERBOSE") && !handle->logger) handle->logger = stdout;
  status_word_device(handle->DeviceID);      // allocate the status word up front, outside any timed region
}

extern "C" void hyacinDestroy(hyacinHandle_t* handle) {
  HYB_CUDA(cudaDeviceSynchronize());
  status_check(handle, "hyacinDestroy");
  const uint32_t own = handle->HandleOwnedResource;
  if ((own & kOwnsCublas) && handle->cublasHandle) cublasDestroy(handle->cublasHandle);
  if ((own & kOwnsCusolver) && handle->cusolverHandle) cusolverDnDestroy(handle->cusolverHandle);
  if ((own & kOwnsMempool) && handle->mempool) HYB_CUDA(cudaMemPoolDestroy(handle->mempool));
  if ((own & kOwnsPinned) && handle->pinnedWorkspace) HYB_CUDA(cudaFreeHost(handle->pinnedWorkspace));
  if ((own & kOwnsTimer) && handle->timer) {
    auto* t = static_cast<SegmentTimer*>(handle->timer);
    for (auto& ev : t->events) cudaEventDestroy(ev.second);
    delete t;
  }
  std::memset(handle, 0, sizeof(hyacinHandle_t));
}

extern "C" void hyacinSync_TimerSegments(const hyacinHandle_t* handle, double* eventMs, int32_t lenMs) {
  auto* t = static_cast<SegmentTimer*>(handle->timer);
  if (!t) { HYB_CUDA(cudaStreamSynchronize(handle->cudaStream)); status_check(handle, "hyacinSync_TimerSegments"); return; }
  cudaEvent_t last; HYB_CUDA(cudaEventCreate(&last));
  HYB_CUDA(cudaEventRecord(last, handle->cudaStream));
  HYB_CUDA(cudaEventSynchronize(last));
  status_check(handle, "hyacinSync_TimerSegments");
  t->events.emplace_back(t->current, last);
  if (eventMs && lenMs > 0) {
    double d = 0., r = 0., c = 0.;
    for (size_t i = 1; i < t->events.size(); ++i) {
      float ms = 0.f; cudaEventElapsedTime(&ms, t->events[i - 1].second, t->events[i].second);
      switch (t->events[i].first) {
        case Segment::Distributed: d += ms; break;
        case Segment::Replicated: r += ms; break;
        case Segment::Comm: c += ms; break;
        default: break;
      }
    }
    for (int i = 0; i < lenMs; ++i) {
      const char q = static_cast<char>(eventMs[i]);
      eventMs[i] = (q == 'D' || q == 'd') ? d : (q == 'R' || q == 'r') ? r : (q == 'C' || q == 'c') ? c : 0.;
    }
  }
  for (auto& ev : t->events) cudaEventDestroy(ev.second);
  t->events.clear(); t->current = Segment::Untimed;
}

// ---- B200-only accounting entry points ------------------------------------------------------------------
extern "C" int64_t hyacinB200LaunchCount(int32_t reset) {
  return reset ? g_launches.exchange(0) : g_launches.load();
}

extern "C" void hyacinB200ProfileEnable(int32_t enable) {
  std::lock_guard<std::mutex> lock(g_profile_mutex);
  for (auto& e : g_profile) { cudaEventDestroy(e.start); cudaEventDestroy(e.stop); }
  g_profile.clear();
  g_tail_ms[0] = g_tail_ms[1] = 0.; g_tail_n[0] = g_tail_n[1] = 0;
  g_profile_on.store(enable ? 1 : 0);
}

namespace {
void profile_collect(double* ms, int* n) {
  std::lock_guard<std::mutex> lock(g_profile_mutex);
  for (int i = 0; i < int(KernelKind::Count); ++i) { ms[i] = 0.; n[i] = 0; }
  for (auto& e : g_profile) {
    float t = 0.f;
    if (cudaEventSynchronize(e.stop) == cudaSuccess && cudaEventElapsedTime(&t, e.start, e.stop) == cudaSuccess) { ms[int(e.kind)] += t; n[int(e.kind)] += 1; }
    cudaEventDestroy(e.start); cudaEventDestroy(e.stop);
  }
  g_profile.clear();
}
}  // namespace

extern "C" void hyacinB200ProfileRead(double* gramMs, int32_t* gramLaunches, double* quantizeMs, int32_t* quantizeLaunches) {
  double ms[int(KernelKind::Count)]; int n[int(KernelKind::Count)];
  profile_collect(ms, n);
  if (gramMs) *gramMs = ms[int(KernelKind::Gram)]; if (gramLaunches) *gramLaunches = n[int(KernelKind::Gram)];
  if (quantizeMs) *quantizeMs = ms[int(KernelKind::Quantize)]; if (quantizeLaunches) *quantizeLaunches = n[int(KernelKind::Quantize)];
  g_tail_ms[0] += ms[int(KernelKind::Cholesky)]; g_tail_n[0] += n[int(KernelKind::Cholesky)];
  g_tail_ms[1] += ms[int(KernelKind::Svd)]; g_tail_n[1] += n[int(KernelKind::Svd)];
}

extern "C" void hyacinB200ProfileReadTail(double* choleskyMs, int32_t* choleskyLaunches, double* svdMs, int32_t* svdCalls) {
  double ms[int(KernelKind::Count)]; int n[int(KernelKind::Count)];
  profile_collect(ms, n);
  g_tail_ms[0] += ms[int(KernelKind::Cholesky)]; g_tail_n[0] += n[int(KernelKind::Cholesky)];
  g_tail_ms[1] += ms[int(KernelKind::Svd)]; g_tail_n[1] += n[int(KernelKind::Svd)];
  if (choleskyMs) *choleskyMs = g_tail_ms[0]; if (choleskyLaunches) *choleskyLaunches = g_tail_n[0];
  if (svdMs) *svdMs = g_tail_ms[1]; if (svdCalls) *svdCalls = g_tail_n[1];
  g_tail_ms[0] = g_tail_ms[1] = 0.; g_tail_n[0] = g_tail_n[1] = 0;
}
