// Truncated pivoted Cholesky of the Gram matrix: G(perm, perm) ~= R^H R, R upper trapezoidal with `rank` rows.
//
// Downstream of the quantized Gram and replicated on every rank; kept behaviourally equal to the reference's
// src/hyacin_potrfp.cu: diagonal pivoting on the largest remaining diagonal entry (:214-272), stop as soon
// as the remaining trace drops to eps^2 times the initial trace (:262) or the rank cap is reached, arithmetic
// in the Gram's own format (float, double or double-double; helpers as in include/internal.hpp:181-227).
//
// The organisation is different.  The reference swaps rows and columns of G in place and computes each new
// row with one block-wide reduction per column and two or three grid barriers per step.  Here the factor is
// written to a separate row-major array R[k][i] indexed by ORIGINAL column i (no swaps; the permutation is
// only recorded), a warp owns 32 consecutive columns so that every load of a previous row is one contiguous
// run, the sum over previous rows is split across the warps of a block and combined in a fixed order, and a
// step costs ONE grid barrier: every block re-reduces the per-block (max, argmax, trace) partials itself.
#include "hyb_internal.h"
#include "tail.h"
#include "ptx_sm100.cuh"
#include <mutex>
#include <cooperative_groups.h>
#include <cfloat>

namespace cg = cooperative_groups;

namespace hyb {
namespace {

// ---- scalar policies ------------------------------------------------------------------------------------
struct DD { double x, y; };

__device__ __forceinline__ DD dd_renorm(double a, double b) { double s = a + b, d = a - s; return DD{s, b + d}; }
__device__ __forceinline__ DD dd_mul(DD a, DD b) { double p = a.x * b.x; return dd_renorm(p, fma(a.x, b.y, a.y * b.x) + fma(a.x, b.x, -p)); }
__device__ __forceinline__ DD dd_sqr(DD a) { double p = a.x * a.x; return dd_renorm(p, fma(a.x + a.x, a.y, fma(a.x, a.x, -p))); }
__device__ __forceinline__ DD dd_add(DD a, DD b) {
  double s = a.x + b.x, d = a.x - s, sd = s + d, e = (b.x + d) + (a.x - sd); return dd_renorm(s, (a.y + b.y) + e);
}
__device__ __forceinline__ DD dd_sub(DD a, DD b) {
  double nb = -b.x, s = a.x + nb, d = a.x - s, sd = s + d, e = (nb + d) + (a.x - sd); return dd_renorm(s, (a.y - b.y) + e);
}

template <typename R> struct Real;
template <> struct Real<float> {
  static __device__ __forceinline__ float zero() { return 0.f; }
  static __device__ __forceinline__ float mul(float a, float b) { return a * b; }
  static __device__ __forceinline__ float add(float a, float b) { return a + b; }
  static __device__ __forceinline__ float sub(float a, float b) { return a - b; }
  static __device__ __forceinline__ float neg(float a) { return -a; }
  static __device__ __forceinline__ float fnma(float a, float b, float c) { return fmaf(-a, b, c); }      // c - a b
  static __device__ __forceinline__ bool less(float a, float b) { return a < b; }
  static __device__ __forceinline__ double to_double(float a) { return double(a); }
  static __device__ __forceinline__ float rsqrt(float a) { return 1.f / sqrtf(a); }
};
template <> struct Real<double> {
  static __device__ __forceinline__ double zero() { return 0.; }
  static __device__ __forceinline__ double mul(double a, double b) { return a * b; }
  static __device__ __forceinline__ double add(double a, double b) { return a + b; }
  static __device__ __forceinline__ double sub(double a, double b) { return a - b; }
  static __device__ __forceinline__ double neg(double a) { return -a; }
  static __device__ __forceinline__ double fnma(double a, double b, double c) { return fma(-a, b, c); }
  static __device__ __forceinline__ bool less(double a, double b) { return a < b; }
  static __device__ __forceinline__ double to_double(double a) { return a; }
  static __device__ __forceinline__ double rsqrt(double a) { return 1. / sqrt(a); }
};
template <> struct Real<DD> {
  static __device__ __forceinline__ DD zero() { return DD{0., 0.}; }
  static __device__ __forceinline__ DD mul(DD a, DD b) { return dd_mul(a, b); }
  static __device__ __forceinline__ DD add(DD a, DD b) { return dd_add(a, b); }
  static __device__ __forceinline__ DD sub(DD a, DD b) { return dd_sub(a, b); }
  static __device__ __forceinline__ DD neg(DD a) { return DD{-a.x, -a.y}; }
  static __device__ __forceinline__ DD fnma(DD a, DD b, DD c) { return dd_sub(c, dd_mul(a, b)); }
  static __device__ __forceinline__ bool less(DD a, DD b) { return a.x < b.x || (a.x == b.x && a.y < b.y); }
  static __device__ __forceinline__ double to_double(DD a) { return a.x; }
  // 1/sqrt(a) to double-double accuracy: two Newton steps y <- y (3/2 - a y^2 / 2) from the double estimate.
  static __device__ __forceinline__ DD rsqrt(DD a) {
    DD y{1. / sqrt(a.x), 0.}; const DD half_a{0.5 * a.x, 0.5 * a.y};
#pragma unroll
    for (int it = 0; it < 2; ++it) y = dd_mul(y, dd_sub(DD{1.5, 0.}, dd_mul(half_a, dd_sqr(y))));
    return y;
  }
};

template <typename R, bool CPLX> struct Elem { R re; };
template <typename R> struct Elem<R, true> { R re, im; };

template <typename R, bool CPLX> struct Ops {
  using E = Elem<R, CPLX>; using T = Real<R>;
  static __device__ __forceinline__ E zero() { E z; z.re = T::zero(); if constexpr (CPLX) z.im = T::zero(); return z; }
  static __device__ __forceinline__ E conj(E a) { if constexpr (CPLX) a.im = T::neg(a.im); return a; }
  // acc - conj(a) * b
  static __device__ __forceinline__ E sub_conj_mul(E acc, E a, E b) {
    if constexpr (CPLX) {
      // conj(a) b = (ar br + ai bi) + i (ar bi - ai br)
      acc.re = T::fnma(a.re, b.re, acc.re); acc.re = T::fnma(a.im, b.im, acc.re);
      acc.im = T::fnma(a.re, b.im, acc.im); acc.im = T::add(acc.im, T::mul(a.im, b.re));
    } else acc.re = T::fnma(a.re, b.re, acc.re);
    return acc;
  }
  static __device__ __forceinline__ E add(E a, E b) { a.re = T::add(a.re, b.re); if constexpr (CPLX) a.im = T::add(a.im, b.im); return a; }
  static __device__ __forceinline__ E scale(E a, R s) { a.re = T::mul(a.re, s); if constexpr (CPLX) a.im = T::mul(a.im, s); return a; }
  static __device__ __forceinline__ R abs2(E a) { R v = T::mul(a.re, a.re); if constexpr (CPLX) v = T::add(v, T::mul(a.im, a.im)); return v; }
};

constexpr int kBlock = 512;               // 16 warps: 32 columns per block, previous rows split 16 ways
constexpr int kWarps = kBlock / 32;

template <typename R, bool CPLX>
struct Partial { R val; double trace; int idx; int pad; };

// jpiv (1-based) is kept as a permutation that is updated by swapping the chosen column into position k, which
// is the bookkeeping of the reference (src/hyacin_potrfp.cu:243-246), so the whole array -- not only its first
// `rank` entries -- comes out the same.  pos[i] is the inverse map: column i is still free while pos[i] >= k.
// TMA = true: the previous rows of the factor reach the SM through a ring of shared-memory stages filled by TMA
// tile loads (32 columns x kRowsPerStage rows, no multicast) that one thread keeps several stages ahead of the
// consumers; the whole pivot column is gathered into shared memory once per step.  The step is bound by the
// latency of these reads, and the ring keeps ~100 KiB in flight per SM where plain loads kept a few KiB.
// TMA = false: plain loads (used when the row pitch of the factor is not a multiple of 16 bytes).
constexpr int kStageBytes = 32768;
template <typename R, bool CPLX, bool TMA>
__global__ void __launch_bounds__(kBlock)
potrfp_kernel(double eps_sq, int n, int cap, const Elem<R, CPLX>* __restrict__ G, int64_t ldg, Elem<R, CPLX>* __restrict__ Rw,
              R* __restrict__ D, int* __restrict__ pos, int32_t* __restrict__ jpiv, Partial<R, CPLX>* __restrict__ partials,
              int32_t* __restrict__ rank_out, int ring_stages, const __grid_constant__ CUtensorMap tmap) {
  using E = Elem<R, CPLX>; using O = Ops<R, CPLX>; using T = Real<R>; using P = Partial<R, CPLX>;
  cg::grid_group grid = cg::this_grid();
  constexpr int kChunk = TMA ? 1 : (sizeof(E) >= 32 ? 512 : 1024);   // previous rows staged per shared-memory pass (plain path)
  constexpr int kRowsPerStage = kStageBytes / (32 * int(sizeof(E)));
  __shared__ E s_pivot_row[kChunk];                 // conj-multiplier: previous rows at the pivot column
  extern __shared__ uint8_t dyn_smem[];             // TMA path: [ring stages][pivot column: cap entries][barriers]
  uint8_t* ring = dyn_smem + ((1024u - (ptx::smem_u32(dyn_smem) & 1023u)) & 1023u);
  E* piv_all = reinterpret_cast<E*>(ring + size_t(ring_stages) * kStageBytes);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(piv_all + (TMA ? cap : 0));
  uint64_t* empty_bar = full_bar + 8;
  __shared__ uint32_t s_abort, s_status;
  uint32_t issued = 0, consumed = 0;                // chunks issued (thread 0) / consumed (every warp) since kernel start
  bool dead = false;                                // a bounded wait expired in this thread
  if constexpr (TMA) {
    if (threadIdx.x == 0) {
      for (int s = 0; s < ring_stages; ++s) { ptx::mbar_init(&full_bar[s], 1); ptx::mbar_init(&empty_bar[s], kWarps); }
      s_abort = 0;
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
  }
  __shared__ E s_partial[kWarps][32];
  __shared__ P s_red[kWarps];
  __shared__ P s_best;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblocks = gridDim.x;

  // ---- step "-1": diagonal, initial partials ----
  {
    P mine; mine.val = T::zero(); mine.trace = 0.; mine.idx = -1; mine.pad = 0;
    for (int i = blockIdx.x * kBlock + threadIdx.x; i < n; i += nblocks * kBlock) {
      const R d = G[i + int64_t(i) * ldg].re;
      D[i] = d; pos[i] = i; jpiv[i] = i + 1;
      mine.trace += T::to_double(d);
      if (mine.idx < 0 || T::less(mine.val, d)) { mine.val = d; mine.idx = i; }
    }
    // block reduce (fixed order: lane tree then warp 0 over warps)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      P other; other.trace = __shfl_down_sync(0xffffffffu, mine.trace, o); other.idx = __shfl_down_sync(0xffffffffu, mine.idx, o);
      if constexpr (sizeof(R) == 16) { other.val.x = __shfl_down_sync(0xffffffffu, mine.val.x, o); other.val.y = __shfl_down_sync(0xffffffffu, mine.val.y, o); }
      else other.val = __shfl_down_sync(0xffffffffu, mine.val, o);
      mine.trace += other.trace;
      if (other.idx >= 0 && (mine.idx < 0 || T::less(mine.val, other.val))) { mine.val = other.val; mine.idx = other.idx; }
    }
    if (lane == 0) s_red[warp] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
      P acc = s_red[0];
      for (int w = 1; w < kWarps; ++w) { acc.trace += s_red[w].trace; if (s_red[w].idx >= 0 && (acc.idx < 0 || T::less(acc.val, s_red[w].val))) { acc.val = s_red[w].val; acc.idx = s_red[w].idx; } }
      partials[blockIdx.x] = acc;
    }
  }
  grid.sync();

  double threshold = 0.;
  int k = 0;
  for (;; ++k) {
    // ---- every block reduces the partials of all blocks in the same order: same pivot everywhere ----
    const P* cur = partials + size_t(k & 1) * nblocks;
    {
      // all threads take part: thread b fetches the partial of block b (L2 loads, these words are rewritten by
      // other blocks every second step), then a fixed-shape tree reduces them -- same tree, same answer, in
      // every block
      P mine; mine.trace = 0.; mine.idx = -1; mine.val = T::zero(); mine.pad = 0;
      for (int b = threadIdx.x; b < nblocks; b += kBlock) {
        P o; o.trace = __ldcg(&cur[b].trace); o.idx = __ldcg(&cur[b].idx);
        if constexpr (sizeof(R) == 16) { o.val.x = __ldcg(&cur[b].val.x); o.val.y = __ldcg(&cur[b].val.y); } else o.val = __ldcg(&cur[b].val);
        mine.trace += o.trace; mine.pad |= __ldcg(&cur[b].pad);
        if (o.idx >= 0 && (mine.idx < 0 || T::less(mine.val, o.val))) { mine.val = o.val; mine.idx = o.idx; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        P other; other.trace = __shfl_down_sync(0xffffffffu, mine.trace, o); other.idx = __shfl_down_sync(0xffffffffu, mine.idx, o);
        if constexpr (sizeof(R) == 16) { other.val.x = __shfl_down_sync(0xffffffffu, mine.val.x, o); other.val.y = __shfl_down_sync(0xffffffffu, mine.val.y, o); }
        else other.val = __shfl_down_sync(0xffffffffu, mine.val, o);
        mine.trace += other.trace; mine.pad |= __shfl_down_sync(0xffffffffu, mine.pad, o);
        if (other.idx >= 0 && (mine.idx < 0 || T::less(mine.val, other.val))) { mine.val = other.val; mine.idx = other.idx; }
      }
      if (lane == 0) s_red[warp] = mine;
      __syncthreads();
      if (threadIdx.x == 0) {
        P acc = s_red[0];
        for (int w = 1; w < kWarps; ++w) { acc.trace += s_red[w].trace; acc.pad |= s_red[w].pad; if (s_red[w].idx >= 0 && (acc.idx < 0 || T::less(acc.val, s_red[w].val))) { acc.val = s_red[w].val; acc.idx = s_red[w].idx; } }
        s_best = acc;
      }
    }
    __syncthreads();
    const P best = s_best;
    // an expired wait anywhere travels through the partials, so that every block leaves at the same step
    if (best.pad) { k = -1; break; }
    if (k == 0) threshold = eps_sq * best.trace;
    // stop: nothing left, rank cap reached, remaining trace at or below the threshold, or a non-positive pivot
    bool stop = best.idx < 0 || k >= cap || (k > 0 && !(threshold < best.trace)) || !(T::to_double(best.val) > 0.);
    if (stop) break;
    const int p = best.idx;
    const R rinv = T::rsqrt(best.val);              // 1 / R[k][p]
    const R rkk = T::mul(best.val, rinv);           // sqrt(d) = d / sqrt(d)
    P mine; mine.val = T::zero(); mine.trace = 0.; mine.idx = -1; mine.pad = 0;
    if constexpr (TMA) {
      // rows 0..k-1 of the factor at the pivot column, once per step (no column group of the previous step is
      // still reading the old copy: the grid barrier that ended that step lies in between)
      for (int t = threadIdx.x; t < k; t += kBlock) piv_all[t] = Rw[size_t(t) * n + p];
      __syncthreads();
    }

    for (int c0 = blockIdx.x * 32; c0 < n; c0 += nblocks * 32) {
      const int i = c0 + lane;
      const bool live = i < n && i != p && __ldcg(&pos[i]) >= k;
      // kUnroll independent accumulators per thread and kUnroll row loads in flight before any is consumed: the
      // step is bound by the latency of these loads (the factor rows live in L2 / HBM), not by arithmetic
      constexpr int kUnroll = sizeof(E) >= 32 ? 4 : 8;
      E accs[kUnroll];
#pragma unroll
      for (int q = 0; q < kUnroll; ++q) accs[q] = O::zero();
      if constexpr (TMA) {
        // chunk c of this column group = factor rows [c * kRowsPerStage, ...) x columns [c0, c0 + 32), one TMA
        // tile (rows past the last written one hold stale data that is never read; columns past n read as zero)
        const int nchunks = (k + kRowsPerStage - 1) / kRowsPerStage;
        const int x0 = c0 * int(sizeof(E) / 4);                 // the tensor map counts 32-bit words
        auto issue = [&](int c) {
          const uint32_t slot = issued % uint32_t(ring_stages), round = issued / uint32_t(ring_stages);
          if (!dead && !ptx::mbar_wait(&empty_bar[slot], (round & 1u) ^ 1u, &s_abort, &s_status, 1u)) dead = true;
          if (!dead) {
            ptx::mbar_expect_tx(&full_bar[slot], kStageBytes);
            ptx::tma_load_2d(ptx::smem_u32(ring + size_t(slot) * kStageBytes), &tmap, &full_bar[slot], x0, c * kRowsPerStage);
          }
          ++issued;
        };
        if (threadIdx.x == 0)
          for (int c = 0; c < min(nchunks, ring_stages - 1); ++c) issue(c);
        for (int c = 0; c < nchunks; ++c) {
          // the slot that chunk c + stages - 1 goes to held chunk c - 1, which this warp released one turn ago:
          // the wait inside issue() only waits for the other warps to release it too
          if (threadIdx.x == 0 && c + ring_stages - 1 < nchunks) issue(c + ring_stages - 1);
          const uint32_t slot = consumed % uint32_t(ring_stages), round = consumed / uint32_t(ring_stages);
          if (!dead && !ptx::mbar_wait(&full_bar[slot], round & 1u, &s_abort, &s_status, 2u)) dead = true;
          const int r0 = c * kRowsPerStage, rows_here = min(kRowsPerStage, k - r0);
          if (live && !dead) {
            const E* tile = reinterpret_cast<const E*>(ring + size_t(slot) * kStageBytes) + lane;
            const E* piv = piv_all + r0;
            int t = warp;
            for (; t + (kUnroll - 1) * kWarps < rows_here; t += kUnroll * kWarps) {
#pragma unroll
              for (int q = 0; q < kUnroll; ++q) accs[q] = O::sub_conj_mul(accs[q], piv[t + q * kWarps], tile[(t + q * kWarps) * 32]);
            }
            for (; t < rows_here; t += kWarps) accs[0] = O::sub_conj_mul(accs[0], piv[t], tile[t * 32]);
          }
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&empty_bar[slot]);
          ++consumed;
        }
      } else {
        for (int l0 = 0; l0 < k; l0 += kChunk) {
          const int lc = min(kChunk, k - l0);
          __syncthreads();
          for (int t = threadIdx.x; t < lc; t += kBlock) s_pivot_row[t] = Rw[size_t(l0 + t) * n + p];
          __syncthreads();
          if (live) {
            const E* base = Rw + size_t(l0) * n + i;
            int t = warp;
            for (; t + (kUnroll - 1) * kWarps < lc; t += kUnroll * kWarps) {
              E rows[kUnroll];
  #pragma unroll
              for (int q = 0; q < kUnroll; ++q) rows[q] = base[size_t(t + q * kWarps) * n];
  #pragma unroll
              for (int q = 0; q < kUnroll; ++q) accs[q] = O::sub_conj_mul(accs[q], s_pivot_row[t + q * kWarps], rows[q]);
            }
            for (; t < lc; t += kWarps) accs[0] = O::sub_conj_mul(accs[0], s_pivot_row[t], base[size_t(t) * n]);
          }
        }
      }
#pragma unroll
      for (int q = kUnroll / 2; q > 0; q >>= 1)
#pragma unroll
        for (int r = 0; r < q; ++r) accs[r] = O::add(accs[r], accs[r + q]);
      const E acc = accs[0];
      s_partial[warp][lane] = acc;
      __syncthreads();
      if (warp == 0) {
        E out = O::zero();
        if (live) {
          // G[p, i] = conj(G[i, p]): column p of the Hermitian matrix is contiguous
          E v = O::conj(G[i + int64_t(p) * ldg]);
#pragma unroll
          for (int w = 0; w < kWarps; ++w) v = O::add(v, s_partial[w][lane]);
          out = O::scale(v, rinv);
          const R d = T::sub(D[i], O::abs2(out));
          D[i] = d;
          mine.trace += T::to_double(d);
          if (mine.idx < 0 || T::less(mine.val, d)) { mine.val = d; mine.idx = i; }
        } else if (i == p) { out.re = rkk; }
        if (i < n) Rw[size_t(k) * n + i] = out;
        if constexpr (TMA) ptx::fence_proxy_async_global();   // later steps read this row through TMA
      }
      __syncthreads();
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) {
      // swap the pivot into position k; both values a displaced column can be seen with are >= k, so readers
      // of pos[] in other blocks classify it as free either way
      const int q = pos[p], other = jpiv[k] - 1;
      jpiv[k] = p + 1; jpiv[q] = other + 1; pos[other] = q; pos[p] = k;
    }
    // block-level partial for the next step (only warp 0 holds data)
    if (warp == 0) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        P other; other.trace = __shfl_down_sync(0xffffffffu, mine.trace, o); other.idx = __shfl_down_sync(0xffffffffu, mine.idx, o);
        if constexpr (sizeof(R) == 16) { other.val.x = __shfl_down_sync(0xffffffffu, mine.val.x, o); other.val.y = __shfl_down_sync(0xffffffffu, mine.val.y, o); }
        else other.val = __shfl_down_sync(0xffffffffu, mine.val, o);
        mine.trace += other.trace;
        if (other.idx >= 0 && (mine.idx < 0 || T::less(mine.val, other.val))) { mine.val = other.val; mine.idx = other.idx; }
      }
      if constexpr (TMA) mine.pad = int(*reinterpret_cast<volatile uint32_t*>(&s_abort));
      if (lane == 0) partials[size_t((k + 1) & 1) * nblocks + blockIdx.x] = mine;
    }
    grid.sync();
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) *rank_out = k;
}

template <typename R, bool CPLX>
int run_potrfp(const hyacinHandle_t* handle, double eps, int cap, int n, const void* G, int64_t ldg, void* Rw, int32_t* jpiv) {
  using E = Elem<R, CPLX>; using P = Partial<R, CPLX>;
  cudaStream_t stream = handle->cudaStream;
  // TMA route: needs the factor's row pitch and base to be multiples of 16 bytes, and shared memory for at least
  // two ring stages beside the pivot column
  CUtensorMap tmap; std::memset(&tmap, 0, sizeof(tmap));
  const size_t pitch = size_t(n) * sizeof(E);
  int stages = 0; size_t dyn_bytes = 0;
  void* kernel = reinterpret_cast<void*>(potrfp_kernel<R, CPLX, false>);
  if (pitch % 16 == 0 && reinterpret_cast<uintptr_t>(Rw) % 16 == 0 && cap > 0) {
    cudaFuncAttributes attr;
    HYB_CUDA(cudaFuncGetAttributes(&attr, potrfp_kernel<R, CPLX, true>));
    int dev = 0, optin = 0;
    HYB_CUDA(cudaGetDevice(&dev));
    HYB_CUDA(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    const size_t fixed = 1024 + size_t(cap) * sizeof(E) + 16 * sizeof(uint64_t);   // alignment slack, pivot column, barriers
    const long long room = (long long)optin - (long long)attr.sharedSizeBytes - (long long)fixed;
    stages = int(std::min<long long>(6, room / kStageBytes));
    EncodeTiledFn encode = stages >= 2 ? encode_tiled() : nullptr;
    if (encode) {
      constexpr int kRowsPerStage = kStageBytes / (32 * int(sizeof(E)));
      const cuuint64_t dims[2] = {cuuint64_t(pitch / 4), cuuint64_t(cap)};
      const cuuint64_t strides[1] = {cuuint64_t(pitch)};
      const cuuint32_t box[2] = {cuuint32_t(32 * sizeof(E) / 4), cuuint32_t(kRowsPerStage)};
      const cuuint32_t elem[2] = {1, 1};
      CUresult r = encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, Rw, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r == CUDA_SUCCESS) {
        dyn_bytes = fixed + size_t(stages) * kStageBytes;
        kernel = reinterpret_cast<void*>(potrfp_kernel<R, CPLX, true>);
        HYB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(dyn_bytes)));
      } else {
        std::fprintf(stderr, "hyacin-b200: tensor map for the Cholesky factor refused (%d); using plain loads\n", int(r));
      }
    }
  }
  int per_sm = 0;
  HYB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kBlock, dyn_bytes));
  int grid = std::max(1, std::min(handle->DeviceSMs * std::max(per_sm, 1), (n + 31) / 32));
  R* D = nullptr; int* pos = nullptr; P* partials = nullptr;
  HYB_CUDA(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&D), size_t(n) * sizeof(R), handle->mempool, stream));
  HYB_CUDA(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&pos), size_t(n) * sizeof(int), handle->mempool, stream));
  HYB_CUDA(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&partials), size_t(2) * grid * sizeof(P), handle->mempool, stream));
  int32_t* rank_host = static_cast<int32_t*>(handle->pinnedWorkspace);
  *rank_host = 0;
  double eps_sq = eps * eps;
  const E* g = static_cast<const E*>(G); E* rw = static_cast<E*>(Rw);
  void* args[] = {&eps_sq, &n, &cap, &g, &ldg, &rw, &D, &pos, &jpiv, &partials, &rank_host, &stages, &tmap};
  count_launch();
  HYB_CUDA(cudaLaunchCooperativeKernel(kernel, dim3(grid), dim3(kBlock), args, dyn_bytes, stream));
  HYB_CUDA(cudaFreeAsync(D, stream)); HYB_CUDA(cudaFreeAsync(pos, stream)); HYB_CUDA(cudaFreeAsync(partials, stream));
  HYB_CUDA(cudaStreamSynchronize(stream));
  if (*rank_host < 0) {
    std::fprintf(stderr, "hyacin-b200: pivoted Cholesky gave up waiting for a tile of the factor; no result\n");
    return 0;
  }
  return *rank_host;
}

}  // namespace

size_t gram_elem_bytes(hyacinPrecision_t gtype) {
  static const int bytes[12] = {8, 16, 4, 8, 2, 4, 16, 32, 12, 24, 16, 32};
  return (int(gtype) >= 0 && int(gtype) < 12) ? size_t(bytes[int(gtype)]) : 0;
}

int potrfp(const hyacinHandle_t* handle, double eps, int cap, int n, hyacinPrecision_t gtype, const void* G, int64_t ldg,
           void* Rw, int32_t* jpiv) {
  int rank = -1;
  switch (gtype) {
    case HYACIN_F32: rank = run_potrfp<float, false>(handle, eps, cap, n, G, ldg, Rw, jpiv); break;
    case HYACIN_F64: rank = run_potrfp<double, false>(handle, eps, cap, n, G, ldg, Rw, jpiv); break;
    case HYACIN_DD: rank = run_potrfp<DD, false>(handle, eps, cap, n, G, ldg, Rw, jpiv); break;
    case HYACIN_F32_COMPLEX: rank = run_potrfp<float, true>(handle, eps, cap, n, G, ldg, Rw, jpiv); break;
    case HYACIN_F64_COMPLEX: rank = run_potrfp<double, true>(handle, eps, cap, n, G, ldg, Rw, jpiv); break;
    case HYACIN_DD_COMPLEX: rank = run_potrfp<DD, true>(handle, eps, cap, n, G, ldg, Rw, jpiv); break;
    default:
      std::fprintf(stderr, "hyacin-b200: Gram format %d (triple-/quad-float) is only produced on GPUs without fast FP64 and is not supported here\n", int(gtype));
      return 0;
  }
  if (handle->logger) {
    static const char* names[12] = {"FP64", "FP64-COMPLEX", "FP32", "FP32-COMPLEX", "", "", "FP128-DD", "FP128-DD-COMPLEX", "", "", "", ""};
    std::fprintf(static_cast<FILE*>(handle->logger), "POTRFP-%s [eps=%.1le] [N=%d] [K=%d] [Cholesky-rank=%d]\n", names[int(gtype)], eps, n, cap, rank);
  }
  return rank;
}

}  // namespace hyb
