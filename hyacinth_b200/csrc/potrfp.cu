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
// only recorded), a block owns a run of consecutive columns so that every load of a previous row is one
// contiguous run, the sum over previous rows is split across the threads of a block and combined in a fixed
// order, and a step costs ONE grid barrier: every block re-reduces the per-block (max, argmax, trace) partials
// itself.  Two kernels: the ring kernel streams the factor through shared memory with TMA tile loads and sizes
// the column runs so that every SM has one; the plain kernel (32 columns per block, ordinary loads) is the
// fallback when no tensor map can be made (callers pad the factor's row pitch to 16 bytes, so alignment never
// forces it).
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
  // c - a b in one pass: exact leading product (p, e), cross terms folded into e, one two-sum for the leading
  // difference, one renormalisation at the end (15 operations against 19 for a product followed by a subtraction)
  static __device__ __forceinline__ DD fnma(DD a, DD b, DD c) {
    const double p = a.x * b.x;
    double e = fma(a.x, b.x, -p);
    e = fma(a.x, b.y, e); e = fma(a.y, b.x, e);
    const double s = c.x - p, bb = s - c.x;
    const double err = (c.x - (s - bb)) - (p + bb);
    return dd_renorm(s, (c.y - e) + err);
  }
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

constexpr int kBlock = 512;               // 16 warps
constexpr int kWarps = kBlock / 32;

template <typename R, bool CPLX>
struct Partial { R val; double trace; int idx; int pad; };

// jpiv (1-based) is kept as a permutation that is updated by swapping the chosen column into position k, which
// is the bookkeeping of the reference (src/hyacin_potrfp.cu:243-246), so the whole array -- not only its first
// `rank` entries -- comes out the same.  pos[i] is the inverse map: column i is still free while pos[i] >= k.
template <typename R, bool CPLX>
__global__ void __launch_bounds__(kBlock)
potrfp_plain_kernel(double eps_sq, int n, int cap, const Elem<R, CPLX>* __restrict__ G, int64_t ldg, Elem<R, CPLX>* __restrict__ Rw,
              R* __restrict__ D, int* __restrict__ pos, int32_t* __restrict__ jpiv, Partial<R, CPLX>* __restrict__ partials,
              int32_t* __restrict__ rank_out, int64_t ldr) {
  using E = Elem<R, CPLX>; using O = Ops<R, CPLX>; using T = Real<R>; using P = Partial<R, CPLX>;
  cg::grid_group grid = cg::this_grid();
  constexpr int kChunk = sizeof(E) >= 32 ? 512 : 1024;   // previous rows staged per shared-memory pass
  __shared__ E s_pivot_row[kChunk];                 // conj-multiplier: previous rows at the pivot column
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
        mine.trace += o.trace;
        if (o.idx >= 0 && (mine.idx < 0 || T::less(mine.val, o.val))) { mine.val = o.val; mine.idx = o.idx; }
      }
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
        s_best = acc;
      }
    }
    __syncthreads();
    const P best = s_best;
    if (k == 0) threshold = eps_sq * best.trace;
    // stop: nothing left, rank cap reached, remaining trace at or below the threshold, or a non-positive pivot
    bool stop = best.idx < 0 || k >= cap || (k > 0 && !(threshold < best.trace)) || !(T::to_double(best.val) > 0.);
    if (stop) break;
    const int p = best.idx;
    const R rinv = T::rsqrt(best.val);              // 1 / R[k][p]
    const R rkk = T::mul(best.val, rinv);           // sqrt(d) = d / sqrt(d)
    P mine; mine.val = T::zero(); mine.trace = 0.; mine.idx = -1; mine.pad = 0;

    for (int c0 = blockIdx.x * 32; c0 < n; c0 += nblocks * 32) {
      const int i = c0 + lane;
      const bool live = i < n && i != p && __ldcg(&pos[i]) >= k;
      // kUnroll independent accumulators per thread and kUnroll row loads in flight before any is consumed: the
      // step is bound by the latency of these loads (the factor rows live in L2 / HBM), not by arithmetic
      constexpr int kUnroll = sizeof(E) >= 32 ? 4 : 8;
      E accs[kUnroll];
#pragma unroll
      for (int q = 0; q < kUnroll; ++q) accs[q] = O::zero();
      for (int l0 = 0; l0 < k; l0 += kChunk) {
        const int lc = min(kChunk, k - l0);
        __syncthreads();
        for (int t = threadIdx.x; t < lc; t += kBlock) s_pivot_row[t] = Rw[size_t(l0 + t) * ldr + p];
        __syncthreads();
        if (live) {
          const E* base = Rw + size_t(l0) * ldr + i;
          int t = warp;
          for (; t + (kUnroll - 1) * kWarps < lc; t += kUnroll * kWarps) {
            E rows[kUnroll];
#pragma unroll
            for (int q = 0; q < kUnroll; ++q) rows[q] = base[size_t(t + q * kWarps) * ldr];
#pragma unroll
            for (int q = 0; q < kUnroll; ++q) accs[q] = O::sub_conj_mul(accs[q], s_pivot_row[t + q * kWarps], rows[q]);
          }
          for (; t < lc; t += kWarps) accs[0] = O::sub_conj_mul(accs[0], s_pivot_row[t], base[size_t(t) * ldr]);
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
        if (i < n) Rw[size_t(k) * ldr + i] = out;
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
      if (lane == 0) partials[size_t((k + 1) & 1) * nblocks + blockIdx.x] = mine;
    }
    grid.sync();
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) *rank_out = k;
}

constexpr int kStageBytes = 65536;      // tile part of a ring stage, at most

// ---- pieces shared by both kernels ------------------------------------------------------------------------
template <typename R, bool CPLX>
__device__ __forceinline__ void merge_partial(Partial<R, CPLX>& a, const Partial<R, CPLX>& b) {
  a.trace += b.trace; a.pad |= b.pad;
  if (b.idx >= 0 && (a.idx < 0 || Real<R>::less(a.val, b.val))) { a.val = b.val; a.idx = b.idx; }
}
__device__ __forceinline__ float shfl_down_real(float v, int o) { return __shfl_down_sync(0xffffffffu, v, o); }
__device__ __forceinline__ double shfl_down_real(double v, int o) { return __shfl_down_sync(0xffffffffu, v, o); }
__device__ __forceinline__ DD shfl_down_real(DD v, int o) { return DD{__shfl_down_sync(0xffffffffu, v.x, o), __shfl_down_sync(0xffffffffu, v.y, o)}; }
__device__ __forceinline__ float shfl_xor_real(float v, int o) { return __shfl_xor_sync(0xffffffffu, v, o); }
__device__ __forceinline__ double shfl_xor_real(double v, int o) { return __shfl_xor_sync(0xffffffffu, v, o); }
__device__ __forceinline__ DD shfl_xor_real(DD v, int o) { return DD{__shfl_xor_sync(0xffffffffu, v.x, o), __shfl_xor_sync(0xffffffffu, v.y, o)}; }
// lanes 0..2^levels-1 of a warp: lane 0 ends up with the merge of all of them, same tree everywhere
template <typename R, bool CPLX>
__device__ __forceinline__ void warp_merge_partial(Partial<R, CPLX>& mine, int first_offset) {
  for (int o = first_offset; o > 0; o >>= 1) {
    Partial<R, CPLX> other;
    other.val = shfl_down_real(mine.val, o); other.trace = __shfl_down_sync(0xffffffffu, mine.trace, o);
    other.idx = __shfl_down_sync(0xffffffffu, mine.idx, o); other.pad = __shfl_down_sync(0xffffffffu, mine.pad, o);
    merge_partial(mine, other);
  }
}
template <typename R, bool CPLX>
__device__ __forceinline__ Partial<R, CPLX> empty_partial() {
  Partial<R, CPLX> p; p.val = Real<R>::zero(); p.trace = 0.; p.idx = -1; p.pad = 0; return p;
}

// ---- ring kernel ------------------------------------------------------------------------------------------
// A block owns `cols` consecutive columns (chosen on the host so that every SM gets one run when n allows it).
// A lane works on column lane % cols and on every (16 * (32 / cols))-th previous row, so small column runs
// still use every lane.  Previous rows arrive in stages of `rows_per_stage` rows through two bulk loads per
// stage: a TMA tile of the block's own columns ("tile"), and the same rows of the pivot column ("strip"), which
// is one contiguous run because the kernel keeps a second, column-major copy Rc[i][k] of the factor.  Tiles of
// the first stages are requested at the top of a step, before the pivot is known; strips follow once it is.
// Thread 0 issues, all 16 warps consume; no multicast anywhere.
struct RingShape { int stages, cols, rows_per_stage, strip_offset, slot_bytes; };
constexpr int kMaxStages = 4;

template <typename R, bool CPLX>
__global__ void __launch_bounds__(kBlock, 1)
potrfp_ring_kernel(double eps_sq, int n, int cap, const Elem<R, CPLX>* __restrict__ G, int64_t ldg, Elem<R, CPLX>* __restrict__ Rw,
                   R* __restrict__ D, int* __restrict__ pos, int32_t* __restrict__ jpiv, Partial<R, CPLX>* __restrict__ partials,
                   int32_t* __restrict__ rank_out, const RingShape shape, const __grid_constant__ CUtensorMap tile_map,
                   Elem<R, CPLX>* __restrict__ Rc, int64_t ldc, int64_t ldr) {
  using E = Elem<R, CPLX>; using O = Ops<R, CPLX>; using T = Real<R>; using P = Partial<R, CPLX>;
  cg::grid_group grid = cg::this_grid();
  constexpr int kUnroll = 4;
  extern __shared__ uint8_t dyn_smem[];
  uint8_t* ring = dyn_smem + ((1024u - (ptx::smem_u32(dyn_smem) & 1023u)) & 1023u);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ring + size_t(shape.stages) * shape.slot_bytes);
  uint64_t* empty_bar = full_bar + kMaxStages;
  __shared__ E s_partial[kWarps][32];
  __shared__ E s_sum[32];
  __shared__ P s_red[kWarps];
  __shared__ P s_best;
  __shared__ R s_scale[2];
  __shared__ uint32_t s_abort, s_status;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblocks = gridDim.x;
  const int cols = shape.cols, rsub = 32 / cols, rps = shape.rows_per_stage;
  const uint32_t S = uint32_t(shape.stages);
  const int lane_row = lane / cols, lane_col = lane - lane_row * cols;
  const bool lane_on = lane_row < rsub;
  const int row_stride = kWarps * rsub, row_first = warp * rsub + lane_row;
  const int rows_per_thread = rps / row_stride, tile_stride = row_stride * cols;
  const uint32_t tile_bytes = uint32_t(rps) * cols * sizeof(E), strip_bytes = uint32_t(rps) * sizeof(E);
  uint32_t issued_tiles = 0, issued_strips = 0;     // thread 0: chunks requested since the kernel started
  uint32_t consumed = 0;                            // every thread: chunks waited for since the kernel started
  bool dead = false;                                // a bounded wait expired in this thread
  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < S; ++s) { ptx::mbar_init(&full_bar[s], 2); ptx::mbar_init(&empty_bar[s], kWarps); }
    s_abort = 0; s_status = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  auto issue_tile = [&](int chunk, int c0) {
    const uint32_t slot = issued_tiles % S, round = issued_tiles / S; ++issued_tiles;
    if (!dead && !ptx::mbar_wait(&empty_bar[slot], (round & 1u) ^ 1u, &s_abort, &s_status, 1u)) dead = true;
    if (dead) return;
    ptx::mbar_expect_tx(&full_bar[slot], tile_bytes);
    ptx::tma_load_2d(ptx::smem_u32(ring + size_t(slot) * shape.slot_bytes), &tile_map, &full_bar[slot], c0 * int(sizeof(E) / 4), chunk * rps);
  };
  auto issue_strip = [&](int chunk, int p) {         // always after issue_tile of the same chunk
    const uint32_t slot = issued_strips % S; ++issued_strips;
    if (dead) return;
    ptx::mbar_expect_tx(&full_bar[slot], strip_bytes);
    ptx::bulk_load(ptx::smem_u32(ring + size_t(slot) * shape.slot_bytes + shape.strip_offset), Rc + size_t(p) * ldc + size_t(chunk) * rps,
                   strip_bytes, &full_bar[slot]);
  };

  // Odd steps walk the previous rows from the last stage to the first: what the step before read last is then
  // read first, so a factor somewhat larger than L2 still finds most of itself there.
  auto chunk_of = [&](int step, int c) { return (step & 1) ? (step + rps - 1) / rps - 1 - c : c; };

  // ---- step "-1": diagonal, initial partials ----
  {
    P mine = empty_partial<R, CPLX>();
    for (int i = blockIdx.x * kBlock + threadIdx.x; i < n; i += nblocks * kBlock) {
      const R d = G[i + int64_t(i) * ldg].re;
      D[i] = d; pos[i] = i; jpiv[i] = i + 1;
      mine.trace += T::to_double(d);
      if (mine.idx < 0 || T::less(mine.val, d)) { mine.val = d; mine.idx = i; }
    }
    warp_merge_partial(mine, 16);
    if (lane == 0) s_red[warp] = mine;
    __syncthreads();
    if (warp == 0) {
      P acc = lane < kWarps ? s_red[lane] : empty_partial<R, CPLX>();
      warp_merge_partial(acc, kWarps / 2);
      if (lane == 0) partials[blockIdx.x] = acc;
    }
  }
  grid.sync();

  double threshold = 0.;
  int k = 0;
  const int first_c0 = blockIdx.x * cols;
  for (;; ++k) {
    const int nchunks = (k + rps - 1) / rps;
    const int n_pro = min(nchunks, int(S) - 1);       // tiles of the first column run requested at the end of step k - 1
    auto chunk_at = [&](int c) { return chunk_of(k, c); };

    // ---- every block reduces the partials of all blocks in the same order: same pivot everywhere ----
    {
      const P* cur = partials + size_t(k & 1) * nblocks;
      P mine = empty_partial<R, CPLX>();
      for (int b = threadIdx.x; b < nblocks; b += kBlock) {
        // L2 loads: these words are rewritten by other blocks every second step
        P o; o.trace = __ldcg(&cur[b].trace); o.idx = __ldcg(&cur[b].idx); o.pad = __ldcg(&cur[b].pad);
        if constexpr (sizeof(R) == 16) { o.val.x = __ldcg(&cur[b].val.x); o.val.y = __ldcg(&cur[b].val.y); } else o.val = __ldcg(&cur[b].val);
        merge_partial(mine, o);
      }
      warp_merge_partial(mine, 16);
      if (lane == 0) s_red[warp] = mine;
      __syncthreads();
      if (warp == 0) {
        P acc = lane < kWarps ? s_red[lane] : empty_partial<R, CPLX>();
        warp_merge_partial(acc, kWarps / 2);
        if (lane == 0) s_best = acc;
      }
      __syncthreads();
    }
    const P best = s_best;
    if (k == 0) threshold = eps_sq * best.trace;
    // stop: a wait expired somewhere (the flag travels with the partials, so every block sees it at the same
    // step), nothing left, rank cap reached, remaining trace at or below the threshold, or a non-positive pivot
    const bool stop = best.pad != 0 || best.idx < 0 || k >= cap || (k > 0 && !(threshold < best.trace)) || !(T::to_double(best.val) > 0.);
    if (stop) {
      // let the tiles requested above land before the block leaves
      if (first_c0 < n) {
        if (threadIdx.x == 0) for (int c = 0; c < n_pro; ++c) issue_strip(chunk_at(c), 0);
        for (int c = 0; c < n_pro; ++c) {
          const uint32_t slot = consumed % S, round = consumed / S; ++consumed;
          if (!dead && !ptx::mbar_wait(&full_bar[slot], round & 1u, &s_abort, &s_status, 3u)) dead = true;
        }
      }
      if (best.pad != 0) k = -1;
      break;
    }
    const int p = best.idx;
    if (threadIdx.x == 32) {                        // off the path of the issuing warp; read after the block barriers below
      const R rinv = T::rsqrt(best.val);            // 1 / R[k][p]
      s_scale[0] = rinv; s_scale[1] = T::mul(best.val, rinv);   // sqrt(d) = d / sqrt(d)
    }
    P mine = empty_partial<R, CPLX>();

    for (int c0 = first_c0; c0 < n; c0 += nblocks * cols) {
      if (threadIdx.x == 0) {
        if (c0 != first_c0) for (int c = 0; c < n_pro; ++c) issue_tile(chunk_at(c), c0);
        for (int c = 0; c < n_pro; ++c) issue_strip(chunk_at(c), p);
      }
      // what the last part of the step needs from global memory is requested now
      const int ei = c0 + lane;
      bool alive = false; E gv = O::zero(); R dv = T::zero();
      if (warp == 0 && lane < cols && ei < n) {
        alive = ei != p && __ldcg(&pos[ei]) >= k;
        // G[p, i] = conj(G[i, p]): column p of the Hermitian matrix is contiguous
        if (alive) { gv = G[ei + int64_t(p) * ldg]; dv = D[ei]; }
      }
      E accs[kUnroll];
#pragma unroll
      for (int q = 0; q < kUnroll; ++q) accs[q] = O::zero();
      for (int c = 0; c < nchunks; ++c) {
        // the slot that chunk c + stages - 1 goes to held chunk c - 1, which this warp released one turn ago:
        // the wait inside issue_tile() only waits for the other warps to release it too
        if (threadIdx.x == 0 && c + int(S) - 1 < nchunks) { issue_tile(chunk_at(c + int(S) - 1), c0); issue_strip(chunk_at(c + int(S) - 1), p); }
        const uint32_t slot = consumed % S, round = consumed / S; ++consumed;
        if (!dead && !ptx::mbar_wait(&full_bar[slot], round & 1u, &s_abort, &s_status, 2u)) dead = true;
        const int rows_here = min(rps, k - chunk_at(c) * rps);
        if (lane_on && !dead) {
          const uint8_t* stage = ring + size_t(slot) * shape.slot_bytes;
          const E* tile = reinterpret_cast<const E*>(stage) + lane_col;
          const E* strip = reinterpret_cast<const E*>(stage + shape.strip_offset);
          if (rows_here == rps && (rows_per_thread & 3) == 0) {
            // whole stage: four rows per turn, one accumulator each, addresses advanced by fixed strides
            const E* tp = tile + row_first * cols; const E* sp = strip + row_first;
            for (int j = 0; j < rows_per_thread; j += 4) {
#pragma unroll
              for (int q = 0; q < 4; ++q) accs[q] = O::sub_conj_mul(accs[q], sp[q * row_stride], tp[q * tile_stride]);
              sp += 4 * row_stride; tp += 4 * tile_stride;
            }
          } else {
            for (int t = row_first; t < rows_here; t += 4 * row_stride) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const int tt = t + q * row_stride;
                if (tt < rows_here) accs[q] = O::sub_conj_mul(accs[q], strip[tt], tile[tt * cols]);
              }
            }
          }
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&empty_bar[slot]);
      }
#pragma unroll
      for (int q = kUnroll / 2; q > 0; q >>= 1)
#pragma unroll
        for (int r = 0; r < q; ++r) accs[r] = O::add(accs[r], accs[r + q]);
      s_partial[warp][lane] = lane_on ? accs[0] : O::zero();
      __syncthreads();
      {
        // 16 consecutive threads hold the 16 warps' sums of one column: fold the row sub-lanes, then a 4-level tree
        const int c = threadIdx.x >> 4, j = threadIdx.x & 15;
        E v = O::zero();
        if (c < cols) for (int r = 0; r < rsub; ++r) v = O::add(v, s_partial[j][c + cols * r]);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) {
          E other; other.re = shfl_xor_real(v.re, o); if constexpr (CPLX) other.im = shfl_xor_real(v.im, o);
          v = O::add(v, other);
        }
        if (j == 0 && c < cols) s_sum[c] = v;
      }
      __syncthreads();
      if (warp == 0 && lane < cols && ei < n) {
        E out = O::zero();
        if (alive) {
          out = O::scale(O::add(O::conj(gv), s_sum[lane]), s_scale[0]);
          const R d = T::sub(dv, O::abs2(out));
          D[ei] = d;
          mine.trace += T::to_double(d);
          if (mine.idx < 0 || T::less(mine.val, d)) { mine.val = d; mine.idx = ei; }
        } else if (ei == p) { out.re = s_scale[1]; }
        Rw[size_t(k) * ldr + ei] = out;
        Rc[size_t(ei) * ldc + k] = out;
        ptx::fence_proxy_async_global();              // later steps read both copies through the async proxy
      }
    }
    // The tiles of this block's first column run for the next step depend on nothing that other blocks do (row k
    // of these columns was written just above, by this warp): request them before the grid barrier.
    if (warp == 0) {
      __syncwarp();
      if (lane == 0 && first_c0 < n) {
        const int next_pro = min((k + 1 + rps - 1) / rps, int(S) - 1);
        for (int c = 0; c < next_pro; ++c) issue_tile(chunk_of(k + 1, c), first_c0);
      }
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) {
      // swap the pivot into position k; both values a displaced column can be seen with are >= k, so readers
      // of pos[] in other blocks classify it as free either way
      const int q = pos[p], other = jpiv[k] - 1;
      jpiv[k] = p + 1; jpiv[q] = other + 1; pos[other] = q; pos[p] = k;
    }
    // block-level partial for the next step (only warp 0 holds data)
    if (warp == 0) {
      warp_merge_partial(mine, 16);
      if (lane == 0) { mine.pad = int(*reinterpret_cast<volatile uint32_t*>(&s_abort)); partials[size_t((k + 1) & 1) * nblocks + blockIdx.x] = mine; }
    }
    grid.sync();
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) *rank_out = k;
}

// ---- host side ----------------------------------------------------------------------------------------------
template <typename R, bool CPLX>
bool plan_ring(const hyacinHandle_t* handle, int cap, int n, void* Rw, int64_t ldr, RingShape* shape, CUtensorMap* tile_map, size_t* dyn_bytes) {
  using E = Elem<R, CPLX>;
  const size_t pitch = size_t(ldr) * sizeof(E);
  if (pitch % 16 != 0 || reinterpret_cast<uintptr_t>(Rw) % 16 != 0 || cap <= 0) return false;
  EncodeTiledFn encode = encode_tiled();
  if (!encode) return false;
  // columns per block: one run per SM when n allows it, a multiple of what keeps tile starts on 16-byte boundaries
  const int align = sizeof(E) >= 16 ? 1 : 16 / int(sizeof(E));
  const int sms = std::max(handle->DeviceSMs, 1);
  const int rounds = (n + 32 * sms - 1) / (32 * sms);
  int cols = (n + sms * rounds - 1) / (sms * rounds);
  cols = std::max(cols, 8);
  cols = std::min(32, (cols + align - 1) / align * align);
  const int row_stride = kWarps * (32 / cols);
  int rps = std::min(256, kStageBytes / (cols * int(sizeof(E))));
  rps = rps >= 4 * row_stride ? rps / (4 * row_stride) * (4 * row_stride) : std::max(row_stride, rps / row_stride * row_stride);
  if (rps > 256) return false;
  const int tile_bytes = rps * cols * int(sizeof(E));
  shape->cols = cols; shape->rows_per_stage = rps;
  shape->strip_offset = (tile_bytes + 127) / 128 * 128;
  shape->slot_bytes = (shape->strip_offset + rps * int(sizeof(E)) + 127) / 128 * 128;
  cudaFuncAttributes attr;
  if (cudaFuncGetAttributes(&attr, potrfp_ring_kernel<R, CPLX>) != cudaSuccess) return false;
  int dev = 0, optin = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return false;
  const long long fixed = 1024 + 2 * kMaxStages * (long long)sizeof(uint64_t);      // alignment slack, barriers
  const long long room = (long long)optin - (long long)attr.sharedSizeBytes - fixed;
  shape->stages = int(std::min<long long>(kMaxStages, room / shape->slot_bytes));
  if (shape->stages < 2) return false;
  *dyn_bytes = size_t(fixed) + size_t(shape->stages) * shape->slot_bytes;
  const cuuint64_t dims[2] = {cuuint64_t(size_t(n) * sizeof(E) / 4), cuuint64_t(cap)};
  const cuuint64_t strides[1] = {cuuint64_t(pitch)};
  const cuuint32_t elem[2] = {1, 1};
  const cuuint32_t tile_box[2] = {cuuint32_t(cols * sizeof(E) / 4), cuuint32_t(rps)};
  CUresult r1 = encode(tile_map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, Rw, dims, strides, tile_box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                       CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r1 != CUDA_SUCCESS) {
    std::fprintf(stderr, "hyacin-b200: tensor map for the Cholesky factor refused (%d); using plain loads\n", int(r1));
    return false;
  }
  return cudaFuncSetAttribute(potrfp_ring_kernel<R, CPLX>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(*dyn_bytes)) == cudaSuccess;
}

template <typename R, bool CPLX>
int run_potrfp(const hyacinHandle_t* handle, double eps, int cap, int n, const void* G, int64_t ldg, void* Rw, int64_t ldr, int32_t* jpiv) {
  using E = Elem<R, CPLX>; using P = Partial<R, CPLX>;
  cudaStream_t stream = handle->cudaStream;
  RingShape shape{}; CUtensorMap tile_map; size_t dyn_bytes = 0;
  std::memset(&tile_map, 0, sizeof(tile_map));
  const bool ring = plan_ring<R, CPLX>(handle, cap, n, Rw, ldr, &shape, &tile_map, &dyn_bytes);
  void* kernel = ring ? reinterpret_cast<void*>(potrfp_ring_kernel<R, CPLX>) : reinterpret_cast<void*>(potrfp_plain_kernel<R, CPLX>);
  if (!ring) dyn_bytes = 0;
  const int group_cols = ring ? shape.cols : 32;
  int per_sm = 0;
  HYB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kBlock, dyn_bytes));
  int grid = std::max(1, std::min(handle->DeviceSMs * std::max(per_sm, 1), (n + group_cols - 1) / group_cols));
  R* D = nullptr; int* pos = nullptr; P* partials = nullptr; E* rc = nullptr;
  // column-major copy of the factor for the ring kernel; a column is padded to whole stages so that a strip never
  // runs past it
  int64_t ldc = 0;
  if (ring) {
    ldc = int64_t(cap + shape.rows_per_stage - 1) / shape.rows_per_stage * shape.rows_per_stage;
    HYB_CUDA(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&rc), size_t(n) * size_t(ldc) * sizeof(E), handle->mempool, stream));
  }
  HYB_CUDA(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&D), size_t(n) * sizeof(R), handle->mempool, stream));
  HYB_CUDA(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&pos), size_t(n) * sizeof(int), handle->mempool, stream));
  HYB_CUDA(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&partials), size_t(2) * grid * sizeof(P), handle->mempool, stream));
  int32_t* rank_host = static_cast<int32_t*>(handle->pinnedWorkspace);
  *rank_host = 0;
  double eps_sq = eps * eps;
  const E* g = static_cast<const E*>(G); E* rw = static_cast<E*>(Rw);
  void* args_ring[] = {&eps_sq, &n, &cap, &g, &ldg, &rw, &D, &pos, &jpiv, &partials, &rank_host, &shape, &tile_map, &rc, &ldc, &ldr};
  void* args_plain[] = {&eps_sq, &n, &cap, &g, &ldg, &rw, &D, &pos, &jpiv, &partials, &rank_host, &ldr};
  count_launch();
  HYB_CUDA(cudaLaunchCooperativeKernel(kernel, dim3(grid), dim3(kBlock), ring ? args_ring : args_plain, dyn_bytes, stream));
  HYB_CUDA(cudaFreeAsync(D, stream)); HYB_CUDA(cudaFreeAsync(pos, stream)); HYB_CUDA(cudaFreeAsync(partials, stream));
  if (rc) HYB_CUDA(cudaFreeAsync(rc, stream));
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

int64_t factor_row_pitch(int n, hyacinPrecision_t gtype) {
  const size_t eb = gram_elem_bytes(gtype);
  const int64_t unit = (eb == 0 || eb >= 16) ? 1 : int64_t(16 / eb);      // 4-, 8- and 12-byte elements: 4, 2, 4 per 16 bytes
  return (int64_t(n) + unit - 1) / unit * unit;
}

int potrfp(const hyacinHandle_t* handle, double eps, int cap, int n, hyacinPrecision_t gtype, const void* G, int64_t ldg,
           void* Rw, int64_t ldr, int32_t* jpiv) {
  int rank = -1;
  switch (gtype) {
    case HYACIN_F32: rank = run_potrfp<float, false>(handle, eps, cap, n, G, ldg, Rw, ldr, jpiv); break;
    case HYACIN_F64: rank = run_potrfp<double, false>(handle, eps, cap, n, G, ldg, Rw, ldr, jpiv); break;
    case HYACIN_DD: rank = run_potrfp<DD, false>(handle, eps, cap, n, G, ldg, Rw, ldr, jpiv); break;
    case HYACIN_F32_COMPLEX: rank = run_potrfp<float, true>(handle, eps, cap, n, G, ldg, Rw, ldr, jpiv); break;
    case HYACIN_F64_COMPLEX: rank = run_potrfp<double, true>(handle, eps, cap, n, G, ldg, Rw, ldr, jpiv); break;
    case HYACIN_DD_COMPLEX: rank = run_potrfp<DD, true>(handle, eps, cap, n, G, ldg, Rw, ldr, jpiv); break;
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
