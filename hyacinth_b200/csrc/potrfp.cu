// Truncated pivoted Cholesky of the Gram matrix: G(perm, perm) ~= R^H R, R upper trapezoidal with `rank` rows.
//
// Downstream of the quantized Gram and replicated on every rank.  The factor must come out with the BITS of the
// reference's src/hyacin_potrfp.cu, because the Jacobi SVD that follows runs only three sweeps and amplifies
// last-bit differences of its input.  What fixes those bits (src/hyacin_potrfp.cu:214-272):
//   * the new row of a column is  w = G[l, j] - sum_m conj(R[m, l]) R[m, j]  summed as 128 chains -- chain t takes
//     the previous rows m = t, t + 128, ... in increasing order, chain 0 starts from the Gram entry, the others
//     from zero (:226-230) -- which are then combined by a shuffle tree over each group of 32 chains (partner
//     t + 1, t + 2, t + 4, t + 8, t + 16) and a left-to-right sum of the four group results (the block reduction
//     of :231); the first step has no sum at all (:223);
//   * the arithmetic of one chain step, of the diagonal update and of the square root, per Gram format (:150-176,
//     :57-66 with the double-double helpers of include/internal.hpp:181-227);
//   * ties between equal diagonal entries go to the entry the reference's reduction meets first (:243-252, :258-261);
//   * the stop rule (:262-264, :269): remaining trace <= eps^2 * initial trace, or N - K columns left, and a single
//     remaining column is always counted.
// The remaining trace is summed in this kernel's own fixed order, not the reference's; it only enters the stop
// test.
//
// The organisation is this build's own.  The reference overwrites G, swaps rows and columns in place and spends
// two or three grid barriers and one block reduction per column and step.  Here G is read only, the factor goes
// to a separate column-major array Rc[column][step] indexed by ORIGINAL column, the permutation lives in each
// block's shared memory, and a step costs one grid barrier.  The live columns (those not yet chosen) are dealt
// out again at every step in position order, so the blocks stay balanced and chosen columns are never read
// again; the live part of the factor never exceeds n^2 / 4 elements and stays in L2.  A block of 18 warps:
// 16 consumer warps (4 groups of columns x 128 chains; thread t of a group owns chain t of up to eight columns,
// which is also its instruction-level parallelism), one producer warp that streams 128-row stages of the
// block's columns and of the pivot column into a shared-memory ring with bulk copies (one copy per column and
// stage; no tensor map, no multicast), and one warp that takes the square root off the critical path.
#include "hyb_internal.h"
#include "tail.h"
#include "ptx_sm100.cuh"
#include <cooperative_groups.h>
#include <cfloat>
#include <algorithm>
#include <cstring>

namespace hyb {
namespace {

// ---- scalar arithmetic, one policy per Gram format --------------------------------------------------------
struct alignas(16) DD { double x, y; };       // 16-byte aligned, like the double2 elements of a double-double Gram matrix

__device__ __forceinline__ DD dd_renorm(double a, double b) { double s = a + b, d = a - s; return DD{s, b + d}; }
__device__ __forceinline__ DD dd_mul(DD a, DD b) { double p = a.x * b.x; return dd_renorm(p, fma(a.x, b.y, a.y * b.x) + fma(a.x, b.x, -p)); }
__device__ __forceinline__ DD dd_sqr(DD a) { double p = a.x * a.x; return dd_renorm(p, fma(a.x + a.x, a.y, fma(a.x, a.x, -p))); }
__device__ __forceinline__ DD dd_add(DD a, DD b) {
  double s = a.x + b.x, d = a.x - s, sd = s + d, e = (b.x + d) + (a.x - sd); return dd_renorm(s, (a.y + b.y) + e);
}
__device__ __forceinline__ DD dd_sub(DD a, DD b) {
  double nb = -b.x, s = a.x + nb, d = a.x - s, sd = s + d, e = (nb + d) + (a.x - sd); return dd_renorm(s, (a.y - b.y) + e);
}
__device__ __forceinline__ DD dd_neg(DD a) { return DD{-a.x, -a.y}; }
// 3/2 + x, x small
__device__ __forceinline__ DD dd_three_halves_plus(DD x) { DD y = dd_renorm(1.5, x.x); y.y += x.y; return y; }

template <typename R> struct Real;
template <> struct Real<float> {
  static __device__ __forceinline__ float zero() { return 0.f; }
  static __device__ __forceinline__ float add(float a, float b) { return a + b; }
  static __device__ __forceinline__ float neg(float a) { return -a; }
  static __device__ __forceinline__ float mul(float a, float b) { return a * b; }
  static __device__ __forceinline__ float fnma(float a, float b, float c) { return fmaf(-a, b, c); }      // c - a b
  static __device__ __forceinline__ float fma_(float a, float b, float c) { return fmaf(a, b, c); }
  static __device__ __forceinline__ bool less(float a, float b) { return a < b; }
  static __device__ __forceinline__ double to_double(float a) { return double(a); }
  // returns sqrt(r) and leaves 1 / sqrt(r) in r
  static __device__ __forceinline__ float root(float& r) { float x = sqrtf(r); r = 1.f / x; return x; }
  // rc = r c;  d -= rc^2
  static __device__ __forceinline__ float downdate(float& d, float r, float c) { float rc = r * c; d = fmaf(-rc, rc, d); return rc; }
};
template <> struct Real<double> {
  static __device__ __forceinline__ double zero() { return 0.; }
  static __device__ __forceinline__ double add(double a, double b) { return a + b; }
  static __device__ __forceinline__ double neg(double a) { return -a; }
  static __device__ __forceinline__ double mul(double a, double b) { return a * b; }
  static __device__ __forceinline__ double fnma(double a, double b, double c) { return fma(-a, b, c); }
  static __device__ __forceinline__ double fma_(double a, double b, double c) { return fma(a, b, c); }
  static __device__ __forceinline__ bool less(double a, double b) { return a < b; }
  static __device__ __forceinline__ double to_double(double a) { return a; }
  static __device__ __forceinline__ double root(double& r) { double x = sqrt(r); r = 1. / x; return x; }
  static __device__ __forceinline__ double downdate(double& d, double r, double c) { double rc = r * c; d = fma(-rc, rc, d); return rc; }
};
template <> struct Real<DD> {
  static __device__ __forceinline__ DD zero() { return DD{0., 0.}; }
  static __device__ __forceinline__ DD add(DD a, DD b) { return dd_add(a, b); }
  static __device__ __forceinline__ DD neg(DD a) { return dd_neg(a); }
  static __device__ __forceinline__ DD mul(DD a, DD b) { return dd_mul(a, b); }
  // a rounded product followed by a rounded difference (not a fused form: the factor's bits depend on it)
  static __device__ __forceinline__ DD fnma(DD a, DD b, DD c) { return dd_sub(c, dd_mul(a, b)); }
  static __device__ __forceinline__ bool less(DD a, DD b) { bool l1 = a.x < b.x, l2 = a.y < b.y, p1 = a.x == b.x; return l1 || (p1 && l2); }
  static __device__ __forceinline__ double to_double(DD a) { return a.x; }
  // 1 / sqrt(r) by two Newton steps y <- y (3/2 - (r / 2) y^2) on the mantissa of the double estimate, the
  // exponent put back at the end; sqrt(r) = r / sqrt(r)
  static __device__ __forceinline__ DD root(DD& r) {
    int e; DD y{frexp(rsqrt(r.x), &e), 0.};
    const int e2 = e + e - 1; DD x{scalbn(-r.x, e2), scalbn(-r.y, e2)};
    y = dd_mul(y, dd_three_halves_plus(dd_mul(x, dd_sqr(y))));
    y = dd_mul(y, dd_three_halves_plus(dd_mul(x, dd_sqr(y))));
    x = r; r = DD{scalbn(y.x, e), scalbn(y.y, e)};
    return dd_mul(x, r);
  }
  static __device__ __forceinline__ DD downdate(DD& d, DD r, DD c) { DD rc = dd_mul(r, c); d = dd_sub(d, dd_sqr(rc)); return rc; }
};

template <typename R, bool CPLX> struct Elem { R re; };
template <typename R> struct Elem<R, true> { R re, im; };

template <typename R, bool CPLX> struct Ops {
  using E = Elem<R, CPLX>; using T = Real<R>;
  static __device__ __forceinline__ E zero() { E z; z.re = T::zero(); if constexpr (CPLX) z.im = T::zero(); return z; }
  static __device__ __forceinline__ E add(E a, E b) { a.re = T::add(a.re, b.re); if constexpr (CPLX) a.im = T::add(a.im, b.im); return a; }
  // one chain step: c - conj(a) b, a from the column being updated, b from the pivot column
  static __device__ __forceinline__ E chain(E c, E a, E b) {
    if constexpr (!CPLX) { c.re = T::fnma(a.re, b.re, c.re); return c; }
    else if constexpr (sizeof(R) == sizeof(DD)) {
      // three products: (a.im - a.re)(b.re + b.im) carries both cross terms
      const R p1 = T::mul(a.re, b.re), p2 = T::mul(a.im, b.im), p3 = T::mul(dd_sub(a.im, a.re), dd_add(b.re, b.im));
      E o; o.re = dd_sub(c.re, dd_add(p1, p2)); o.im = dd_add(dd_sub(p1, p2), dd_add(p3, c.im)); return o;
    } else {
      E o; o.re = T::fnma(a.re, b.re, T::fnma(a.im, b.im, c.re)); o.im = T::fnma(a.re, b.im, T::fma_(a.im, b.re, c.im)); return o;
    }
  }
  // new row entry r conj(w), and the diagonal entry of that column reduced by its squared modulus
  static __device__ __forceinline__ E finish(R& d, R r, E w) {
    if constexpr (!CPLX) { E o; o.re = T::downdate(d, r, w.re); return o; }
    else if constexpr (sizeof(R) == sizeof(DD)) {
      E o; o.re = T::mul(r, w.re); o.im = T::mul(r, T::neg(w.im));
      d = dd_sub(d, dd_add(dd_sqr(o.re), dd_sqr(o.im))); return o;
    } else {
      E o; o.re = r * w.re; o.im = -r * w.im;
      d = T::fnma(o.re, o.re, T::fnma(o.im, o.im, d)); return o;
    }
  }
};

__device__ __forceinline__ float shfl_down_real(float v, int o) { return __shfl_down_sync(0xffffffffu, v, o); }
__device__ __forceinline__ double shfl_down_real(double v, int o) { return __shfl_down_sync(0xffffffffu, v, o); }
__device__ __forceinline__ DD shfl_down_real(DD v, int o) { return DD{__shfl_down_sync(0xffffffffu, v.x, o), __shfl_down_sync(0xffffffffu, v.y, o)}; }
__device__ __forceinline__ float shfl_xor_real(float v, int o) { return __shfl_xor_sync(0xffffffffu, v, o); }
__device__ __forceinline__ double shfl_xor_real(double v, int o) { return __shfl_xor_sync(0xffffffffu, v, o); }
__device__ __forceinline__ DD shfl_xor_real(DD v, int o) { return DD{__shfl_xor_sync(0xffffffffu, v.x, o), __shfl_xor_sync(0xffffffffu, v.y, o)}; }
template <typename R, bool CPLX>
__device__ __forceinline__ Elem<R, CPLX> shfl_xor_elem(Elem<R, CPLX> v, int o) {
  Elem<R, CPLX> r; r.re = shfl_xor_real(v.re, o); if constexpr (CPLX) r.im = shfl_xor_real(v.im, o); return r;
}

// ---- block geometry -----------------------------------------------------------------------------------------
constexpr int kChains = 128;                        // chains per column = rows per stage
constexpr int kGroups = 4;                          // column groups of a block
constexpr int kConsumers = kChains * kGroups;       // 16 warps
constexpr int kConsumerWarps = kConsumers / 32;
constexpr int kProducerWarp = kConsumerWarps;       // warp 16
constexpr int kScalarWarp = kConsumerWarps + 1;     // warp 17
constexpr int kThreads = kConsumers + 64;
// columns of one group in one pass: eight chains per thread, four for the 32-byte elements (registers)
template <typename E> struct PerGroup { static constexpr int value = sizeof(E) >= 32 ? 4 : 8; };
constexpr int kMaxStages = 4;

// The best remaining diagonal entry seen so far, the remaining trace, and whether a bounded wait expired.
// key: place of the entry in the order in which the reference's reduction meets the candidates -- among equal
// values the smallest key wins.
// abs_sum: sum of the magnitudes behind `trace`; it bounds how far two summation orders of the trace can differ.
template <typename R> struct Partial { R val; double trace; double abs_sum; int pos; int key; int flag; int pad; };

template <typename R> __device__ __forceinline__ Partial<R> empty_partial() {
  Partial<R> p; p.val = Real<R>::zero(); p.trace = 0.; p.abs_sum = 0.; p.pos = -1; p.key = 0x7fffffff; p.flag = 0; p.pad = 0; return p;
}
// A candidate replaces the current best only if it is larger; the search starts from zero, so entries <= 0 are
// never chosen (src/hyacin_potrfp.cu:111-116).
template <typename R> __device__ __forceinline__ void merge_partial(Partial<R>& a, const Partial<R>& b) {
  a.trace += b.trace; a.abs_sum += b.abs_sum; a.flag |= b.flag;
  if (b.pos < 0) return;
  const bool take = a.pos < 0 || Real<R>::less(a.val, b.val) || (!Real<R>::less(b.val, a.val) && b.key < a.key);
  if (take) { a.val = b.val; a.pos = b.pos; a.key = b.key; }
}
template <typename R> __device__ __forceinline__ void offer(Partial<R>& a, R d, int pos, int key) {
  a.trace += Real<R>::to_double(d); a.abs_sum += fabs(Real<R>::to_double(d));
  if (!Real<R>::less(Real<R>::zero(), d)) return;
  if (a.pos < 0 || Real<R>::less(a.val, d) || (!Real<R>::less(d, a.val) && key < a.key)) { a.val = d; a.pos = pos; a.key = key; }
}
template <typename R> __device__ __forceinline__ void warp_merge_partial(Partial<R>& mine) {
  for (int o = 16; o > 0; o >>= 1) {
    Partial<R> other;
    other.val = shfl_down_real(mine.val, o); other.trace = __shfl_down_sync(0xffffffffu, mine.trace, o);
    other.abs_sum = __shfl_down_sync(0xffffffffu, mine.abs_sum, o);
    other.pos = __shfl_down_sync(0xffffffffu, mine.pos, o); other.key = __shfl_down_sync(0xffffffffu, mine.key, o);
    other.flag = __shfl_down_sync(0xffffffffu, mine.flag, o); other.pad = 0;
    merge_partial(mine, other);
  }
}
// Candidate number `th` (with `second` set for the one extra candidate that the reference's first thread takes
// before its own) -> its priority.  The reference reduces 128 candidates per block with lower threads first, then
// lets thread (b - 1) mod 128 of block 0 walk the results of blocks b, b + 128, ..., its own block first
// (src/hyacin_potrfp.cu:255-261).
__device__ __forceinline__ int candidate_key(int th, int second) {
  const int b = th >> 7, t = th & 127;
  int walker = 0, turn = 0;
  if (b > 0) { walker = (b - 1) & 127; turn = ((b - 1) >> 7) + (walker == 0 ? 1 : 0); }
  return (((walker * 32 + turn) * 128 + t) << 1) | second;
}

// ---- one synchronisation per step --------------------------------------------------------------------------
// At the end of a step every block writes its record for the next one; a cooperative grid barrier follows, and at
// the top of the next step every block reads ALL records and reduces them in the same order.  Two sets of records
// alternate by step parity.  (Letting the records themselves be the barrier -- stamped with the step, written with
// release semantics and polled by every block -- was measured and is slower: 148 x 148 polling reads compete with
// the writes they wait for.)
__device__ __forceinline__ float ldcg_real(const float* p) { return __ldcg(p); }
__device__ __forceinline__ double ldcg_real(const double* p) { return __ldcg(p); }
__device__ __forceinline__ DD ldcg_real(const DD* p) { return DD{__ldcg(&p->x), __ldcg(&p->y)}; }

template <typename R> __device__ __forceinline__ void publish(Partial<R>* slot, const Partial<R>& p) {
  slot->val = p.val; slot->trace = p.trace; slot->abs_sum = p.abs_sum; slot->pos = p.pos; slot->key = p.key; slot->flag = p.flag;
}
template <typename R> __device__ __forceinline__ Partial<R> fetch(const Partial<R>* slot) {
  // L2 loads: these words are rewritten by other blocks every second step
  Partial<R> p = empty_partial<R>();
  p.val = ldcg_real(&slot->val); p.trace = __ldcg(&slot->trace); p.abs_sum = __ldcg(&slot->abs_sum); p.pos = __ldcg(&slot->pos); p.key = __ldcg(&slot->key); p.flag = __ldcg(&slot->flag);
  return p;
}

struct RingShape { int stages, cw, slot_bytes, strip_off, perm_off, bar_off; };

__device__ __forceinline__ void named_barrier(int id, int count) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory"); }

// ---- pieces of a consumer's pass ----------------------------------------------------------------------------
// The stages of one pass, for a thread that owns chain `chain` of CPG columns starting at tile column c_first.
template <typename R, bool CPLX, int CPG>
__device__ __forceinline__ void consume_stages(Elem<R, CPLX>* acc, const uint8_t* ring, const RingShape& shape, uint64_t* full_bar, uint64_t* empty_bar,
                                               uint32_t& consumed, bool& dead, uint32_t S, int nstages, int k, int chain, int c_first, int lane,
                                               volatile uint32_t* abort_flag, uint32_t* status) {
  using E = Elem<R, CPLX>; using O = Ops<R, CPLX>;
  for (int s = 0; s < nstages; ++s) {
    const uint32_t slot = consumed % S, round = consumed / S; ++consumed;
    if (!dead && !ptx::mbar_wait(&full_bar[slot], round & 1u, abort_flag, status, 12u)) dead = true;
    if (!dead && s * kChains + chain < k) {
      const uint8_t* base = ring + size_t(slot) * shape.slot_bytes;
      const E b = reinterpret_cast<const E*>(base + shape.strip_off)[chain];
      const E* tile = reinterpret_cast<const E*>(base) + size_t(c_first) * kChains + chain;
#pragma unroll
      for (int q = 0; q < CPG; ++q) acc[q] = O::chain(acc[q], tile[q * kChains], b);
    }
    __syncwarp();
    if (lane == 0) ptx::mbar_arrive(&empty_bar[slot]);
  }
}

// 32 chains -> one value per column, with the tree of the reference's block reduction: at every level a lane's
// value is added to that of the lane 1, 2, 4, 8, 16 higher (lower lane first).  While a lane still holds several
// columns, the two lanes of a pair split them -- each sends the half it gives up and keeps the half it sums -- so
// the arithmetic is that of the plain tree at a fraction of the additions.  On return lane l < MPG holds the
// result of column bit_reverse(l).
template <typename R, bool CPLX, int MPG>
__device__ __forceinline__ Elem<R, CPLX> tree_reduce(Elem<R, CPLX>* acc, int lane) {
  using O = Ops<R, CPLX>;
  int held = MPG;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const bool upper = (lane & o) != 0;
    if (held > 1) {
      held >>= 1;
#pragma unroll
      for (int q = 0; q < MPG / 2; ++q) {
        if (q < held) {
          const Elem<R, CPLX> give = upper ? acc[q] : acc[q + held];
          const Elem<R, CPLX> got = shfl_xor_elem<R, CPLX>(give, o);
          acc[q] = upper ? O::add(got, acc[q + held]) : O::add(acc[q], got);
        }
      }
    } else {
      const Elem<R, CPLX> got = shfl_xor_elem<R, CPLX>(acc[0], o);
      acc[0] = upper ? O::add(got, acc[0]) : O::add(acc[0], got);
    }
  }
  return acc[0];
}
template <int MPG> __device__ __forceinline__ int tree_column_of_lane(int lane) {
  int c = 0;
#pragma unroll
  for (int bit = 1, out = MPG >> 1; out > 0; bit <<= 1, out >>= 1) if (lane & bit) c |= out;
  return c;
}

// ---- the kernel ---------------------------------------------------------------------------------------------
// The remaining trace summed in the order of the reference's reduction (src/hyacin_potrfp.cu:128-132, 243-261), for the
// stop comparison when it falls within rounding distance (exactly rank-deficient matrices: the remaining diagonal is
// rounding noise) and for the initial trace behind the threshold.  Candidate number th sits in thread th % 128 of block
// th / 128 of the reference; its thread 0 first takes the column that was swapped into the pivot's old place (relative
// position j_rel, if j_rel > 0), then its own; a block sums its 128 threads by the shuffle tree and its four warps left to
// right; thread t of block 0 adds the sums of blocks t + 1, t + 129, ... to its own start value (thread 0: its block's sum,
// the others: zero) and the 128 threads are summed by the same tree.  Candidate th is the column at position
// base + th + 1, or base + th + 2 from the swapped one on.  Holds while every reference thread has at most one candidate:
// n <= kExactColumns.  Called by all threads of the block; the result is the same in every block.
constexpr int kExactBlocks = 148;
constexpr int kExactColumns = kExactBlocks * 128;
template <typename R>
__device__ __forceinline__ double reference_order_trace(const R* D, const uint16_t* perm, int base, int j_rel, int count,
                                                        double* s_agg, double* s_out, int tid) {
  const int warp = tid >> 5, lane = tid & 31;
  const int nb = count > 0 ? (count + 127) >> 7 : 1;
  for (int b = warp; b < nb; b += kThreads / 32) {
    double w4[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int th = 128 * b + 32 * q + lane;
      double x = 0.0;
      if (th < count) {
        const int l = (j_rel > 0 && th + 1 >= j_rel) ? th + 2 : th + 1;
        x = Real<R>::to_double(ldcg_real(&D[perm[base + l]]));
      }
      if (th == 0 && j_rel > 0) x = Real<R>::to_double(ldcg_real(&D[perm[base + j_rel]])) + x;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) x += __shfl_down_sync(0xffffffffu, x, o);
      w4[q] = x;
    }
    if (lane == 0) s_agg[b] = ((w4[0] + w4[1]) + w4[2]) + w4[3];
  }
  __syncthreads();
  if (warp == 0) {
    double w4[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int t = 32 * q + lane;
      double u = t == 0 ? s_agg[0] : 0.0;
      for (int i = t + 1; i < nb; i += 128) u += s_agg[i];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) u += __shfl_down_sync(0xffffffffu, u, o);
      w4[q] = u;
    }
    if (lane == 0) *s_out = ((w4[0] + w4[1]) + w4[2]) + w4[3];
  }
  __syncthreads();
  return *s_out;
}

template <typename R, bool CPLX>
__global__ void __launch_bounds__(kThreads, 1)
potrfp_chain_kernel(double eps_sq, int n, int cap, const Elem<R, CPLX>* __restrict__ G, int64_t ldg, Elem<R, CPLX>* __restrict__ Rc, int64_t ldc,
                    R* __restrict__ D, int32_t* __restrict__ jpiv, int32_t* __restrict__ pos_out, Partial<R>* __restrict__ partials,
                    int32_t* __restrict__ rank_out, const RingShape shape, uint32_t* __restrict__ status) {
  using E = Elem<R, CPLX>; using O = Ops<R, CPLX>; using T = Real<R>; using P = Partial<R>;
  cooperative_groups::grid_group grid = cooperative_groups::this_grid();
  extern __shared__ uint8_t dyn_smem[];
  uint8_t* ring = dyn_smem + ((128u - (ptx::smem_u32(dyn_smem) & 127u)) & 127u);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ring + shape.bar_off);
  uint64_t* empty_bar = full_bar + kMaxStages;
  uint16_t* perm = reinterpret_cast<uint16_t*>(ring + shape.perm_off);     // position -> original column
  __shared__ E s_part[kGroups][32];                 // tree result of each group of 32 chains, per column of the pass
  __shared__ P s_red[2][kThreads / 32];             // by step parity: a warp may still read one step's while another writes the next's
  __shared__ R s_rinv;
  __shared__ double s_agg[kExactBlocks], s_exact;
  __shared__ uint32_t s_abort, s_issued;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nblocks = gridDim.x;
  const int cw = shape.cw;
  const uint32_t S = uint32_t(shape.stages);
  const int grp = warp >> 2, chain = ((warp & 3) << 5) | lane;       // consumers: column group, chain number 0..127
  constexpr uint32_t kColBytes = kChains * sizeof(E);
  constexpr int kMaxPerGroup = PerGroup<E>::value;
  uint32_t issued = 0, consumed = 0;                 // stages requested (producer) / waited for (consumers) so far
  bool dead = false;

  if (tid == 0) {
    for (uint32_t s = 0; s < S; ++s) { ptx::mbar_init(&full_bar[s], 1); ptx::mbar_init(&empty_bar[s], kConsumerWarps); }
    s_abort = 0; s_issued = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = tid; i < n; i += kThreads) perm[i] = uint16_t(i);

  // ---- diagonal, first candidates -----------------------------------------------------------------------
  {
    P mine = empty_partial<R>();
    for (int i = blockIdx.x * kThreads + tid; i < n; i += nblocks * kThreads) {
      const R d = G[i + int64_t(i) * ldg].re;
      D[i] = d;
      offer(mine, d, i, candidate_key(i, 0));
    }
    warp_merge_partial(mine);
    if (lane == 0) s_red[1][warp] = mine;
    __syncthreads();
    if (tid == 0) {
      P acc = s_red[1][0];
      for (int w = 1; w < kThreads / 32; ++w) merge_partial(acc, s_red[1][w]);
      publish(&partials[blockIdx.x], acc);
    }
  }
  grid.sync();

  const int iter_n = cap >= n ? 1 : n - cap;         // columns left at which the rank cap stops the loop
  double threshold = 0.;
  int k = 0, rank = 0, j_last = 0;
  for (;; ++k) {
    // The remaining diagonal lives in two arrays that alternate by step: step k reads D_now and writes D_next, so a block
    // that still sums D_now for its stop decision (reference_order_trace) is not overtaken by the writes of step k; the
    // grid barrier at the end of step k separates those reads from the writes of step k + 1 into the same array.
    const R* D_now = D + size_t(k & 1) * n;
    R* D_next = D + size_t((k + 1) & 1) * n;
    // ---- read and reduce the records of all blocks in the same order: same pivot everywhere ----
    P best;
    {
      P mine = empty_partial<R>();
      if (tid < nblocks) {
        mine = fetch(&partials[size_t(k & 1) * nblocks + tid]);
      }
      if (warp * 32 < nblocks) { warp_merge_partial(mine); if (lane == 0) s_red[k & 1][warp] = mine; }
      __syncthreads();
      best = s_red[k & 1][0];
      for (int w = 1; w * 32 < nblocks; ++w) merge_partial(best, s_red[k & 1][w]);
    }
    const bool have = best.pos >= 0;
    if (best.flag) { rank = -1; break; }
    if (k == 0) {
      if (!have) { rank = 0; break; }
      threshold = eps_sq * (n <= kExactColumns ? reference_order_trace<R>(D_now, perm, -1, 0, n, s_agg, &s_exact, tid) : best.trace);
    } else {
      const int remaining = n - k;
      double trace = best.trace;
      // this build's sum and the reference's differ by at most a few n ulps of the summed magnitudes: only a comparison
      // closer than that needs the reference's own order
      if (n <= kExactColumns && have && remaining > iter_n && fabs(trace - threshold) <= 1.8e-15 * double(n) * best.abs_sum)
        trace = reference_order_trace<R>(D_now, perm, k - 1, j_last, remaining - (j_last > 0 ? 1 : 0), s_agg, &s_exact, tid);
      if (!(have && threshold < trace) || remaining <= iter_n) {
        rank = k + (remaining == 1 ? 1 : 0);
        if (remaining == 1 && blockIdx.x == 0 && tid == 0) {
          // a last single column is counted whatever its diagonal entry is; its row holds the root alone
          R v = have ? best.val : T::zero();
          E out = O::zero(); out.re = T::root(v);
          Rc[size_t(perm[k]) * ldc + k] = out;
        }
        break;
      }
    }
    // The chosen column moves to position k and the column that was there takes its place.  The shared permutation
    // is updated at the END of the step (the order of columns that are never chosen is part of the result, so the
    // swap happens only for steps that run); until then everybody reads it through column_at().
    const int q_pivot = best.pos, j = q_pivot - k;   // position of the pivot before the swap, and relative to k
    j_last = j;
    const int pc = perm[q_pivot], front = perm[k];
    auto column_at = [&](int q) -> int { return q == q_pivot ? front : int(perm[q]); };

    const int live = n - k - 1;                      // positions k + 1 .. n - 1 after the swap
    const int per_block = (live + nblocks - 1) / nblocks;
    const int lo = k + 1 + blockIdx.x * per_block, hi = min(n, lo + per_block);
    const int nstages = (k + kChains - 1) / kChains;
    const int passes = lo < hi ? (hi - lo + cw - 1) / cw : 0;
    if (passes == 0) __syncthreads();                // nothing else keeps the warps of this block together before the swap

    if (warp == kScalarWarp) {
      if (lane == 0) {
        R v = best.val;
        const R root = T::root(v);                   // v <- 1 / sqrt(v)
        s_rinv = v;
        if (blockIdx.x == 0) { E out = O::zero(); out.re = root; Rc[size_t(pc) * ldc + k] = out; }
      }
      __syncwarp();
      for (int p = 0; p < passes; ++p) named_barrier(1, kConsumers + 32);
    } else if (warp == kProducerWarp) {
      for (int p = 0; p < passes; ++p) {
        const int r0 = lo + p * cw, cwr = min(cw, hi - r0);
        const E* src = lane < cwr ? Rc + size_t(column_at(r0 + lane)) * ldc : nullptr;
        const E* strip_src = Rc + size_t(pc) * ldc;
        for (int s = 0; s < nstages; ++s) {
          const uint32_t slot = issued % S, round = issued / S; ++issued;
          int ok = 1;
          if (lane == 0) {
            if (!dead && !ptx::mbar_wait(&empty_bar[slot], (round & 1u) ^ 1u, &s_abort, status, 11u)) dead = true;
            ok = dead ? 0 : 1;
            if (ok) ptx::mbar_expect_tx(&full_bar[slot], uint32_t(cwr + 1) * kColBytes);
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) { dead = true; continue; }
          uint8_t* base = ring + size_t(slot) * shape.slot_bytes;
          if (src) ptx::bulk_load(ptx::smem_u32(base + size_t(lane) * kColBytes), src + size_t(s) * kChains, kColBytes, &full_bar[slot]);
          if (lane == 0) ptx::bulk_load(ptx::smem_u32(base + shape.strip_off), strip_src + size_t(s) * kChains, kColBytes, &full_bar[slot]);
        }
      }
      if (lane == 0) s_issued = issued;
    } else {
      P mine = empty_partial<R>();
      for (int p = 0; p < passes; ++p) {
        const int r0 = lo + p * cw, cwr = min(cw, hi - r0);
        const int cpg = (cwr + kGroups - 1) / kGroups;             // columns per group in this pass (the last groups may get fewer)
        const int c_first = grp * cpg;
        const int my_cols = max(0, min(cpg, cwr - c_first));
        E acc[kMaxPerGroup];
#pragma unroll
        for (int q = 0; q < kMaxPerGroup; ++q) acc[q] = O::zero();
        if (chain == 0) {
          // chain 0 starts from the Gram entry (row = this column, column = pivot column)
#pragma unroll
          for (int q = 0; q < kMaxPerGroup; ++q)
            if (q < my_cols) acc[q] = G[int64_t(column_at(r0 + c_first + q)) + int64_t(pc) * ldg];
        }
        // what the end of the pass needs from global memory is requested now
        R dv = T::zero(); int my_col = 0;
        if (tid < cwr) { my_col = column_at(r0 + tid); dv = ldcg_real(&D_now[my_col]); }
#define HYB_STAGES(N) case N: consume_stages<R, CPLX, N>(acc, ring, shape, full_bar, empty_bar, consumed, dead, S, nstages, k, chain, c_first, lane, &s_abort, status); break;
        if constexpr (kMaxPerGroup == 8) {
          switch (my_cols) { HYB_STAGES(0) HYB_STAGES(1) HYB_STAGES(2) HYB_STAGES(3) HYB_STAGES(4) HYB_STAGES(5) HYB_STAGES(6) HYB_STAGES(7) default: HYB_STAGES(8) }
        } else {
          switch (my_cols) { HYB_STAGES(0) HYB_STAGES(1) HYB_STAGES(2) HYB_STAGES(3) default: HYB_STAGES(4) }
        }
#undef HYB_STAGES
        if (k > 0) {
          const E sum = tree_reduce<R, CPLX, kMaxPerGroup>(acc, lane);
          const int c = tree_column_of_lane<kMaxPerGroup>(lane);
          if (lane < kMaxPerGroup && c < my_cols) s_part[warp & 3][c_first + c] = sum;
        } else if (chain == 0) {
#pragma unroll
          for (int q = 0; q < kMaxPerGroup; ++q)
            if (q < my_cols) s_part[0][c_first + q] = acc[q];
        }
        named_barrier(1, kConsumers + 32);             // with the scalar warp: s_rinv is ready as well
        if (tid < cwr) {
          E w = s_part[0][tid];
          if (k > 0) { w = O::add(w, s_part[1][tid]); w = O::add(w, s_part[2][tid]); w = O::add(w, s_part[3][tid]); }
          const E out = O::finish(dv, s_rinv, w);
          Rc[size_t(my_col) * ldc + k] = out;
          D_next[my_col] = dv;
          ptx::fence_proxy_async_global();              // later steps read the factor through the async proxy
          // place of this column in the reference's scan of the remaining diagonal: the column that moved from
          // position k to the pivot's old place comes first, then the others by position (src/hyacin_potrfp.cu:243-252)
          const int l = r0 + tid - k;
          int key;
          if (j > 0 && l == j) key = candidate_key(0, 0);
          else if (j > 0) key = candidate_key(l - (l > j ? 1 : 0) - 1, 1);
          else key = candidate_key(l - 1, 1);
          offer(mine, dv, r0 + tid, key);
        }
        if (p + 1 < passes) named_barrier(2, kConsumers);          // s_part is rewritten by the next pass
      }
      if (warp == 0) {
        warp_merge_partial(mine);
        if (lane == 0) {
          perm[q_pivot] = uint16_t(front); perm[k] = uint16_t(pc);
          mine.flag = int(*reinterpret_cast<volatile uint32_t*>(&s_abort));
          publish(&partials[size_t((k + 1) & 1) * nblocks + blockIdx.x], mine);
        }
      }
    }
    grid.sync();
  }

  if (rank < 0) {
    // a wait expired somewhere: let this block's copies in flight land before it leaves
    __syncthreads();
    if (tid == 0) {
      const uint32_t until = *reinterpret_cast<volatile uint32_t*>(&s_issued);
      for (uint32_t c = consumed; c < until; ++c) {
        for (uint32_t it = 0; it < ptx::kSpinLimit; ++it) { if (ptx::mbar_try_wait(&full_bar[c % S], (c / S) & 1u)) break; __nanosleep(64); }
      }
    }
    __syncthreads();
  }
  if (blockIdx.x == 0) {
    for (int i = tid; i < n; i += kThreads) { jpiv[i] = int32_t(perm[i]) + 1; pos_out[perm[i]] = i; }
    if (tid == 0) *rank_out = rank;
  }
}

// ---- host side ----------------------------------------------------------------------------------------------
template <typename R, bool CPLX>
bool plan_ring(int n, RingShape* shape, size_t* dyn_bytes) {
  using E = Elem<R, CPLX>;
  cudaFuncAttributes attr;
  if (cudaFuncGetAttributes(&attr, potrfp_chain_kernel<R, CPLX>) != cudaSuccess) return false;
  int dev = 0, optin = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return false;
  const long long perm_bytes = ((long long)n * 2 + 127) / 128 * 128;
  const long long fixed = 128 + 128 + perm_bytes;                 // alignment slack, barriers, permutation
  const long long room = (long long)optin - (long long)attr.sharedSizeBytes - fixed;
  const int col_bytes = kChains * int(sizeof(E));
  // widest pass that leaves room for three stages, at most PerGroup::value columns per group
  int cw = int(std::min<long long>(kGroups * PerGroup<E>::value, room / (3LL * col_bytes) - 1));
  if (cw < kGroups) return false;
  shape->cw = cw;
  shape->strip_off = cw * col_bytes;
  shape->slot_bytes = (cw + 1) * col_bytes;
  shape->stages = int(std::min<long long>(kMaxStages, room / shape->slot_bytes));
  shape->bar_off = shape->stages * shape->slot_bytes;
  shape->perm_off = shape->bar_off + 128;
  *dyn_bytes = size_t(shape->perm_off + perm_bytes + 128);
  return cudaFuncSetAttribute(potrfp_chain_kernel<R, CPLX>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(*dyn_bytes)) == cudaSuccess;
}

template <typename R, bool CPLX>
int run_potrfp(const hyacinHandle_t* handle, double eps, int cap, int n, const void* G, int64_t ldg, void* Rc, int64_t ldc, int32_t* jpiv, int32_t* pos) {
  using E = Elem<R, CPLX>; using P = Partial<R>;
  cudaStream_t stream = handle->cudaStream;
  if (n > 65535 || cap <= 0) return 0;
  RingShape shape{}; size_t dyn_bytes = 0;
  if (!plan_ring<R, CPLX>(n, &shape, &dyn_bytes)) {
    std::fprintf(stderr, "hyacin-b200: pivoted Cholesky: no room for the shared-memory ring (n = %d)\n", n);
    return 0;
  }
  // one block per SM at most (the kernel is launched cooperatively), at least four columns per block
  const int grid = std::max(1, std::min(std::max(handle->DeviceSMs, 1), (n + 3) / 4));
  R* D = nullptr; P* partials = nullptr;
  HYB_CUDA(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&D), size_t(2) * n * sizeof(R), handle->mempool, stream));      // two arrays, by step parity
  HYB_CUDA(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&partials), size_t(2) * grid * sizeof(P), handle->mempool, stream));
  int32_t* rank_host = static_cast<int32_t*>(handle->pinnedWorkspace);
  *rank_host = 0;
  double eps_sq = eps * eps;
  const E* g = static_cast<const E*>(G); E* rc = static_cast<E*>(Rc);
  uint32_t* status = status_word_device(handle->DeviceID);
  void* args[] = {&eps_sq, &n, &cap, &g, &ldg, &rc, &ldc, &D, &jpiv, &pos, &partials, &rank_host, &shape, &status};
  count_launch();
  {
    ProfileScope scope(stream, KernelKind::Cholesky);
    HYB_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(potrfp_chain_kernel<R, CPLX>), dim3(grid), dim3(kThreads), args, dyn_bytes, stream));
  }
  HYB_CUDA(cudaFreeAsync(D, stream)); HYB_CUDA(cudaFreeAsync(partials, stream));
  HYB_CUDA(cudaStreamSynchronize(stream));
  if (*rank_host < 0) {
    std::fprintf(stderr, "hyacin-b200: pivoted Cholesky gave up waiting for a stage of the factor; no result\n");
    return 0;
  }
  return *rank_host;
}

}  // namespace

size_t gram_elem_bytes(hyacinPrecision_t gtype) {
  static const int bytes[12] = {8, 16, 4, 8, 2, 4, 16, 32, 12, 24, 16, 32};
  return (int(gtype) >= 0 && int(gtype) < 12) ? size_t(bytes[int(gtype)]) : 0;
}

// one row more than the cap: with cap = n - 1 the last single column is still counted and gets a row of its own
int64_t factor_col_pitch(int cap) { return (int64_t(std::max(cap, 1)) + 1 + kChains - 1) / kChains * kChains; }

int potrfp(const hyacinHandle_t* handle, double eps, int cap, int n, hyacinPrecision_t gtype, const void* G, int64_t ldg,
           void* Rc, int64_t ldc, int32_t* jpiv, int32_t* pos) {
  int rank = -1;
  switch (gtype) {
    case HYACIN_F32: rank = run_potrfp<float, false>(handle, eps, cap, n, G, ldg, Rc, ldc, jpiv, pos); break;
    case HYACIN_F64: rank = run_potrfp<double, false>(handle, eps, cap, n, G, ldg, Rc, ldc, jpiv, pos); break;
    case HYACIN_DD: rank = run_potrfp<DD, false>(handle, eps, cap, n, G, ldg, Rc, ldc, jpiv, pos); break;
    case HYACIN_F32_COMPLEX: rank = run_potrfp<float, true>(handle, eps, cap, n, G, ldg, Rc, ldc, jpiv, pos); break;
    case HYACIN_F64_COMPLEX: rank = run_potrfp<double, true>(handle, eps, cap, n, G, ldg, Rc, ldc, jpiv, pos); break;
    case HYACIN_DD_COMPLEX: rank = run_potrfp<DD, true>(handle, eps, cap, n, G, ldg, Rc, ldc, jpiv, pos); break;
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
