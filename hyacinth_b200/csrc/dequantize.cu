// Packed integer Gram -> floating-point Gram matrix, and the choice of its format.
//
// Results must be bit-identical to the reference's, because the pivoted Cholesky that follows picks pivots
// from them; the conversion therefore keeps the reference's operation order (src/fp_i63tp_dequantize.cu:56-69
// for double / double-double, :71-88 for triple- and quad-float, helpers in include/internal.hpp:181-227).
// What is new is the data movement: the reference writes the mirrored half with a 16- or 32-byte store per
// thread at a stride of one matrix column; here a 32 x 32 tile goes through shared memory so that both the
// upper tile and its mirror image are written as contiguous runs.
#include "hyb_internal.h"
#include "slices.cuh"
#include <climits>

namespace hyb {
namespace {

struct dd2 { double2 re, im; };      // complex double-double  (reference: complex_double2)
struct tf2 { float3 re, im; };       // complex triple-float
struct qf2 { float4 re, im; };       // complex quad-float

// ---- error-free transformations, as in the reference's helpers -----------------------------------------
__device__ __forceinline__ double2 renorm(double2 a) { double s = a.x + a.y, d = a.x - s; return make_double2(s, a.y + d); }
__device__ __forceinline__ double2 dd_add(double2 a, double2 b) {
  double s = a.x + b.x, d = a.x - s, sd = s + d, e = (b.x + d) + (a.x - sd);
  return renorm(make_double2(s, (a.y + b.y) + e));
}
__device__ __forceinline__ void two_sum(float a, float b, float& s, float& e) { s = a + b; float d = a - s, sd = s + d; e = (b + d) + (a - sd); }
__device__ __forceinline__ float3 renorm(float3 a) {
  float x = a.x + a.y, y = (a.x - x) + a.y, s0 = x + a.z, z = (x - s0) + a.z, s1 = y + z;
  return make_float3(s0, s1, (y - s1) + z);
}
__device__ __forceinline__ float4 renorm(float4 a) {
  float x = a.x + a.y, y = (a.x - x) + a.y, s0 = x + a.z, z = (x - s0) + a.z, s1 = y + z, s2 = (y - s1) + z;
  x = s0 + a.w; float w = (s0 - x) + a.w; y = s1 + w; w += s1 - y; z = s2 + w;
  return make_float4(x, y, z, (s2 - z) + w);
}
__device__ __forceinline__ float3 tf_add(float3 a, float3 b) {
  float s0, s1, e0, e1; two_sum(a.x, b.x, s0, e0); two_sum(a.y, b.y, s1, e1); two_sum(s1, e0, s1, e0);
  return renorm(make_float3(s0, s1, (a.z + b.z) + (e0 + e1)));
}
__device__ __forceinline__ float4 qf_add(float4 a, float4 b) {
  float s0, s1, s2, e0, e1, e2;
  two_sum(a.x, b.x, s0, e0); two_sum(a.y, b.y, s1, e1); two_sum(a.z, b.z, s2, e2);
  two_sum(s1, e0, s1, e0); two_sum(s2, e1, s2, e1);
  two_sum(s2, e0, s2, e0);
  return renorm(make_float4(s0, s1, s2, (a.w + b.w) + (e0 + e1 + e2)));
}

// (high 32 bits as signed) * 2^32 and low 32 bits as unsigned: an exact two-term split of a 64-bit limb.
__device__ __forceinline__ double2 limb_split(uint64_t i) { return make_double2(scalbn(double(int32_t(i >> 32)), 32), double(uint32_t(i))); }
// Three 24-bit pieces of a limb scaled by 2^-126 (keeps single precision inside its exponent range).
__device__ __forceinline__ float3 limb_split_tf(uint64_t i) {
  return renorm(make_float3(scalbnf(float(int16_t(i >> 48)), -78), scalbnf(float(uint32_t(i >> 24) & 0xFFFFFFu), -102),
                            scalbnf(float(uint32_t(i) & 0xFFFFFFu), -126)));
}

template <int ORDER> __device__ __forceinline__ double to_f64(const uint64_t (&a)[ORDER], int e) {
  double res = double(int64_t(a[ORDER - 1]));
#pragma unroll
  for (int l = ORDER - 2; l >= 0; --l) { double2 i = limb_split(a[l]); res = (scalbn(res, 63) + i.x) + i.y; }
  return scalbn(res, e);
}
template <int ORDER> __device__ __forceinline__ double2 to_dd(const uint64_t (&a)[ORDER], int e) {
  double2 res = renorm(limb_split(a[ORDER - 1]));
#pragma unroll
  for (int l = ORDER - 2; l >= 0; --l) res = dd_add(make_double2(scalbn(res.x, 63), scalbn(res.y, 63)), renorm(limb_split(a[l])));
  return make_double2(scalbn(res.x, e), scalbn(res.y, e));
}
template <int ORDER> __device__ __forceinline__ float3 to_tf(const uint64_t (&a)[ORDER], int e) {
  float3 res = limb_split_tf(a[ORDER - 1]);
#pragma unroll
  for (int l = ORDER - 2; l >= 0; --l) res = tf_add(make_float3(scalbnf(res.x, 63), scalbnf(res.y, 63), scalbnf(res.z, 63)), limb_split_tf(a[l]));
  e += 126; return make_float3(scalbnf(res.x, e), scalbnf(res.y, e), scalbnf(res.z, e));
}
template <int ORDER> __device__ __forceinline__ float4 to_qf(const uint64_t (&a)[ORDER], int e) {
  float3 t = limb_split_tf(a[ORDER - 1]); float4 res = make_float4(t.x, t.y, t.z, 0.f);
#pragma unroll
  for (int l = ORDER - 2; l >= 0; --l) {
    float3 n = limb_split_tf(a[l]);
    res = qf_add(make_float4(scalbnf(res.x, 63), scalbnf(res.y, 63), scalbnf(res.z, 63), scalbnf(res.w, 63)), make_float4(n.x, n.y, n.z, 0.f));
  }
  e += 126; return make_float4(scalbnf(res.x, e), scalbnf(res.y, e), scalbnf(res.z, e), scalbnf(res.w, e));
}

template <typename R> struct Conv;
template <> struct Conv<double> { template <int O> static __device__ double run(const uint64_t (&a)[O], int e) { return to_f64<O>(a, e); }
  static __device__ double neg(double v) { return -v; } static __device__ double zero() { return 0.0; } };
template <> struct Conv<float> { template <int O> static __device__ float run(const uint64_t (&a)[O], int e) { return float(to_f64<O>(a, e)); }
  static __device__ float neg(float v) { return -v; } static __device__ float zero() { return 0.f; } };
template <> struct Conv<double2> { template <int O> static __device__ double2 run(const uint64_t (&a)[O], int e) { return to_dd<O>(a, e); }
  static __device__ double2 neg(double2 v) { return make_double2(-v.x, -v.y); } static __device__ double2 zero() { return make_double2(0., 0.); } };
template <> struct Conv<float3> { template <int O> static __device__ float3 run(const uint64_t (&a)[O], int e) { return to_tf<O>(a, e); }
  static __device__ float3 neg(float3 v) { return make_float3(-v.x, -v.y, -v.z); } static __device__ float3 zero() { return make_float3(0.f, 0.f, 0.f); } };
template <> struct Conv<float4> { template <int O> static __device__ float4 run(const uint64_t (&a)[O], int e) { return to_qf<O>(a, e); }
  static __device__ float4 neg(float4 v) { return make_float4(-v.x, -v.y, -v.z, -v.w); } static __device__ float4 zero() { return make_float4(0.f, 0.f, 0.f, 0.f); } };

template <typename R, bool CPLX> struct Elem { R re; };
template <typename R> struct Elem<R, true> { R re, im; };

// One 32 x 32 tile (ty <= tx) per CTA of 32 x 8 threads.  Phase 1 converts the entries with y <= x, writes
// them to G[y, x] (y fastest) and parks the conjugate in shared memory; phase 2 writes the parked values to
// G[x, y] (x fastest).  On the diagonal the mirrored value lands last, as it does in the reference
// (src/fp_i63tp_dequantize.cu:127), so the imaginary part of a diagonal entry is -0.0.
// SRC: where the integers come from -- the packed limbs (LimbSource) or, after a cross-rank sum, the summed
// slices (SliceSource): the post-collective epilogue then needs no pass that writes the limbs back.
template <int ORDER, typename R, bool CPLX, typename SRC>
__global__ void __launch_bounds__(256)
dequantize_kernel(int n, const SRC src, const int32_t* __restrict__ vexp, Elem<R, CPLX>* __restrict__ G, int64_t ldg) {
  using E = Elem<R, CPLX>;
  __shared__ E tile[32][33];
  // enumerate upper-triangle tile pairs: blockIdx.x -> (by <= bx)
  int bx = int((sqrtf(8.f * float(blockIdx.x) + 1.f) - 1.f) * 0.5f);
  while ((bx + 1) * (bx + 2) / 2 <= int(blockIdx.x)) ++bx;
  while (bx * (bx + 1) / 2 > int(blockIdx.x)) --bx;
  const int by = int(blockIdx.x) - bx * (bx + 1) / 2;
  const int lx = threadIdx.x, ly = threadIdx.y;

  const int y = by * 32 + lx;
  const int ey = y < n ? vexp[y] : INT_MAX;
#pragma unroll
  for (int j = ly; j < 32; j += 8) {
    const int x = bx * 32 + j;
    if (x < n && y <= x) {
      const int ex = vexp[x];
      E f;
      if (ex == INT_MAX || ey == INT_MAX) { f.re = Conv<R>::zero(); if constexpr (CPLX) f.im = Conv<R>::zero(); }
      else {
        const uint64_t idx = uint64_t(y) + (uint64_t(x) * (uint64_t(x) + 1)) / 2;
        uint64_t a[ORDER];
        src.template load<ORDER>(idx, 0, a);
        f.re = Conv<R>::template run<ORDER>(a, -(ex + ey));
        if constexpr (CPLX) {
          src.template load<ORDER>(idx, 1, a);
          f.im = Conv<R>::template run<ORDER>(a, -(ex + ey));
        }
      }
      G[y + int64_t(x) * ldg] = f;
      if constexpr (CPLX) f.im = Conv<R>::neg(f.im);
      tile[j][lx] = f;
    }
  }
  __syncthreads();
  // mirror: element (row x', column y') with x' = bx*32 + lx, y' = by*32 + j  takes conj of (y', x')
  const int xm = bx * 32 + lx;
#pragma unroll
  for (int j = ly; j < 32; j += 8) {
    const int ym = by * 32 + j;
    if (xm < n && ym <= xm) G[xm + int64_t(ym) * ldg] = tile[lx][j];
  }
}

template <int BLOCK, int ORDER, typename SRC>
__global__ void __launch_bounds__(BLOCK)
gram_range_kernel(int n, const SRC src, const int32_t* __restrict__ vexp, int32_t* __restrict__ out) {
  // key = bit length of the diagonal entry minus twice its column exponent (its true-scale magnitude);
  // the answer is the bit length at the largest key, the longer one on ties.
  __shared__ int s_key[BLOCK / 32], s_len[BLOCK / 32];
  int key = INT_MIN, len = 0;
  for (int i = threadIdx.x; i < n; i += BLOCK) {
    const int e = vexp[i];
    if (e == INT_MAX) continue;
    uint64_t d[ORDER];
    src.template load<ORDER>((uint64_t(i) * (uint64_t(i) + 3)) / 2, 0, d);
    int l = 64 - __clzll((long long)d[0]);
    if (ORDER > 1) { int ln = 127 - __clzll((long long)d[ORDER > 1 ? 1 : 0]); l = ln > 63 ? ln : l; }
    if (ORDER > 2) { int ln = 190 - __clzll((long long)d[ORDER > 2 ? 2 : 0]); l = ln > 126 ? ln : l; }
    const int k = l - (e + e);
    if (k > key || (k == key && l > len)) { key = k; len = l; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    int ok = __shfl_xor_sync(0xffffffffu, key, o), ol = __shfl_xor_sync(0xffffffffu, len, o);
    if (ok > key || (ok == key && ol > len)) { key = ok; len = ol; }
  }
  if ((threadIdx.x & 31) == 0) { s_key[threadIdx.x >> 5] = key; s_len[threadIdx.x >> 5] = len; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < BLOCK / 32; ++w) if (s_key[w] > key || (s_key[w] == key && s_len[w] > len)) { key = s_key[w]; len = s_len[w]; }
    *out = len;
  }
}

template <typename R, bool CPLX, typename SRC>
void run_dequantize(cudaStream_t stream, int n, int order, const SRC& src, const int32_t* vexp, void* G, int64_t ldg) {
  const int nb = (n + 31) / 32; const unsigned blocks = unsigned(int64_t(nb) * (nb + 1) / 2);
  dim3 threads(32, 8);
  auto* g = static_cast<Elem<R, CPLX>*>(G);
  switch (order) {
    case 1: dequantize_kernel<1, R, CPLX, SRC><<<blocks, threads, 0, stream>>>(n, src, vexp, g, ldg); break;
    case 2: dequantize_kernel<2, R, CPLX, SRC><<<blocks, threads, 0, stream>>>(n, src, vexp, g, ldg); break;
    case 3: dequantize_kernel<3, R, CPLX, SRC><<<blocks, threads, 0, stream>>>(n, src, vexp, g, ldg); break;
    default: break;
  }
}

template <typename SRC>
void range_from(cudaStream_t stream, int n, int order, const SRC& src, const int32_t* vexp, int32_t* bits_out) {
  count_launch();
  switch (order) {
    case 1: gram_range_kernel<512, 1, SRC><<<1, 512, 0, stream>>>(n, src, vexp, bits_out); break;
    case 2: gram_range_kernel<512, 2, SRC><<<1, 512, 0, stream>>>(n, src, vexp, bits_out); break;
    case 3: gram_range_kernel<512, 3, SRC><<<1, 512, 0, stream>>>(n, src, vexp, bits_out); break;
    default: break;
  }
  HYB_CUDA(cudaGetLastError());
}

template <typename SRC>
void dequantize_from(cudaStream_t stream, int n, int order, const SRC& src, const int32_t* vexp, hyacinPrecision_t gtype, void* G, int64_t ldg) {
  count_launch();
  switch (gtype) {
    case HYACIN_F64: run_dequantize<double, false>(stream, n, order, src, vexp, G, ldg); break;
    case HYACIN_F32: run_dequantize<float, false>(stream, n, order, src, vexp, G, ldg); break;
    case HYACIN_DD: run_dequantize<double2, false>(stream, n, order, src, vexp, G, ldg); break;
    case HYACIN_TF: run_dequantize<float3, false>(stream, n, order, src, vexp, G, ldg); break;
    case HYACIN_QF: run_dequantize<float4, false>(stream, n, order, src, vexp, G, ldg); break;
    case HYACIN_F64_COMPLEX: run_dequantize<double, true>(stream, n, order, src, vexp, G, ldg); break;
    case HYACIN_F32_COMPLEX: run_dequantize<float, true>(stream, n, order, src, vexp, G, ldg); break;
    case HYACIN_DD_COMPLEX: run_dequantize<double2, true>(stream, n, order, src, vexp, G, ldg); break;
    case HYACIN_TF_COMPLEX: run_dequantize<float3, true>(stream, n, order, src, vexp, G, ldg); break;
    case HYACIN_QF_COMPLEX: run_dequantize<float4, true>(stream, n, order, src, vexp, G, ldg); break;
    default: break;
  }
  HYB_CUDA(cudaGetLastError());
}

}  // namespace

void launch_gram_range(cudaStream_t stream, int n, int order, const uint64_t* C, const int32_t* vexp, int32_t* bits_out) {
  range_from(stream, n, order, LimbSource{C, (uint64_t(n) * n + n) / 2}, vexp, bits_out);
}
void launch_dequantize(cudaStream_t stream, int n, int order, const uint64_t* C, const int32_t* vexp,
                       hyacinPrecision_t gtype, void* G, int64_t ldg) {
  dequantize_from(stream, n, order, LimbSource{C, (uint64_t(n) * n + n) / 2}, vexp, gtype, G, ldg);
}
void launch_gram_range_slices(cudaStream_t stream, int n, int order, int ranks, const uint64_t* S, const int32_t* vexp, int32_t* bits_out) {
  range_from(stream, n, order, SliceSource{S, (uint64_t(n) * n + n) / 2, slice_plan(order, ranks)}, vexp, bits_out);
}
void launch_dequantize_slices(cudaStream_t stream, int n, int order, int ranks, const uint64_t* S, const int32_t* vexp,
                              hyacinPrecision_t gtype, void* G, int64_t ldg) {
  dequantize_from(stream, n, order, SliceSource{S, (uint64_t(n) * n + n) / 2, slice_plan(order, ranks)}, vexp, gtype, G, ldg);
}

}  // namespace hyb
