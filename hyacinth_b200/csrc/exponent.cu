// Column-exponent pass of the quantized Gram: one streaming read of A, 128-bit loads, integer reductions.
//
// Behaviour follows the reference's src/fp_exponent.cu (vector_exponent_batch_kernel :25-35,
// vector_exponent_reduc_kernel :37-43, vector_range_batch_kernel :67-73); the kernels are new:
//   * the maximum of |a| is taken on the IEEE bit patterns (monotone for non-negative finite values), so the
//     reduction is integer-only and NaNs drop out like they do under fmax;
//   * every CTA folds its partial result straight into the per-segment row and the global row of the exponent
//     table with atomicMin -- integer min is order independent, so the table is deterministic and the
//     reference's second (reduction) kernel disappears;
//   * complex columns are scanned as twice as many reals, which is max(|re|, |im|).
#include "hyb_internal.h"
#include <cuda_fp16.h>
#include <climits>
#include <algorithm>

namespace hyb {
namespace {

constexpr int kWarpsPerCta = 8;
constexpr int kRowsPerCta = 4096;     // real elements scanned per warp and CTA

__global__ void fill_i32_kernel(int32_t* p, int64_t count, int32_t value) {
  int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < count) p[i] = value;
}

template <typename T> struct Bits;
template <> struct Bits<double> {
  using word = unsigned long long;
  static __device__ __forceinline__ word abs_bits(double v) {
    word b = (word)__double_as_longlong(v) & 0x7fffffffffffffffull;
    return b > 0x7ff0000000000000ull ? 0ull : b;            // NaN contributes nothing
  }
  // Exponent e with value = f * 2^e, f in [1/2, 1); INT_MAX for zero and subnormal maxima.
  static __device__ __forceinline__ int frexp_exp(word b) { int be = int(b >> 52); return be == 0 ? INT_MAX : be - 1022; }
};
template <> struct Bits<float> {
  using word = unsigned int;
  static __device__ __forceinline__ word abs_bits(float v) {
    word b = __float_as_uint(v) & 0x7fffffffu;
    return b > 0x7f800000u ? 0u : b;
  }
  static __device__ __forceinline__ int frexp_exp(word b) { int be = int(b >> 23); return be == 0 ? INT_MAX : be - 126; }
};
template <> struct Bits<__half> {
  using word = unsigned int;
  static __device__ __forceinline__ word abs_bits(__half v) {
    word b = (word)__half_as_ushort(v) & 0x7fffu;
    return b > 0x7c00u ? 0u : b;
  }
  // A half maximum is compared as a float: half subnormals are float normals (only zero gives INT_MAX).
  static __device__ __forceinline__ int frexp_exp(word b) {
    float f = __half2float(__ushort_as_half((unsigned short)b));
    return Bits<float>::frexp_exp(__float_as_uint(f));
  }
};

template <typename W> __device__ __forceinline__ W warp_max(W v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { W other = __shfl_xor_sync(0xffffffffu, v, o); v = other > v ? other : v; }
  return v;
}

// grid.x = batches * blocks_per_segment, grid.y = ceil(N / kWarpsPerCta).
// `seg_len`, `last_len`, `ld` count REAL elements (already doubled for complex input).
template <typename T>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
column_exponent_kernel(const T* __restrict__ A, int64_t ld, int64_t seg_len, int64_t last_len, int batches,
                       int blocks_per_segment, int n, int u, int32_t* __restrict__ vexp) {
  using B = Bits<T>; using W = typename B::word;
  constexpr int kVec = 16 / sizeof(T);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = blockIdx.y * kWarpsPerCta + warp;
  const int seg = blockIdx.x / blocks_per_segment, blk = blockIdx.x % blocks_per_segment;
  if (col >= n) return;
  const int64_t len = (seg + 1 == batches) ? last_len : seg_len;
  int64_t r0 = int64_t(blk) * kRowsPerCta, r1 = r0 + kRowsPerCta; if (r1 > len) r1 = len;
  if (r0 >= r1) return;
  const T* p = A + int64_t(col) * ld + int64_t(seg) * seg_len;
  W best = 0;
  // head: scalar until the address is 16-byte aligned
  int64_t i = r0;
  int64_t mis = (reinterpret_cast<uintptr_t>(p + i) & 15) / sizeof(T);
  int64_t head = mis ? (kVec - mis) : 0; if (head > r1 - i) head = r1 - i;
  if (lane < head) { W b = B::abs_bits(p[i + lane]); best = b > best ? b : best; }
  i += head;
  // body: one 16-byte load per lane per step, four steps in flight
  const int64_t body_end = i + ((r1 - i) / kVec) * kVec;
  for (int64_t k = i + int64_t(lane) * kVec; k < body_end; k += 4 * 32 * kVec) {
    uint4 v[4];
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      int64_t kk = k + int64_t(s) * 32 * kVec;
      v[s] = kk < body_end ? __ldg(reinterpret_cast<const uint4*>(p + kk)) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const T* e = reinterpret_cast<const T*>(&v[s]);
#pragma unroll
      for (int t = 0; t < kVec; ++t) { W b = B::abs_bits(e[t]); best = b > best ? b : best; }
    }
  }
  // tail
  for (int64_t k = body_end + lane; k < r1; k += 32) { W b = B::abs_bits(p[k]); best = b > best ? b : best; }
  best = warp_max(best);
  if (lane == 0) {
    int e = B::frexp_exp(best);
    if (e != INT_MAX) {                    // tables start at INT_MAX, so zero blocks have nothing to add
      int m = u - e;
      atomicMin(&vexp[int64_t(1 + seg) * n + col], m);
      atomicMin(&vexp[col], m);
    }
  }
}

// Transposed input ('T' / 'C'): the matrix is stored n x rows, so the n entries of one row of op(A) are
// contiguous.  Threads map to consecutive real columns (complex columns count twice, which again gives
// max(|re|, |im|)), each walks down kRowsPerCtaT rows of one segment keeping its own maximum, and folds it
// into the table with atomicMin -- no cross-thread reduction at all.
constexpr int kRowsPerCtaT = 2048;

template <typename T>
__global__ void __launch_bounds__(256)
column_exponent_transposed_kernel(const T* __restrict__ A, int64_t ld, int mul, int64_t seg_rows, int64_t last_rows, int batches,
                                  int blocks_per_segment, int n, int u, int32_t* __restrict__ vexp) {
  using B = Bits<T>; using W = typename B::word;
  const int jj = blockIdx.y * 256 + threadIdx.x;                 // real column index in [0, mul * n)
  const int seg = blockIdx.x / blocks_per_segment, blk = blockIdx.x % blocks_per_segment;
  if (jj >= mul * n) return;
  const int64_t len = (seg + 1 == batches) ? last_rows : seg_rows;
  int64_t r0 = int64_t(blk) * kRowsPerCtaT, r1 = r0 + kRowsPerCtaT; if (r1 > len) r1 = len;
  if (r0 >= r1) return;
  const T* p = A + jj + (int64_t(seg) * seg_rows + r0) * ld;
  W best = 0;
  int64_t i = r0;
  for (; i + 4 <= r1; i += 4) {
    const T a0 = p[0], a1 = p[ld], a2 = p[2 * ld], a3 = p[3 * ld];
    p += 4 * ld;
    W b0 = B::abs_bits(a0), b1 = B::abs_bits(a1), b2 = B::abs_bits(a2), b3 = B::abs_bits(a3);
    b0 = b0 > b1 ? b0 : b1; b2 = b2 > b3 ? b2 : b3; b0 = b0 > b2 ? b0 : b2; best = b0 > best ? b0 : best;
  }
  for (; i < r1; ++i) { const W b = B::abs_bits(*p); p += ld; best = b > best ? b : best; }
  const int e = B::frexp_exp(best);
  if (e != INT_MAX) {
    const int m = u - e, col = jj / mul;
    atomicMin(&vexp[int64_t(1 + seg) * n + col], m);
    atomicMin(&vexp[col], m);
  }
}

__global__ void __launch_bounds__(256)
vector_range_kernel(int n, int u, const int32_t* __restrict__ vexp, int32_t* __restrict__ seg_u) {
  __shared__ int32_t warp_best[8];
  const int32_t* mexp = vexp + int64_t(1 + blockIdx.x) * n;
  int32_t best = INT_MIN;
  for (int j = threadIdx.x; j < n; j += blockDim.x) {
    int32_t e = mexp[j];
    if (e < INT_MAX) { int32_t d = vexp[j] - e; best = d > best ? d : best; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { int32_t other = __shfl_xor_sync(0xffffffffu, best, o); best = other > best ? other : best; }
  if ((threadIdx.x & 31) == 0) warp_best[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) best = warp_best[w] > best ? warp_best[w] : best;
    seg_u[blockIdx.x] = best == INT_MIN ? INT_MIN : u + best;
  }
}

template <typename T>
void run_exponents(cudaStream_t stream, int cplx, int batches, int seg_m, int last_m, int n, const void* A, int64_t lda,
                   int u, int32_t* vexp) {
  const int64_t mul = cplx ? 2 : 1;
  int64_t seg_len = int64_t(seg_m) * mul, last_len = int64_t(last_m) * mul;
  int64_t longest = batches > 1 ? (seg_len > last_len ? seg_len : last_len) : last_len;
  int blocks_per_segment = int((longest + kRowsPerCta - 1) / kRowsPerCta);
  if (blocks_per_segment < 1) blocks_per_segment = 1;
  dim3 grid(unsigned(int64_t(batches) * blocks_per_segment), unsigned((n + kWarpsPerCta - 1) / kWarpsPerCta));
  column_exponent_kernel<T><<<grid, kWarpsPerCta * 32, 0, stream>>>(static_cast<const T*>(A), lda * mul, seg_len, last_len,
                                                                     batches, blocks_per_segment, n, u, vexp);
}

template <typename T>
void run_exponents_transposed(cudaStream_t stream, int cplx, int batches, int seg_m, int last_m, int n, const void* A, int64_t lda,
                              int u, int32_t* vexp) {
  const int mul = cplx ? 2 : 1;
  const int64_t longest = batches > 1 ? std::max(seg_m, last_m) : last_m;
  int blocks_per_segment = int((longest + kRowsPerCtaT - 1) / kRowsPerCtaT); if (blocks_per_segment < 1) blocks_per_segment = 1;
  dim3 grid(unsigned(int64_t(batches) * blocks_per_segment), unsigned((int64_t(n) * mul + 255) / 256));
  column_exponent_transposed_kernel<T><<<grid, 256, 0, stream>>>(static_cast<const T*>(A), lda * mul, mul, seg_m, last_m, batches,
                                                                 blocks_per_segment, n, u, vexp);
}

}  // namespace

void launch_column_exponents(cudaStream_t stream, hyacinPrecision_t atype, int batches, int seg_m, int last_m, int n,
                             const void* A, int64_t lda, int u, int32_t* vexp, char op) {
  const bool empty = batches <= 0 || u < 0;
  // Without rows or with a negative bit budget only the global row is defined (all columns "zero").
  int64_t count = empty ? int64_t(n) : int64_t(batches + 1) * n;
  fill_i32_kernel<<<unsigned((count + 255) / 256), 256, 0, stream>>>(vexp, count, INT_MAX);
  count_launch();
  if (empty) return;
  count_launch();
  const int cplx = is_complex(atype);
  if (op == 'T' || op == 'C') {
    switch (base_type(atype)) {
      case HYACIN_F64: run_exponents_transposed<double>(stream, cplx, batches, seg_m, last_m, n, A, lda, u, vexp); break;
      case HYACIN_F32: run_exponents_transposed<float>(stream, cplx, batches, seg_m, last_m, n, A, lda, u, vexp); break;
      case HYACIN_F16: run_exponents_transposed<__half>(stream, cplx, batches, seg_m, last_m, n, A, lda, u, vexp); break;
      default: break;
    }
    HYB_CUDA(cudaGetLastError());
    return;
  }
  switch (base_type(atype)) {
    case HYACIN_F64: run_exponents<double>(stream, cplx, batches, seg_m, last_m, n, A, lda, u, vexp); break;
    case HYACIN_F32: run_exponents<float>(stream, cplx, batches, seg_m, last_m, n, A, lda, u, vexp); break;
    case HYACIN_F16: run_exponents<__half>(stream, cplx, batches, seg_m, last_m, n, A, lda, u, vexp); break;
    default: break;
  }
  HYB_CUDA(cudaGetLastError());
}

void launch_vector_range(cudaStream_t stream, int batches, int n, int u, const int32_t* vexp, int32_t* seg_u) {
  if (batches <= 0) return;
  vector_range_kernel<<<batches, 256, 0, stream>>>(n, u, vexp, seg_u);
  count_launch();
  HYB_CUDA(cudaGetLastError());
}

}  // namespace hyb
