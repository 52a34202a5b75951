// Quantiser: floating-point rows of A -> centred int8 CRT residue planes, the operands of the Gram kernel.
//
// Contract (reference: src/quantize_limbs.cu:14-18 for the rounding, src/quantize_crt_real.cu:30-34,63-67 and
// src/quantize_crt_complex.cu:30-42 for the residue planes): q = rint_ties_even(a * 2^vexp[col]); each plane
// holds q mod m as an int8.  Any representative in [-128, 127] is admissible -- the Gram of residues is only
// ever used modulo m -- so this kernel stores ((q + 128) mod m) - 128.
//
// How the residue is formed (new): q is biased by 2^(8 nb - 1) so that its nb bytes are unsigned; then
//   q + 128 = bias_m + sum_b byte_b * (256^b mod m)   (mod m)
// is one dp4a per four bytes, and the sum (< 2^20) is reduced with a single exact multiply-high.
// Each thread converts eight consecutive rows of one column and stores one 64-bit word per plane, so loads
// and stores of a warp are contiguous 2 KiB / 256 B runs.
#include "hyb_internal.h"
#include "crt_tables.h"
#include <cuda_fp16.h>
#include <climits>
#include <cstdlib>
#include <cstring>

namespace hyb {
namespace {

// HYACIN_B200_QUANT_REDUCTION=int selects the integer reduction of the residue sums (multiply-high + multiply-subtract);
// the default is the float reduction described at quantize_crt_kernel.  Same integer Gram either way.
bool float_reduction() {
  static const bool on = [] { const char* v = std::getenv("HYACIN_B200_QUANT_REDUCTION"); return !(v && v[0] == 'i'); }();
  return on;
}

struct QuantConsts {
  uint32_t modulus[crt::kMaxModuli];
  uint32_t magic[crt::kMaxModuli];          // ceil(2^32 / m)
  uint32_t bias[crt::kMaxModuli];           // (128 - 2^(8 nb - 1)) mod m
  uint32_t weight[crt::kMaxModuli][3];      // 256^b mod m, four per word
  uint32_t fr_inv[crt::kMaxModuli], fr_add[crt::kMaxModuli];   // float reduction: bits of float(1 / m) and of the additive constant
};

struct QuantParams {
  const void* A; int64_t lda;               // elements
  const int32_t* vexp;
  int8_t* W; int64_t col_pitch, plane_pitch, part_pitch;   // bytes; part_pitch = rows per part (ldk)
  int rows, ldk, n, moduli, value_bytes;
  int op;                                   // 0: A is rows x n ('N'); 1: A is stored n x rows ('T'); 2: same, conjugated ('C')
  QuantConsts k;                            // kernel parameters live in the constant bank
};

template <typename T> __device__ __forceinline__ double load_as_double(const T* p);
template <> __device__ __forceinline__ double load_as_double<double>(const double* p) { return *p; }
template <> __device__ __forceinline__ double load_as_double<float>(const float* p) {
  float f = *p;
  // Single-precision subnormals count as zero, as in a flush-to-zero (fast-math) build of the reference.
  return fabsf(f) < 1.17549435e-38f ? 0.0 : double(f);
}
template <> __device__ __forceinline__ double load_as_double<__half>(const __half* p) { return double(__half2float(*p)); }

__device__ __forceinline__ double pow2(int e) { return __longlong_as_double((long long)(e + 1023) << 52); }

// rint(v) biased by 2^(8 nb - 1), as little-endian 32-bit words.  |v| <= 2^80.
template <int NW>
__device__ __forceinline__ void biased_words(double v, int value_bytes, bool negate, uint32_t (&w)[3]) {
  if (NW <= 2) {
    long long q = __double2ll_rn(v);                      // ties to even; |v| < 2^63 on this path
    if (negate) q = -q;
    unsigned long long b = (unsigned long long)q + (1ull << (8 * value_bytes - 1));
    w[0] = uint32_t(b); w[1] = uint32_t(b >> 32); w[2] = 0;
  } else {
    __int128 q;
    if (fabs(v) < 4611686018427387904.0) q = __double2ll_rn(v);
    else {                                                // already an integer: split exactly at 2^32
      double hi = trunc(v * 2.3283064365386963e-10), lo = v - hi * 4294967296.0;
      q = ((__int128)__double2ll_rn(hi) << 32) + (__int128)__double2ll_rn(lo);
    }
    if (negate) q = -q;
    unsigned __int128 b = (unsigned __int128)q + ((unsigned __int128)1 << (8 * value_bytes - 1));
    w[0] = uint32_t(b); w[1] = uint32_t(b >> 32); w[2] = uint32_t(b >> 64);
  }
}

// grid.x covers ldk / (kRows * blockDim.x) row groups, grid.y = columns.
// PARTS = 1: real input.  PARTS = 3: complex input -> planes (re, im, -re) stacked along K in each column.
// Each thread converts kRows = 8 consecutive rows of one column: the per-modulus constants are fetched once per
// eight values, the loads are 16-byte vectors when the column is 16-byte aligned, and every plane receives one
// 8-byte store per thread (256 contiguous bytes per warp).
constexpr int kRows = 8;
static_assert(crt::kModulus[0] == 256, "the quantiser takes the low byte as the residue of the first modulus");

template <typename T, int PARTS>
__device__ __forceinline__ void load_rows(const T* __restrict__ src, int valid, double s1, double s2, double (&v)[kRows][PARTS == 1 ? 1 : 2]) {
  constexpr int kReal = PARTS == 1 ? 1 : 2;
  constexpr int kCount = kRows * kReal;                 // scalars this thread reads
  constexpr int kVec = 16 / int(sizeof(T));             // scalars per 16-byte vector
  T raw[kCount];
  if (valid == kRows && (reinterpret_cast<uintptr_t>(src) & 15) == 0 && kCount % kVec == 0) {
#pragma unroll
    for (int q = 0; q < kCount / kVec; ++q) reinterpret_cast<uint4*>(raw)[q] = __ldg(reinterpret_cast<const uint4*>(src) + q);
  } else {
#pragma unroll
    for (int q = 0; q < kCount; ++q) raw[q] = (q / kReal) < valid ? src[q] : T(0);
  }
#pragma unroll
  for (int r = 0; r < kRows; ++r)
#pragma unroll
    for (int c = 0; c < kReal; ++c) v[r][c] = (load_as_double<T>(&raw[r * kReal + c]) * s1) * s2;
}

// Front end shared by both quantisers: which (column, first row) this thread converts and the kRows scaled
// values a * 2^vexp[col] of that column.
//   TRANS = false ('N'): grid.x covers ldk / (kRows * 256) row groups, grid.y = columns; a thread reads eight
//                        consecutive rows of its column straight from global memory (16-byte vectors).
//   TRANS = true ('T' / 'C'): the matrix is stored transposed, so consecutive COLUMNS are contiguous.  A block
//                        owns 64 rows x 32 columns, reads them with the column index on the fast lanes (256-byte
//                        runs), transposes through shared memory, and then every thread again holds eight
//                        consecutive rows of one column.  This replaces the transposed copy of the whole matrix
//                        that the reference makes before quantising (src/lra.cpp:63-65, src/matcopy.cu:36-43).
template <typename T, int PARTS, bool TRANS>
__device__ __forceinline__ bool fetch_scaled(const void* A, int64_t lda, const int32_t* __restrict__ vexp, int rows, int ldk, int n, int op,
                                             int& col, int& row0, double (&v)[kRows][PARTS == 1 ? 1 : 2]) {
  constexpr int kReal = PARTS == 1 ? 1 : 2;
  if constexpr (!TRANS) {
    col = blockIdx.y;
    row0 = (blockIdx.x * blockDim.x + threadIdx.x) * kRows;
    if (row0 >= ldk) return false;
    const int expon = vexp[col];
    // a * 2^expon as two exact scalings: the halves stay representable for every admissible exponent, and a
    // product that leaves the normal range on the way is far below 1/2 at the end, i.e. rounds to zero anyway.
    double s1 = 0.0, s2 = 0.0;
    if (expon != INT_MAX) { int h = expon / 2; s1 = pow2(h); s2 = pow2(expon - h); }
    const T* src = static_cast<const T*>(A) + (int64_t(col) * lda + row0) * kReal;
    int valid = rows - row0; valid = valid < 0 ? 0 : (valid > kRows ? kRows : valid);
    load_rows<T, PARTS>(src, valid, s1, s2, v);
    return true;
  } else {
    __shared__ double tile[kReal][64][33];
    const int i0 = blockIdx.x * 64, j0 = blockIdx.y * 32;
    const int tj = threadIdx.x & 31, ti = threadIdx.x >> 5;
    const T* base = static_cast<const T*>(A);
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const int i = i0 + ti + 8 * r, j = j0 + tj;
      const bool in = i < rows && j < n;
#pragma unroll
      for (int c = 0; c < kReal; ++c) {
        double x = in ? load_as_double<T>(base + (int64_t(j) + int64_t(i) * lda) * kReal + c) : 0.0;
        if (c == 1 && op == 2) x = -x;
        tile[c][ti + 8 * r][tj] = x;
      }
    }
    __syncthreads();
    const int cj = threadIdx.x >> 3, ci = threadIdx.x & 7;
    col = j0 + cj; row0 = i0 + ci * kRows;
    if (col >= n || row0 >= ldk) return false;
    const int expon = vexp[col];
    double s1 = 0.0, s2 = 0.0;
    if (expon != INT_MAX) { int h = expon / 2; s1 = pow2(h); s2 = pow2(expon - h); }
#pragma unroll
    for (int r = 0; r < kRows; ++r)
#pragma unroll
      for (int c = 0; c < kReal; ++c) v[r][c] = (tile[c][ci * kRows + r][cj] * s1) * s2;
    return true;
  }
}

// FR ("float reduction"): the quotient of the residue sum comes from the floating-point pipe instead of an integer
// multiply-high.  The dp4a accumulator starts at the bit pattern of a float X (>= 2^23, where floats are the
// integers), so its result read as a float IS X + t exactly; q_m = fmaf(X + t, 1/m, add) is 1.5 * 2^23 + q with q
// an integer within 1/2 + 6e-4 of t / m (the fused multiply-add rounds once, to unit spacing), and the low byte of
// (X + t) - bits(q_m) * m, one integer multiply-add, is r = t - q m in two's complement: X and bits(1.5 * 2^23) * m
// are multiples of 256.  |r| <= 127 for every t the quantiser can form; the constants come from
// gen_crt_tables.py, which verifies that for each modulus over the whole range of t.  Per residue: two dp4a, one
// fused multiply-add on either floating-point pipe, one integer multiply-add -- against two dp4a, a multiply-high
// (two passes of the integer pipe) and an integer multiply-add.
template <typename T, int NW, int PARTS, bool TRANS, bool FR>
__global__ void __launch_bounds__(256) quantize_crt_kernel(const __grid_constant__ QuantParams p) {
  constexpr int kReal = PARTS == 1 ? 1 : 2;
  int col, row0; double v[kRows][kReal];
  if (!fetch_scaled<T, PARTS, TRANS>(p.A, p.lda, p.vexp, p.rows, p.ldk, p.n, p.op, col, row0, v)) return;

  int8_t* dst = p.W + int64_t(col) * p.col_pitch + row0;
#pragma unroll
  for (int part = 0; part < PARTS; ++part) {
    uint32_t w[kRows][3];
#pragma unroll
    for (int r = 0; r < kRows; ++r) biased_words<NW>(v[r][part == 1 ? 1 : 0], p.value_bytes, part == 2, w[r]);
    int8_t* out = dst + int64_t(part) * p.part_pitch;
    // Unrolled over the whole table with a uniform guard: the per-modulus constants then sit at fixed offsets of
    // the parameter bank and feed the arithmetic instructions directly, with no loads and no loop bookkeeping.
#pragma unroll
    for (int i = 0; i < crt::kMaxModuli; ++i) {
      if (i >= p.moduli) break;
      const uint32_t bias = p.k.bias[i], w0 = p.k.weight[i][0], w1 = p.k.weight[i][1], w2 = p.k.weight[i][2];
      const uint32_t magic = p.k.magic[i], modulus = p.k.modulus[i];
      const uint32_t neg_modulus = 0u - modulus;      // t - q m as one multiply-add
      uint32_t r8[kRows];
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        // modulus 256 (first in the table): the bias 2^(8 nb - 1) is a multiple of 256 for nb > 1, so the low byte of the
        // biased value is the low byte of q itself, i.e. its centred residue (for nb = 1 the bias is 128 and is flipped
        // away below); the packing takes only that byte
        if (i == 0) { r8[r] = w[r][0]; continue; }
        uint32_t t = __dp4a(w[r][0], w0, bias);
        if (NW > 1) t = __dp4a(w[r][1], w1, t);
        if (NW > 2) t = __dp4a(w[r][2], w2, t);
        if constexpr (!FR) r8[r] = __umulhi(t, magic) * neg_modulus + t;           // exact: t * modulus < 2^32
        else r8[r] = __float_as_uint(fmaf(__uint_as_float(t), __uint_as_float(p.k.fr_inv[i]), __uint_as_float(p.k.fr_add[i]))) * neg_modulus + t;
      }
      // four residues per word by byte permutes (ALU pipe); the integer reduction leaves (q + 128) mod m and needs
      // -128 per byte, the float reduction and modulus 256 leave the centred residue itself
      const uint32_t flip = (i == 0 ? p.value_bytes == 1 : !FR) ? 0x80808080u : 0u;
      uint2 packed;
      packed.x = __byte_perm(__byte_perm(r8[0], r8[1], 0x0040), __byte_perm(r8[2], r8[3], 0x0040), 0x5410) ^ flip;
      packed.y = __byte_perm(__byte_perm(r8[4], r8[5], 0x0040), __byte_perm(r8[6], r8[7], 0x0040), 0x5410) ^ flip;
      *reinterpret_cast<uint2*>(out + int64_t(i) * p.plane_pitch) = packed;
    }
  }
}

// Real input in 'N' orientation, sixteen rows per thread: the per-modulus work of a thread that does not depend on the
// row (guard, plane address, constants moved to registers) is spread over twice as many values, and every plane receives
// one 16-byte store per thread (512 contiguous bytes per warp).  The kernel is bound by instruction issue inside the
// power-capped step, so instructions saved are time saved.
template <typename T, int NW, bool FR>
__global__ void __launch_bounds__(256) quantize_crt_rows16_kernel(const __grid_constant__ QuantParams p) {
  constexpr int kWide = 2 * kRows;
  const int col = blockIdx.y, row0 = (blockIdx.x * blockDim.x + threadIdx.x) * kWide;
  if (row0 >= p.ldk) return;
  const int expon = p.vexp[col];
  double s1 = 0.0, s2 = 0.0;
  if (expon != INT_MAX) { int h = expon / 2; s1 = pow2(h); s2 = pow2(expon - h); }
  const T* src = static_cast<const T*>(p.A) + (int64_t(col) * p.lda + row0);
  uint32_t w[kWide][3];
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    double v[kRows][1];
    int valid = p.rows - row0 - half * kRows; valid = valid < 0 ? 0 : (valid > kRows ? kRows : valid);
    load_rows<T, 1>(src + half * kRows, valid, s1, s2, v);
#pragma unroll
    for (int r = 0; r < kRows; ++r) biased_words<NW>(v[r][0], p.value_bytes, false, w[half * kRows + r]);
  }
  int8_t* out = p.W + int64_t(col) * p.col_pitch + row0;
#pragma unroll
  for (int i = 0; i < crt::kMaxModuli; ++i) {
    if (i >= p.moduli) break;
    const uint32_t bias = p.k.bias[i], w0 = p.k.weight[i][0], w1 = p.k.weight[i][1], w2 = p.k.weight[i][2];
    const uint32_t magic = p.k.magic[i], neg_modulus = 0u - p.k.modulus[i];
    uint32_t r8[kWide];
#pragma unroll
    for (int r = 0; r < kWide; ++r) {
      if (i == 0) { r8[r] = w[r][0]; continue; }              // modulus 256: see quantize_crt_kernel
      uint32_t t = __dp4a(w[r][0], w0, bias);
      if (NW > 1) t = __dp4a(w[r][1], w1, t);
      if (NW > 2) t = __dp4a(w[r][2], w2, t);
      if constexpr (!FR) r8[r] = __umulhi(t, magic) * neg_modulus + t;
      else r8[r] = __float_as_uint(fmaf(__uint_as_float(t), __uint_as_float(p.k.fr_inv[i]), __uint_as_float(p.k.fr_add[i]))) * neg_modulus + t;
    }
    const uint32_t flip = (i == 0 ? p.value_bytes == 1 : !FR) ? 0x80808080u : 0u;
    uint4 packed;
    packed.x = __byte_perm(__byte_perm(r8[0], r8[1], 0x0040), __byte_perm(r8[2], r8[3], 0x0040), 0x5410) ^ flip;
    packed.y = __byte_perm(__byte_perm(r8[4], r8[5], 0x0040), __byte_perm(r8[6], r8[7], 0x0040), 0x5410) ^ flip;
    packed.z = __byte_perm(__byte_perm(r8[8], r8[9], 0x0040), __byte_perm(r8[10], r8[11], 0x0040), 0x5410) ^ flip;
    packed.w = __byte_perm(__byte_perm(r8[12], r8[13], 0x0040), __byte_perm(r8[14], r8[15], 0x0040), 0x5410) ^ flip;
    *reinterpret_cast<uint4*>(out + int64_t(i) * p.plane_pitch) = packed;
  }
}

// ---- complex input, moduli with a square root of -1 -------------------------------------------------------------
// Every modulus m of the crt2m set has an iota with iota^2 = -1 (mod m), so the complex value re + i im is carried by
// the two residues p = re - iota im and q = re + iota im, and P^T Q = Re(A^H A) + iota Im(A^H A) (mod m) entry by entry:
// one integer product per pair of entries instead of the two that separate real and imaginary planes need
// (reference: src/quantize_crt_complex.cu:30-42, with its own table).  iota is folded into the byte weights of
// the imaginary part, so p and q are each four dp4a (for values of up to 8 bytes) and one reduction:
//   p + 128 = bias_p + sum_b re_b (256^b mod m) + sum_b im_b (-iota 256^b mod m)        (sum < 2^22)
// Planes: W[modulus][column][part * ldk + row], part 0 = p, part 1 = q.
struct Quant2mConsts {
  uint32_t modulus[crt2m::kMaxModuli], magic[crt2m::kMaxModuli], bias_p[crt2m::kMaxModuli], bias_q[crt2m::kMaxModuli];
  uint32_t w_re[crt2m::kMaxModuli][3], w_im_p[crt2m::kMaxModuli][3], w_im_q[crt2m::kMaxModuli][3];
  uint32_t fr_inv[crt2m::kMaxModuli], fr_add[crt2m::kMaxModuli];
};
struct Quant2mParams {
  const void* A; int64_t lda; const int32_t* vexp;
  int8_t* W; int64_t col_pitch, plane_pitch, part_pitch;
  int rows, ldk, n, moduli, value_bytes, op;
  Quant2mConsts k;
};

template <typename T, int NW, bool TRANS, bool FR>
__global__ void __launch_bounds__(256) quantize_crt2m_kernel(const __grid_constant__ Quant2mParams p) {
  int col, row0; double v[kRows][2];
  if (!fetch_scaled<T, 3, TRANS>(p.A, p.lda, p.vexp, p.rows, p.ldk, p.n, p.op, col, row0, v)) return;
  uint32_t wr[kRows][3], wi[kRows][3];
#pragma unroll
  for (int r = 0; r < kRows; ++r) { biased_words<NW>(v[r][0], p.value_bytes, false, wr[r]); biased_words<NW>(v[r][1], p.value_bytes, false, wi[r]); }
  int8_t* out = p.W + int64_t(col) * p.col_pitch + row0;
#pragma unroll
  for (int i = 0; i < crt2m::kMaxModuli; ++i) {
    if (i >= p.moduli) break;
    const uint32_t magic = p.k.magic[i], modulus = p.k.modulus[i];
    uint32_t rp[kRows], rq[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      uint32_t base = __dp4a(wr[r][0], p.k.w_re[i][0], 0u);
      if (NW > 1) base = __dp4a(wr[r][1], p.k.w_re[i][1], base);
      if (NW > 2) base = __dp4a(wr[r][2], p.k.w_re[i][2], base);
      uint32_t tp = __dp4a(wi[r][0], p.k.w_im_p[i][0], base + p.k.bias_p[i]), tq = __dp4a(wi[r][0], p.k.w_im_q[i][0], base + p.k.bias_q[i]);
      if (NW > 1) { tp = __dp4a(wi[r][1], p.k.w_im_p[i][1], tp); tq = __dp4a(wi[r][1], p.k.w_im_q[i][1], tq); }
      if (NW > 2) { tp = __dp4a(wi[r][2], p.k.w_im_p[i][2], tp); tq = __dp4a(wi[r][2], p.k.w_im_q[i][2], tq); }
      if constexpr (!FR) {
        rp[r] = tp - __umulhi(tp, magic) * modulus;                     // exact: t < 2^23, t * modulus < 2^32
        rq[r] = tq - __umulhi(tq, magic) * modulus;
      } else {
        const float inv = __uint_as_float(p.k.fr_inv[i]), add = __uint_as_float(p.k.fr_add[i]);
        rp[r] = tp - __float_as_uint(fmaf(__uint_as_float(tp), inv, add)) * modulus;
        rq[r] = tq - __float_as_uint(fmaf(__uint_as_float(tq), inv, add)) * modulus;
      }
    }
    constexpr uint32_t flip = FR ? 0u : 0x80808080u;
    uint2 pp, qq;
    pp.x = __byte_perm(__byte_perm(rp[0], rp[1], 0x0040), __byte_perm(rp[2], rp[3], 0x0040), 0x5410) ^ flip;
    pp.y = __byte_perm(__byte_perm(rp[4], rp[5], 0x0040), __byte_perm(rp[6], rp[7], 0x0040), 0x5410) ^ flip;
    qq.x = __byte_perm(__byte_perm(rq[0], rq[1], 0x0040), __byte_perm(rq[2], rq[3], 0x0040), 0x5410) ^ flip;
    qq.y = __byte_perm(__byte_perm(rq[4], rq[5], 0x0040), __byte_perm(rq[6], rq[7], 0x0040), 0x5410) ^ flip;
    *reinterpret_cast<uint2*>(out + int64_t(i) * p.plane_pitch) = pp;
    *reinterpret_cast<uint2*>(out + int64_t(i) * p.plane_pitch + p.part_pitch) = qq;
  }
}

template <typename T, bool FR>
void launch_2m_typed(cudaStream_t stream, const Quant2mParams& p) {
  const int nw = (p.value_bytes + 3) / 4;
  if (p.op == 0) {
    dim3 grid(unsigned((p.ldk / kRows + 255) / 256), unsigned(p.n));
    if (nw <= 1) quantize_crt2m_kernel<T, 1, false, FR><<<grid, 256, 0, stream>>>(p);
    else if (nw == 2) quantize_crt2m_kernel<T, 2, false, FR><<<grid, 256, 0, stream>>>(p);
    else quantize_crt2m_kernel<T, 3, false, FR><<<grid, 256, 0, stream>>>(p);
  } else {
    dim3 grid(unsigned(p.ldk / 64), unsigned((p.n + 31) / 32));
    if (nw <= 1) quantize_crt2m_kernel<T, 1, true, FR><<<grid, 256, 0, stream>>>(p);
    else if (nw == 2) quantize_crt2m_kernel<T, 2, true, FR><<<grid, 256, 0, stream>>>(p);
    else quantize_crt2m_kernel<T, 3, true, FR><<<grid, 256, 0, stream>>>(p);
  }
}

// ---- balanced base-256 digits ("limbs") --------------------------------------------------------------------
// q + sum_k 128 * 256^k has unsigned bytes b_k with q = sum_k (b_k - 128) 256^k, so digit k is simply byte k with
// its top bit flipped: no carries.  `order` digits hold every |q| <= 2^(8 order - 2).
struct LimbParams {
  const void* A; int64_t lda; const int32_t* vexp;
  int8_t* W; int64_t col_pitch, plane_pitch, part_pitch;
  int rows, ldk, n, order, op;
};

template <typename T, int NW, int PARTS, bool TRANS>
__global__ void __launch_bounds__(256) quantize_limbs_kernel(const __grid_constant__ LimbParams p) {
  constexpr int kReal = PARTS == 1 ? 1 : 2;
  int col, row0; double v[kRows][kReal];
  if (!fetch_scaled<T, PARTS, TRANS>(p.A, p.lda, p.vexp, p.rows, p.ldk, p.n, p.op, col, row0, v)) return;
  // bias words: 0x80 in each of the `order` low bytes
  uint32_t bias[3];
#pragma unroll
  for (int w = 0; w < 3; ++w) { const int nb = p.order - 4 * w; bias[w] = nb >= 4 ? 0x80808080u : (nb <= 0 ? 0u : (0x80808080u >> (8 * (4 - nb)))); }
  int8_t* dst = p.W + int64_t(col) * p.col_pitch + row0;
#pragma unroll
  for (int part = 0; part < PARTS; ++part) {
    uint32_t w[kRows][3];
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      const double x = v[r][part == 1 ? 1 : 0];
      if (NW <= 2) {
        long long q = __double2ll_rn(x); if (part == 2) q = -q;
        const unsigned long long b = (unsigned long long)q + ((unsigned long long)bias[1] << 32 | bias[0]);
        w[r][0] = uint32_t(b); w[r][1] = uint32_t(b >> 32); w[r][2] = 0;
      } else {
        __int128 q;
        if (fabs(x) < 4611686018427387904.0) q = __double2ll_rn(x);
        else { const double hi = trunc(x * 2.3283064365386963e-10), lo = x - hi * 4294967296.0; q = ((__int128)__double2ll_rn(hi) << 32) + (__int128)__double2ll_rn(lo); }
        if (part == 2) q = -q;
        const unsigned __int128 b = (unsigned __int128)q + (((unsigned __int128)bias[2] << 64) | ((unsigned __int128)bias[1] << 32) | bias[0]);
        w[r][0] = uint32_t(b); w[r][1] = uint32_t(b >> 32); w[r][2] = uint32_t(b >> 64);
      }
    }
    int8_t* out = dst + int64_t(part) * p.part_pitch;
#pragma unroll
    for (int k = 0; k < 4 * NW; ++k) {
      if (k < p.order) {
        uint32_t d[kRows];
#pragma unroll
        for (int r = 0; r < kRows; ++r) d[r] = w[r][k >> 2] >> (8 * (k & 3));
        uint2 packed;
        packed.x = __byte_perm(__byte_perm(d[0], d[1], 0x0040), __byte_perm(d[2], d[3], 0x0040), 0x5410) ^ 0x80808080u;
        packed.y = __byte_perm(__byte_perm(d[4], d[5], 0x0040), __byte_perm(d[6], d[7], 0x0040), 0x5410) ^ 0x80808080u;
        *reinterpret_cast<uint2*>(out + int64_t(k) * p.plane_pitch) = packed;
      }
    }
  }
}

template <typename T, int PARTS>
void launch_limbs_typed(cudaStream_t stream, const LimbParams& p) {
  const int nw = (p.order + 3) / 4;
  if (p.op == 0) {
    dim3 grid(unsigned((p.ldk / kRows + 255) / 256), unsigned(p.n));
    if (nw <= 1) quantize_limbs_kernel<T, 1, PARTS, false><<<grid, 256, 0, stream>>>(p);
    else if (nw == 2) quantize_limbs_kernel<T, 2, PARTS, false><<<grid, 256, 0, stream>>>(p);
    else quantize_limbs_kernel<T, 3, PARTS, false><<<grid, 256, 0, stream>>>(p);
  } else {
    dim3 grid(unsigned(p.ldk / 64), unsigned((p.n + 31) / 32));
    if (nw <= 1) quantize_limbs_kernel<T, 1, PARTS, true><<<grid, 256, 0, stream>>>(p);
    else if (nw == 2) quantize_limbs_kernel<T, 2, PARTS, true><<<grid, 256, 0, stream>>>(p);
    else quantize_limbs_kernel<T, 3, PARTS, true><<<grid, 256, 0, stream>>>(p);
  }
}

template <typename T, int PARTS, bool FR>
void launch_typed_fr(cudaStream_t stream, const QuantParams& p) {
  const int nw = (p.value_bytes + 3) / 4;
  static const bool rows8 = [] { const char* e = std::getenv("HYACIN_B200_QUANT_ROWS"); return e && e[0] == '8'; }();      // diagnosis: A/B the two kernels
  if (PARTS == 1 && p.op == 0 && !rows8 && p.ldk % (2 * kRows) == 0 && (reinterpret_cast<uintptr_t>(p.W) & 15) == 0 && p.col_pitch % 16 == 0) {
    dim3 grid(unsigned((p.ldk / (2 * kRows) + 255) / 256), unsigned(p.n));
    if (nw <= 1) quantize_crt_rows16_kernel<T, 1, FR><<<grid, 256, 0, stream>>>(p);
    else if (nw == 2) quantize_crt_rows16_kernel<T, 2, FR><<<grid, 256, 0, stream>>>(p);
    else quantize_crt_rows16_kernel<T, 3, FR><<<grid, 256, 0, stream>>>(p);
    return;
  }
  if (p.op == 0) {
    dim3 grid(unsigned((p.ldk / kRows + 255) / 256), unsigned(p.n));
    if (nw <= 1) quantize_crt_kernel<T, 1, PARTS, false, FR><<<grid, 256, 0, stream>>>(p);
    else if (nw == 2) quantize_crt_kernel<T, 2, PARTS, false, FR><<<grid, 256, 0, stream>>>(p);
    else quantize_crt_kernel<T, 3, PARTS, false, FR><<<grid, 256, 0, stream>>>(p);
  } else {
    dim3 grid(unsigned(p.ldk / 64), unsigned((p.n + 31) / 32));
    if (nw <= 1) quantize_crt_kernel<T, 1, PARTS, true, FR><<<grid, 256, 0, stream>>>(p);
    else if (nw == 2) quantize_crt_kernel<T, 2, PARTS, true, FR><<<grid, 256, 0, stream>>>(p);
    else quantize_crt_kernel<T, 3, PARTS, true, FR><<<grid, 256, 0, stream>>>(p);
  }
}

template <typename T, int PARTS>
void launch_typed(cudaStream_t stream, QuantParams& p) {
  if (float_reduction()) {
    for (int i = 1; i < crt::kMaxModuli; ++i) {
      // residue of q itself (drop the +128 of the integer scheme), summed on top of the bits of the float X
      const uint32_t m = p.k.modulus[i];
      p.k.bias[i] = crt::kFrBase[i] + (p.k.bias[i] + m - 128u % m) % m;
      p.k.fr_inv[i] = crt::kFrInv[i]; p.k.fr_add[i] = crt::kFrAdd[i];
    }
    launch_typed_fr<T, PARTS, true>(stream, p);
  } else launch_typed_fr<T, PARTS, false>(stream, p);
}

}  // namespace

void launch_quantize_crt(cudaStream_t stream, hyacinPrecision_t atype, int rows, int n, const void* A, int64_t lda,
                         const int32_t* vexp, const CrtPlan& plan, int8_t* W, int64_t ldk, char op) {
  const int cplx = is_complex(atype);
  if (plan.two_m) {
    if (!cplx || plan.moduli > crt2m::kMaxModuli) return;
    Quant2mParams q;
    const bool fr = float_reduction();
    for (int i = 0; i < crt2m::kMaxModuli; ++i) {
      const uint32_t m = crt2m::kModulus[i];
      q.k.modulus[i] = m; q.k.magic[i] = crt2m::kMagicCeil[i];
      q.k.bias_p[i] = crt2m::kBiasP[i][plan.value_bytes - 1]; q.k.bias_q[i] = crt2m::kBiasQ[i][plan.value_bytes - 1];
      q.k.fr_inv[i] = crt2m::kFrInv[i]; q.k.fr_add[i] = crt2m::kFrAdd[i];
      if (fr) {      // residues of p and q themselves, summed on top of the bits of the float X
        q.k.bias_p[i] = crt2m::kFrBase[i] + (q.k.bias_p[i] + m - 128u % m) % m;
        q.k.bias_q[i] = crt2m::kFrBase[i] + (q.k.bias_q[i] + m - 128u % m) % m;
      }
      for (int w = 0; w < 3; ++w) { q.k.w_re[i][w] = crt2m::kByteWeight[i][w]; q.k.w_im_p[i][w] = crt2m::kByteWeightMinusI[i][w]; q.k.w_im_q[i][w] = crt2m::kByteWeightPlusI[i][w]; }
    }
    q.A = A; q.lda = lda; q.vexp = vexp; q.W = W;
    q.part_pitch = ldk; q.col_pitch = ldk * 2; q.plane_pitch = q.col_pitch * n;
    q.rows = rows; q.ldk = int(ldk); q.n = n; q.moduli = plan.moduli; q.value_bytes = plan.value_bytes;
    q.op = op == 'T' ? 1 : op == 'C' ? 2 : 0;
    ProfileScope prof(stream, KernelKind::Quantize);
    count_launch();
    switch (int(atype)) {
      case HYACIN_F64_COMPLEX: fr ? launch_2m_typed<double, true>(stream, q) : launch_2m_typed<double, false>(stream, q); break;
      case HYACIN_F32_COMPLEX: fr ? launch_2m_typed<float, true>(stream, q) : launch_2m_typed<float, false>(stream, q); break;
      default: fr ? launch_2m_typed<__half, true>(stream, q) : launch_2m_typed<__half, false>(stream, q); break;
    }
    HYB_CUDA(cudaGetLastError());
    return;
  }
  QuantParams p;
  for (int i = 0; i < crt::kMaxModuli; ++i) {   // the bias depends on the byte width of the values
    p.k.modulus[i] = crt::kModulus[i]; p.k.magic[i] = crt::kMagicCeil[i];
    p.k.bias[i] = crt::kPow2Bias[i][plan.value_bytes - 1]; p.k.fr_inv[i] = p.k.fr_add[i] = 0u;
    for (int w = 0; w < 3; ++w) p.k.weight[i][w] = crt::kByteWeight[i][w];
  }
  p.A = A; p.lda = lda; p.vexp = vexp; p.W = W;
  p.part_pitch = ldk; p.col_pitch = ldk * (cplx ? 3 : 1); p.plane_pitch = p.col_pitch * n;
  p.rows = rows; p.ldk = int(ldk); p.n = n; p.moduli = plan.moduli; p.value_bytes = plan.value_bytes;
  p.op = op == 'T' ? 1 : op == 'C' ? 2 : 0;
  ProfileScope prof(stream, KernelKind::Quantize);
  count_launch();
  switch (int(atype)) {
    case HYACIN_F64: launch_typed<double, 1>(stream, p); break;
    case HYACIN_F32: launch_typed<float, 1>(stream, p); break;
    case HYACIN_F16: launch_typed<__half, 1>(stream, p); break;
    case HYACIN_F64_COMPLEX: launch_typed<double, 3>(stream, p); break;
    case HYACIN_F32_COMPLEX: launch_typed<float, 3>(stream, p); break;
    case HYACIN_F16_COMPLEX: launch_typed<__half, 3>(stream, p); break;
    default: break;
  }
  HYB_CUDA(cudaGetLastError());
}

void launch_quantize_limbs(cudaStream_t stream, hyacinPrecision_t atype, int rows, int n, const void* A, int64_t lda,
                           const int32_t* vexp, int order, int8_t* W, int64_t ldk, char op) {
  if (order < 1 || order > crt::kMaxBytes) return;
  const int cplx = is_complex(atype);
  LimbParams p;
  p.A = A; p.lda = lda; p.vexp = vexp; p.W = W;
  p.part_pitch = ldk; p.col_pitch = ldk * (cplx ? 3 : 1); p.plane_pitch = p.col_pitch * n;
  p.rows = rows; p.ldk = int(ldk); p.n = n; p.order = order; p.op = op == 'T' ? 1 : op == 'C' ? 2 : 0;
  ProfileScope prof(stream, KernelKind::Quantize);
  count_launch();
  switch (int(atype)) {
    case HYACIN_F64: launch_limbs_typed<double, 1>(stream, p); break;
    case HYACIN_F32: launch_limbs_typed<float, 1>(stream, p); break;
    case HYACIN_F16: launch_limbs_typed<__half, 1>(stream, p); break;
    case HYACIN_F64_COMPLEX: launch_limbs_typed<double, 3>(stream, p); break;
    case HYACIN_F32_COMPLEX: launch_limbs_typed<float, 3>(stream, p); break;
    case HYACIN_F16_COMPLEX: launch_limbs_typed<__half, 3>(stream, p); break;
    default: break;
  }
  HYB_CUDA(cudaGetLastError());
}

}  // namespace hyb
