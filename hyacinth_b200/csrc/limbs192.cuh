// 192-bit two's-complement helpers and the packed 63-bit-limb format of the integer Gram
// (value = a0 + a1 2^63 + a2 2^126, lower limbs in [0, 2^63), last limb a signed 64-bit word; reference:
// src/limbs_diag.cu:24 and include/internal.hpp:116-159).  Device code only.
#pragma once
#include <stdint.h>

namespace hyb {

struct U192 { uint64_t w[3]; };

__device__ __forceinline__ void mul_small_add(U192& v, uint32_t m, uint32_t a) {
  unsigned __int128 t = (unsigned __int128)v.w[0] * m + a; v.w[0] = uint64_t(t);
  t = (unsigned __int128)v.w[1] * m + uint64_t(t >> 64); v.w[1] = uint64_t(t);
  v.w[2] = v.w[2] * m + uint64_t(t >> 64);
}
__device__ __forceinline__ void add192(U192& v, const U192& o) {
  unsigned __int128 t = (unsigned __int128)v.w[0] + o.w[0]; v.w[0] = uint64_t(t);
  t = (unsigned __int128)v.w[1] + o.w[1] + uint64_t(t >> 64); v.w[1] = uint64_t(t);
  v.w[2] = v.w[2] + o.w[2] + uint64_t(t >> 64);
}
__device__ __forceinline__ void sub192(U192& v, const uint64_t (&o)[3]) {
  unsigned __int128 t = (unsigned __int128)v.w[0] - o[0]; v.w[0] = uint64_t(t);
  uint64_t borrow = uint64_t(t >> 64) & 1u;
  t = (unsigned __int128)v.w[1] - o[1] - borrow; v.w[1] = uint64_t(t);
  borrow = uint64_t(t >> 64) & 1u;
  v.w[2] = v.w[2] - o[2] - borrow;
}
__device__ __forceinline__ bool greater192(const U192& v, const uint64_t (&o)[3]) {   // unsigned v > o
  if (v.w[2] != o[2]) return v.w[2] > o[2];
  if (v.w[1] != o[1]) return v.w[1] > o[1];
  return v.w[0] > o[0];
}
__device__ __forceinline__ void sar63(U192& v) {   // arithmetic shift right by 63 (two's complement)
  const uint64_t ext = uint64_t(int64_t(v.w[2]) >> 63);
  const uint64_t n0 = (v.w[0] >> 63) | (v.w[1] << 1), n1 = (v.w[1] >> 63) | (v.w[2] << 1), n2 = (v.w[2] >> 63) | (ext << 1);
  v.w[0] = n0; v.w[1] = n1; v.w[2] = n2;
}
// 63-bit limbs (signed last limb) -> 192-bit two's complement.
__device__ __forceinline__ U192 limbs_to_u192(const uint64_t* p, int64_t stride, int order) {
  U192 v; const uint64_t a0 = p[0];
  if (order == 1) { v.w[0] = a0; v.w[1] = v.w[2] = uint64_t(int64_t(a0) >> 63); return v; }
  const uint64_t a1 = p[stride];
  if (order == 2) {
    const uint64_t ext = uint64_t(int64_t(a1) >> 63);
    v.w[0] = a0 | (a1 << 63); v.w[1] = (a1 >> 1) | (ext << 63); v.w[2] = ext; return v;
  }
  const uint64_t a2 = p[2 * stride], ext = uint64_t(int64_t(a2) >> 63);
  v.w[0] = a0 | (a1 << 63); v.w[1] = (a1 >> 1) | (a2 << 62); v.w[2] = (a2 >> 2) | (ext << 62);
  return v;
}
__device__ __forceinline__ void store_limbs(U192 v, uint64_t* p, int64_t stride, int order) {
  constexpr uint64_t m63 = 0x7fffffffffffffffull;
  if (order == 1) { p[0] = v.w[0]; return; }
  p[0] = v.w[0] & m63; sar63(v);
  if (order == 2) { p[stride] = v.w[0]; return; }
  p[stride] = v.w[0] & m63; sar63(v);
  p[2 * stride] = v.w[0];
}

// v += (sign-extended 32-bit x) << shift, 0 <= shift < 160.
__device__ __forceinline__ void add_i32_shifted(U192& v, int32_t x, int shift) {
  const uint64_t lo = uint64_t(int64_t(x)), ext = uint64_t(int64_t(x) >> 63);
  const int ws = shift >> 6, bs = shift & 63;
  // the shifted operand as three words: word k takes bits from (lo, ext, ext) moved up by `shift`
  uint64_t t0 = lo, t1 = ext, t2 = ext;
  if (bs) { t2 = (t2 << bs) | (t1 >> (64 - bs)); t1 = (t1 << bs) | (t0 >> (64 - bs)); t0 <<= bs; }
  uint64_t s0 = ws == 0 ? t0 : 0, s1 = ws == 0 ? t1 : (ws == 1 ? t0 : 0), s2 = ws == 0 ? t2 : (ws == 1 ? t1 : t0);
  unsigned __int128 c = (unsigned __int128)v.w[0] + s0; v.w[0] = uint64_t(c);
  c = (unsigned __int128)v.w[1] + s1 + uint64_t(c >> 64); v.w[1] = uint64_t(c);
  v.w[2] = v.w[2] + s2 + uint64_t(c >> 64);
}

}  // namespace hyb
