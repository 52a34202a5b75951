// Slices of a multi-limb integer for the cross-rank sum: how a value is cut before the all-reduce and put together
// after it.  Shared by the slicing kernels and by the kernels that read the summed slices directly.
#pragma once
#include <stdint.h>

namespace hyb {

// Slices 0 .. slices-2 hold `width` unsigned bits each, the last one the remaining (signed) top bits.
struct SlicePlan { int slices; int width; };
SlicePlan slice_plan(int order, int ranks);

struct W192 { uint64_t w[3]; };

__device__ __forceinline__ W192 load_value(const uint64_t* p, uint64_t stride, int order) {
  W192 v; const uint64_t a0 = p[0];
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
__device__ __forceinline__ void sar(W192& v, int s) {      // arithmetic shift right, 0 < s < 64
  const uint64_t ext = uint64_t(int64_t(v.w[2]) >> 63);
  v.w[0] = (v.w[0] >> s) | (v.w[1] << (64 - s)); v.w[1] = (v.w[1] >> s) | (v.w[2] << (64 - s)); v.w[2] = (v.w[2] >> s) | (ext << (64 - s));
}
__device__ __forceinline__ void add_shifted(W192& v, uint64_t s, bool is_signed, int shift) {   // v += s << shift
  const uint64_t ext = is_signed ? uint64_t(int64_t(s) >> 63) : 0;
  uint64_t t[3] = {s, ext, ext};
  const int ws = shift >> 6, bs = shift & 63;
  uint64_t sh[3];
#pragma unroll
  for (int k = 2; k >= 0; --k) {
    const uint64_t lo = (k - ws >= 0) ? t[k - ws] : 0, below = (k - ws - 1 >= 0) ? t[k - ws - 1] : 0;
    sh[k] = bs ? (lo << bs) | (below >> (64 - bs)) : lo;
  }
  unsigned __int128 c = (unsigned __int128)v.w[0] + sh[0]; v.w[0] = uint64_t(c);
  c = (unsigned __int128)v.w[1] + sh[1] + uint64_t(c >> 64); v.w[1] = uint64_t(c);
  v.w[2] = v.w[2] + sh[2] + uint64_t(c >> 64);
}

// Limbs of value `idx` of panel `panel`, from the packed limb array C[panel][limb][count] ...
struct LimbSource {
  const uint64_t* C; uint64_t count;
  template <int ORDER> __device__ __forceinline__ void load(uint64_t idx, int panel, uint64_t (&a)[ORDER]) const {
#pragma unroll
    for (int l = 0; l < ORDER; ++l) a[l] = C[(uint64_t(panel) * ORDER + l) * count + idx];
  }
};
// ... or from the summed slices S[panel][slice][count], re-assembled in registers.
struct SliceSource {
  const uint64_t* S; uint64_t count; SlicePlan plan;
  template <int ORDER> __device__ __forceinline__ void load(uint64_t idx, int panel, uint64_t (&a)[ORDER]) const {
    W192 v; v.w[0] = v.w[1] = v.w[2] = 0;
    const uint64_t* src = S + uint64_t(panel) * plan.slices * count + idx;
    for (int s = 0; s < plan.slices; ++s) add_shifted(v, src[uint64_t(s) * count], s + 1 == plan.slices, s * plan.width);
    constexpr uint64_t m63 = 0x7fffffffffffffffull;
#pragma unroll
    for (int l = 0; l + 1 < ORDER; ++l) { a[l] = v.w[0] & m63; sar(v, 63); }
    a[ORDER - 1] = v.w[0];
  }
};

}  // namespace hyb
