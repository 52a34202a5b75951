// CRT reconstruction: residue bytes of the Gram tiles -> exact signed integers in packed 63-bit limbs.
//
// Contract (reference: src/crt_reconstruct_real.cu:51-92, write_a :40-49): the value represented by the
// residues, taken in the symmetric range (-P/2, P/2), is added to (beta) or stored into the packed upper
// triangle C[limb][y + x(x+1)/2], limbs of 63 bits with a signed last limb.
//
// The algorithm is not the reference's.  The reference sums s_x * (P / m_x) with multi-word constants and
// balances signs on the fly.  Here the residues go through Garner's mixed-radix conversion, which needs only
// byte-sized constants (m_j^-1 mod m_i), and the digits are folded by Horner's rule into a 192-bit integer;
// because the residues of all row chunks were accumulated modulo m inside the Gram kernel's epilogue, this
// runs once per hyacinXherkBatch call instead of once per 8192-row flush.
//
// Mapping: one CTA per (tile, 32-column strip); thread = Gram row y inside the tile.  A thread reads its 32
// residue bytes of every modulus (one 32-byte sector each) and writes entries (y, x) for 32 consecutive x;
// the threads of a warp hold consecutive y, so every store instruction covers one contiguous run of C.
#include "hyb_internal.h"
#include "crt_tables.h"
#include "limbs192.cuh"

namespace hyb {
namespace {

__constant__ uint16_t c_modulus[crt::kMaxModuli] = HYB_CRT_MODULUS_INIT;
__constant__ uint32_t c_magic[crt::kMaxModuli] = HYB_CRT_MAGIC_CEIL_INIT;
__constant__ uint8_t c_inv[crt::kMaxModuli][crt::kMaxModuli] = HYB_CRT_INV_INIT;
__constant__ uint64_t c_product[crt::kMaxModuli][3] = HYB_CRT_PRODUCT_INIT;
__constant__ uint64_t c_half_product[crt::kMaxModuli][3] = HYB_CRT_HALF_PRODUCT_INIT;
__constant__ uint16_t c_lift[crt::kMaxModuli] = HYB_CRT_LIFT_INIT;
// the same for the moduli of complex input (crt2m); padded to the size of the first set
__constant__ uint16_t c2_modulus[crt::kMaxModuli] = HYB_CRT2M_MODULUS_INIT;
__constant__ uint32_t c2_magic[crt::kMaxModuli] = HYB_CRT2M_MAGIC_CEIL_INIT;
__constant__ uint8_t c2_inv[crt::kMaxModuli][crt::kMaxModuli] = HYB_CRT2M_INV_INIT;
__constant__ uint64_t c2_product[crt::kMaxModuli][3] = HYB_CRT2M_PRODUCT_INIT;
__constant__ uint64_t c2_half_product[crt::kMaxModuli][3] = HYB_CRT2M_HALF_PRODUCT_INIT;
__constant__ uint16_t c2_lift[crt::kMaxModuli] = HYB_CRT2M_LIFT_INIT;
__constant__ uint16_t c2_inv_two[crt::kMaxModuli] = HYB_CRT2M_INV_TWO_INIT;
__constant__ uint16_t c2_inv_two_iota[crt::kMaxModuli] = HYB_CRT2M_INV_TWO_IOTA_INIT;
static_assert(crt2m::kMaxModuli <= crt::kMaxModuli, "crt2m tables are stored in arrays sized for crt");

template <int SET> struct Tables;
template <> struct Tables<0> {
  static __device__ __forceinline__ uint32_t modulus(int i) { return c_modulus[i]; }
  static __device__ __forceinline__ uint32_t magic(int i) { return c_magic[i]; }
  static __device__ __forceinline__ uint32_t lift(int i) { return c_lift[i]; }
  static __device__ __forceinline__ uint32_t inv(int j, int i) { return c_inv[j][i]; }
  static __device__ __forceinline__ const uint64_t (&product(int k))[3] { return c_product[k]; }
  static __device__ __forceinline__ const uint64_t (&half_product(int k))[3] { return c_half_product[k]; }
};
template <> struct Tables<1> {
  static __device__ __forceinline__ uint32_t modulus(int i) { return c2_modulus[i]; }
  static __device__ __forceinline__ uint32_t magic(int i) { return c2_magic[i]; }
  static __device__ __forceinline__ uint32_t lift(int i) { return c2_lift[i]; }
  static __device__ __forceinline__ uint32_t inv(int j, int i) { return c2_inv[j][i]; }
  static __device__ __forceinline__ const uint64_t (&product(int k))[3] { return c2_product[k]; }
  static __device__ __forceinline__ const uint64_t (&half_product(int k))[3] { return c2_half_product[k]; }
};

// KMAX: compile-time bound on the number of moduli (keeps the residues in registers).
// SET: 0 = moduli of crt, 1 = moduli of crt2m.
template <int KMAX, int COLS, int SET>
__global__ void __launch_bounds__(kTileY)
reconstruct_kernel(int n, int k, int tiles_y, int num_tiles, const uint8_t* __restrict__ residues, int beta, int order,
                   uint64_t* __restrict__ C) {
  constexpr int kWords = COLS / 4;
  using Tb = Tables<SET>;
  int ty, tx; tile_coords(tiles_y, blockIdx.x, &ty, &tx);
  const int y = ty * kTileY + threadIdx.x;
  const int x0 = tx * kTileX + blockIdx.y * COLS;
  if (x0 + COLS - 1 < ty * kTileY || x0 >= n) return;       // strip entirely below the diagonal or outside
  if (y >= n) return;
  const int64_t tri = (int64_t(n) * n + n) / 2;

  uint32_t r[KMAX][kWords];
#pragma unroll
  for (int i = 0; i < KMAX; ++i) {
    if (i < k) {
      const uint8_t* src = residues + (size_t(i) * num_tiles + blockIdx.x) * size_t(kTileY * kTileX) +
                           size_t(threadIdx.x) * kTileX + blockIdx.y * COLS;
#pragma unroll
      for (int w = 0; w < kWords; w += 4) {
        const uint4 q = *reinterpret_cast<const uint4*>(src + 4 * w);
        r[i][w] = q.x; r[i][w + 1] = q.y; r[i][w + 2] = q.z; r[i][w + 3] = q.w;
      }
    }
  }

#pragma unroll
  for (int w = 0; w < kWords; ++w) {
#pragma unroll 1
    for (int b = 0; b < 4; ++b) {
      const int x = x0 + 4 * w + b;
      // Garner: mixed-radix digits a_i with value = a_0 + a_1 m_0 + a_2 m_0 m_1 + ...
      uint32_t a[KMAX];
#pragma unroll
      for (int i = 0; i < KMAX; ++i) {
        if (i < k) {
          uint32_t t = r[i][w] & 0xFFu; r[i][w] >>= 8;
          const uint32_t mi = Tb::modulus(i), magic = Tb::magic(i);
          const uint32_t lift = Tb::lift(i);                           // multiple of m_i above every digit a_j <= 255
#pragma unroll
          for (int j = 0; j < i; ++j) {
            // (t - a_j) * m_j^-1 mod m_i; the lift keeps the difference positive, the product stays below 2^18
            // so the multiply-high quotient is exact.
            const uint32_t d = (t + lift - a[j]) * Tb::inv(j, i);
            t = d - __umulhi(d, magic) * mi;
          }
          a[i] = t;
        } else a[i] = 0;
      }
      if (x < n && y <= x) {
        // Horner: value = a_0 + m_0 (a_1 + m_1 (a_2 + ...)), in [0, P).
        U192 v; v.w[0] = 0; v.w[1] = 0; v.w[2] = 0;
#pragma unroll
        for (int i = KMAX - 1; i >= 0; --i) if (i < k) mul_small_add(v, Tb::modulus(i), a[i]);
        // Symmetric range: values above P/2 stand for v - P (two's complement from here on).
        if (greater192(v, Tb::half_product(k - 1))) sub192(v, Tb::product(k - 1));
        uint64_t* dst = C + y + (int64_t(x) * (x + 1)) / 2;
        if (beta) { const U192 old = limbs_to_u192(dst, tri, order); add192(v, old); }
        store_limbs(v, dst, tri, order);
      }
    }
  }
}

}  // namespace

void launch_reconstruct(cudaStream_t stream, int n, int moduli, const uint8_t* residues, int beta, int order,
                        uint64_t* C_panel, int table) {
  if (n <= 0 || moduli <= 0 || order <= 0) return;
  const TilePlan tp = make_tile_plan(n);
  count_launch();
#define HYB_RECONSTRUCT(KMAX, COLS, SET) \
  reconstruct_kernel<KMAX, COLS, SET><<<dim3(tp.num_tiles, kTileX / COLS), kTileY, 0, stream>>>(n, moduli, tp.tiles_y, tp.num_tiles, residues, beta, order, C_panel)
  if (table == 0) {
    if (moduli <= 8) HYB_RECONSTRUCT(8, 32, 0); else if (moduli <= 16) HYB_RECONSTRUCT(16, 32, 0); else HYB_RECONSTRUCT(24, 16, 0);
  } else {
    if (moduli <= 8) HYB_RECONSTRUCT(8, 32, 1); else if (moduli <= 16) HYB_RECONSTRUCT(16, 32, 1); else HYB_RECONSTRUCT(24, 16, 1);
  }
#undef HYB_RECONSTRUCT
  HYB_CUDA(cudaGetLastError());
}

// ---- crt2m: product over all tiles -> real / imaginary residues over the upper-triangle tiles ------------------
namespace {
// One CTA per (upper-triangle tile, modulus), 256 threads.  Entry (y, x) of the tile needs X[y][x], which sits in
// the same place of the full tile (ty, tx), and X[x][y], which sits transposed in the full tiles (2 tx + h, ty / 2),
// h = 0, 1: each of those contributes a 128 x 128 block that is staged in shared memory and read transposed.
__global__ void __launch_bounds__(256)
crt2m_rotate_kernel(int n, int tiles_y, int tiles_x, int num_tri, const uint8_t* __restrict__ full, uint8_t* __restrict__ re_out,
                    uint8_t* __restrict__ im_out) {
  __shared__ uint8_t blk[128][132];
  int ty, tx; tile_coords(tiles_y, blockIdx.x, &ty, &tx);
  const int m = blockIdx.y;
  const uint32_t modulus = c2_modulus[m], magic = c2_magic[m], inv2 = c2_inv_two[m], inv2i = c2_inv_two_iota[m];
  const size_t tile_bytes = size_t(kTileY) * kTileX;
  const uint8_t* direct = full + (size_t(m) * tiles_y * tiles_x + size_t(ty) + size_t(tx) * tiles_y) * tile_bytes;
  uint8_t* re_t = re_out + (size_t(m) * num_tri + blockIdx.x) * tile_bytes;
  uint8_t* im_t = im_out + (size_t(m) * num_tri + blockIdx.x) * tile_bytes;
  for (int h = 0; h < 2; ++h) {
    const int src_ty = 2 * tx + h, src_tx = ty >> 1, col0 = (ty & 1) * 128;
    __syncthreads();
    if (src_ty < tiles_y) {
      const uint8_t* src = full + (size_t(m) * tiles_y * tiles_x + size_t(src_ty) + size_t(src_tx) * tiles_y) * tile_bytes + col0;
      for (int idx = threadIdx.x; idx < 128 * 32; idx += 256) {        // 128 rows (x) of 32 words (y)
        const int xr = idx >> 5, w = idx & 31;
        *reinterpret_cast<uint32_t*>(&blk[xr][4 * w]) = *reinterpret_cast<const uint32_t*>(src + size_t(xr) * kTileX + 4 * w);
      }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < 128 * 32; idx += 256) {          // 128 rows (y) of 32 words (x)
      const int yr = idx >> 5, w = idx & 31;
      const uint32_t a4 = *reinterpret_cast<const uint32_t*>(direct + size_t(yr) * kTileX + 128 * h + 4 * w);
      uint32_t re4 = 0, im4 = 0;
      if (src_ty < tiles_y) {
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const uint32_t a = (a4 >> (8 * b)) & 0xFFu, t = blk[4 * w + b][yr];
          const uint32_t s = (a + t) * inv2, d = (a + modulus - t) * inv2i;      // both below 2^17
          re4 |= (s - __umulhi(s, magic) * modulus) << (8 * b);
          im4 |= (d - __umulhi(d, magic) * modulus) << (8 * b);
        }
      }
      *reinterpret_cast<uint32_t*>(re_t + size_t(yr) * kTileX + 128 * h + 4 * w) = re4;
      *reinterpret_cast<uint32_t*>(im_t + size_t(yr) * kTileX + 128 * h + 4 * w) = im4;
    }
  }
}
}  // namespace

void launch_crt2m_rotate(cudaStream_t stream, int n, int moduli, const uint8_t* full_residues, uint8_t* re_residues, uint8_t* im_residues) {
  if (n <= 0 || moduli <= 0) return;
  const TilePlan tp = make_tile_plan(n);
  count_launch();
  crt2m_rotate_kernel<<<dim3(tp.num_tiles, moduli), 256, 0, stream>>>(n, tp.tiles_y, tp.tiles_x, tp.num_tiles, full_residues, re_residues, im_residues);
  HYB_CUDA(cudaGetLastError());
}

}  // namespace hyb
