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

// KMAX: compile-time bound on the number of moduli (keeps the residues in registers).
template <int KMAX, int COLS>
__global__ void __launch_bounds__(kTileY)
reconstruct_kernel(int n, int k, int tiles_y, int num_tiles, const uint8_t* __restrict__ residues, int beta, int order,
                   uint64_t* __restrict__ C) {
  constexpr int kWords = COLS / 4;
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
          const uint32_t mi = c_modulus[i], magic = c_magic[i];
#pragma unroll
          for (int j = 0; j < i; ++j) {
            // (t - a_j) * m_j^-1 mod m_i; 2 m_i >= 302 > a_j keeps the difference positive, the product stays
            // below 2^18 so the multiply-high quotient is exact.
            const uint32_t d = (t + 2 * mi - a[j]) * c_inv[j][i];
            t = d - __umulhi(d, magic) * mi;
          }
          a[i] = t;
        } else a[i] = 0;
      }
      if (x < n && y <= x) {
        // Horner: value = a_0 + m_0 (a_1 + m_1 (a_2 + ...)), in [0, P).
        U192 v; v.w[0] = 0; v.w[1] = 0; v.w[2] = 0;
#pragma unroll
        for (int i = KMAX - 1; i >= 0; --i) if (i < k) mul_small_add(v, c_modulus[i], a[i]);
        // Symmetric range: values above P/2 stand for v - P (two's complement from here on).
        if (greater192(v, c_half_product[k - 1])) sub192(v, c_product[k - 1]);
        uint64_t* dst = C + y + (int64_t(x) * (x + 1)) / 2;
        if (beta) { const U192 old = limbs_to_u192(dst, tri, order); add192(v, old); }
        store_limbs(v, dst, tri, order);
      }
    }
  }
}

}  // namespace

void launch_reconstruct(cudaStream_t stream, int n, int moduli, const uint8_t* residues, int beta, int order,
                        uint64_t* C_panel) {
  if (n <= 0 || moduli <= 0 || order <= 0) return;
  const TilePlan tp = make_tile_plan(n);
  count_launch();
  if (moduli <= 8) {
    dim3 grid(tp.num_tiles, kTileX / 32);
    reconstruct_kernel<8, 32><<<grid, kTileY, 0, stream>>>(n, moduli, tp.tiles_y, tp.num_tiles, residues, beta, order, C_panel);
  } else if (moduli <= 16) {
    dim3 grid(tp.num_tiles, kTileX / 32);
    reconstruct_kernel<16, 32><<<grid, kTileY, 0, stream>>>(n, moduli, tp.tiles_y, tp.num_tiles, residues, beta, order, C_panel);
  } else {
    dim3 grid(tp.num_tiles, kTileX / 16);
    reconstruct_kernel<24, 16><<<grid, kTileY, 0, stream>>>(n, moduli, tp.tiles_y, tp.num_tiles, residues, beta, order, C_panel);
  }
  HYB_CUDA(cudaGetLastError());
}

}  // namespace hyb
