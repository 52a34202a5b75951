// Residue Gram kernel for sm_100a: int8 x int8 -> int32 on the 5th-generation tensor cores.
//
// Replaces, for the CRT route, the reference's cuBLAS INT8 GEMM calls plus the int32 scratch pass that
// reduces them modulo m (src/hyacin_herk.cpp:95-109,163-189 and src/crt_diag_real.cu:13-29): the modular
// reduction is the epilogue of the GEMM tile, so the only thing that leaves the SM is one byte per
// (entry, modulus).
//
// Three kernels.  gram_wide_kernel (last in the file) is the one the CRT route runs: clusters of two CTAs with
// tcgen05.mma.cta_group::2 on items of two neighbouring 256 x 256 tiles that share their A rows.  gram_pair_kernel is
// its predecessor on single 256 x 256 tiles (kept for A/B runs and as the fallback).  gram_kernel<LIMBS> is the
// single-CTA form (128 x 256 tiles); it carries the limb route and is the last fallback of the CRT route.  Structure
// of the single-CTA form (one CTA per SM, persistent over (modulus, tile) work items):
//   warp 0     TMA producer: 128-byte-swizzled K-major boxes of the A operand (128 Gram rows) and the B
//              operand (256 Gram columns) into a 4-stage shared-memory ring, completion on mbarriers;
//   warp 1     MMA issuer: one thread issues tcgen05.mma.cta_group::1.kind::i8 (M128 N256 K32) on shared-memory
//              descriptors, accumulating in one of two 256-column TMEM buffers; tcgen05.commit releases the
//              stage and, after the last K block, hands the accumulator to the epilogue;
//   warps 2-5  epilogue: tcgen05.ld of the int32 accumulator (32 lanes x 32 columns per load), reduction
//              modulo m, optional accumulation onto the residues of earlier row chunks, 32-byte stores.
// The two TMEM buffers let the epilogue of one tile overlap the main loop of the next.
// No TMA load in this file uses cluster multicast (tcgen05.commit of the two-CTA kernels does address both CTAs of
// its pair).  Every wait is bounded: a wait that expires raises a status word for the host and makes all roles
// leave their loops so that TMEM is still released.
#include "hyb_internal.h"
#include "crt_tables.h"
#include "limbs192.cuh"
#include "ptx_sm100.cuh"
#include <cuda.h>
#include <mutex>
#include <cstdlib>

namespace hyb {
namespace {

constexpr int kStages = 4;
constexpr int kUmmaK = 32;                                    // K per tcgen05.mma for 8-bit operands
constexpr uint32_t kABytes = kTileY * kStageK;                // 16 KiB
constexpr uint32_t kBBytes = kTileX * kStageK;                // 32 KiB
constexpr uint32_t kStageBytes = kABytes + kBBytes;           // 48 KiB
constexpr int kThreads = 192;
constexpr int kEpilogueWarps = 4;
constexpr uint32_t kTmemCols = 512;                           // two accumulators of kTileX columns
constexpr size_t kSmemBytes = 1024 /*alignment slack*/ + size_t(kStages) * kStageBytes + 256 /*barriers*/;

struct ModConsts {
  uint32_t modulus[crt::kMaxModuli];
  uint32_t magic[crt::kMaxModuli];      // floor(2^32 / m)
  uint32_t bias[crt::kMaxModuli];       // multiple of m in (2^31 - m, 2^31]: makes the accumulator non-negative
};

struct GramParams {
  uint8_t* residues; uint32_t* status;
  int ka0, kb0;                 // first K row of the A / B operand inside a column
  int num_kblocks;              // k_rows / kStageK
  int num_tiles, tiles_y, moduli, accumulate;
  int full;                     // 1: tile index = ty + tx tiles_y over all tiles (the product is not symmetric)
  // limb mode: planes are the balanced base-256 digits of the quantised values; the accumulator of shift s
  // collects every digit pair (i, j) with i + j = s and is added to the packed integer Gram at bit 8 s
  uint64_t* gram; int64_t tri; int n, order, limb_panels, overwrite;
  // limb mode with few tiles: one work group per (tile, shift) instead of per tile, so that a small Gram still fills the
  // GPU; the int32 accumulators go to scratch[tile][shift][kTileY][kTileX] and limb_combine_kernel adds them up
  int32_t* scratch; int split;
  ModConsts k;
};

// Shift handled by the r-th group of a tile when the shifts are dealt heaviest first: the middle shift order - 1 collects
// `order` digit pairs, its neighbours one fewer each.
__host__ __device__ inline int shift_of_rank(int r, int order) { return (r & 1) ? order - 1 - (r + 1) / 2 : order - 1 + r / 2; }

using namespace ptx;

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, stored with the 128-byte
// swizzle: groups of 8 rows (1024 bytes) follow each other, so the stride byte offset is 1024.
__device__ __forceinline__ uint64_t smem_desc_k128(uint32_t saddr) {
  uint64_t d = 0;
  d |= uint64_t((saddr & 0x3FFFFu) >> 4);          // start address, 16-byte units
  d |= uint64_t(1) << 16;                          // leading byte offset (unused for swizzled K-major)
  d |= uint64_t(1024 >> 4) << 32;                  // stride byte offset
  d |= uint64_t(1) << 46;                          // descriptor version of sm_100
  d |= uint64_t(2) << 61;                          // SWIZZLE_128B
  return d;
}
// kind::i8 instruction descriptor: s8 x s8 -> s32, both operands K-major, M = 128, N = 256.
constexpr uint32_t kInstrDesc = (2u << 4) | (1u << 7) | (1u << 10) | (uint32_t(kTileX >> 3) << 17) | (uint32_t(kTileY >> 4) << 24);

struct Barriers {
  uint64_t full[kStages], empty[kStages], acc_full[2], acc_empty[2];
  uint32_t tmem_base; uint32_t abort_flag;
};

// LIMBS = false: one work group per (modulus, tile), one accumulator, epilogue = residue bytes.
// LIMBS = true : one work group per tile, 2 order - 1 accumulators (one per shift) handled one after the other by
//                the same CTA, epilogue = read-modify-write of the packed 63-bit limbs (the same thread owns an
//                entry for every shift, so no atomics are needed).
__device__ __forceinline__ void tile_of(const GramParams& p, int t, int* ty, int* tx) {
  if (p.full) { *tx = t / p.tiles_y; *ty = t - *tx * p.tiles_y; } else tile_coords(p.tiles_y, t, ty, tx);
}

template <bool LIMBS>
__global__ void __launch_bounds__(kThreads, 1)
gram_kernel(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ GramParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;                 // swizzle atoms need 1 KiB alignment
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  Barriers* bars = reinterpret_cast<Barriers*>(aligned + size_t(kStages) * kStageBytes);
  volatile uint32_t* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool split = LIMBS && p.split != 0;
  const int num_groups = LIMBS ? (split ? p.num_tiles * (2 * p.order - 1) : p.num_tiles) : p.moduli * p.num_tiles;
  const int subs = LIMBS ? (split ? 1 : 2 * p.order - 1) : 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&bars->full[s], 1); mbar_init(&bars->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&bars->acc_full[a], 1); mbar_init(&bars->acc_empty[a], kEpilogueWarps); }
    bars->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(&bars->tmem_base, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0; bool ok = true;
      for (int group = blockIdx.x; group < num_groups && ok; group += gridDim.x) {
        int ty, tx; tile_of(p, group % p.num_tiles, &ty, &tx);
        for (int step = 0; step < subs && ok; ++step) {
          const int sub = split ? shift_of_rank(group / p.num_tiles, p.order) : step;
          // plane pairs of this accumulator: (m, m) for residues; (i, sub - i) for limbs
          const int first = LIMBS ? (sub - (p.order - 1) > 0 ? sub - (p.order - 1) : 0) : group / p.num_tiles;
          const int last = LIMBS ? (sub < p.order - 1 ? sub : p.order - 1) : first;
          for (int pa = first; pa <= last && ok; ++pa) {
            const int pb = LIMBS ? sub - pa : pa;
            for (int kb = 0; kb < p.num_kblocks; ++kb) {
              if (!(ok = mbar_wait(&bars->empty[stage], phase ^ 1u, abort_flag, p.status, 1u))) break;
              mbar_expect_tx(&bars->full[stage], kStageBytes);
              const uint32_t sa = base + stage * kStageBytes, sb = sa + kABytes;
              tma_load_3d(sa, &tmap, &bars->full[stage], p.ka0 + kb * kStageK, ty * kTileY, pa);
              tma_load_3d(sb, &tmap, &bars->full[stage], p.kb0 + kb * kStageK, tx * kTileX, pb);
              tma_load_3d(sb + kABytes, &tmap, &bars->full[stage], p.kb0 + kb * kStageK, tx * kTileX + kTileY, pb);
              if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0; bool ok = true;
      for (int group = blockIdx.x; group < num_groups && ok; group += gridDim.x)
      for (int step = 0; step < subs && ok; ++step) {
        const int sub = split ? shift_of_rank(group / p.num_tiles, p.order) : step;
        if (!(ok = mbar_wait(&bars->acc_empty[acc], acc_phase ^ 1u, abort_flag, p.status, 2u))) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * kTileX;
        const int pairs = LIMBS ? ((sub < p.order - 1 ? sub : p.order - 1) - (sub - (p.order - 1) > 0 ? sub - (p.order - 1) : 0) + 1) : 1;
        const int total_kb = pairs * p.num_kblocks;
        for (int kb = 0; kb < total_kb; ++kb) {
          if (!(ok = mbar_wait(&bars->full[stage], phase, abort_flag, p.status, 3u))) break;
          tc_fence_after();
          const uint32_t sa = base + stage * kStageBytes, sb = sa + kABytes;
          const uint64_t adesc = smem_desc_k128(sa), bdesc = smem_desc_k128(sb);
#pragma unroll
          for (int k = 0; k < kStageK / kUmmaK; ++k) {
            // advancing K inside the swizzle row: +32 bytes = +2 in 16-byte units of the start-address field
            umma_i8(tmem_d, adesc + uint64_t(2 * k), bdesc + uint64_t(2 * k), kInstrDesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&bars->empty[stage]);              // frees the stage once these MMAs have read it
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(&bars->acc_full[acc]);               // accumulator complete -> epilogue
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ---------------- epilogue warps ----------------
    const int lane_group = warp & 3;                     // TMEM lanes 32 * (warp % 4) .. +31 are visible to this warp
    const int row = lane_group * 32 + lane;
    uint32_t acc = 0, acc_phase = 0; bool ok = true;
    for (int group = blockIdx.x; group < num_groups && ok; group += gridDim.x)
    for (int step = 0; step < subs && ok; ++step) {
      const int sub = split ? shift_of_rank(group / p.num_tiles, p.order) : step;
      const int m = LIMBS ? 0 : group / p.num_tiles, tile = group % p.num_tiles;
      ok = mbar_wait(&bars->acc_full[acc], acc_phase, abort_flag, p.status, 4u);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t(lane_group * 32) << 16) + acc * kTileX;
      if (LIMBS && split) {
        // raw accumulator of this (tile, shift) to scratch: 128 contiguous bytes per thread and load
        int32_t* out = p.scratch + ((size_t(tile) * (2 * p.order - 1) + sub) * kTileY + row) * size_t(kTileX);
#pragma unroll 1
        for (int c = 0; c < kTileX / 32; ++c) {
          uint32_t v[32];
          tmem_ld32(taddr + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 8; ++q) reinterpret_cast<uint4*>(out + c * 32)[q] = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        }
      } else if constexpr (LIMBS) {
        int ty, tx; tile_of(p, tile, &ty, &tx);
        const int y = ty * kTileY + row;
        const bool store_only = p.overwrite && sub == 0;        // first shift of the first chunk of a beta = 0 call
#pragma unroll 1
        for (int c = 0; c < kTileX / 32; ++c) {
          uint32_t v[32];
          tmem_ld32(taddr + c * 32, v);
          tmem_ld_wait();
#pragma unroll 4
          for (int q = 0; q < 32; ++q) {
            const int x = tx * kTileX + c * 32 + q;
            if (y < p.n && x < p.n && y <= x) {
              uint64_t* dst = p.gram + y + (int64_t(x) * (x + 1)) / 2;
              U192 acc192; acc192.w[0] = acc192.w[1] = acc192.w[2] = 0;
              if (!store_only) acc192 = limbs_to_u192(dst, p.tri, p.limb_panels);
              add_i32_shifted(acc192, int32_t(v[q]), 8 * sub);
              store_limbs(acc192, dst, p.tri, p.limb_panels);
            }
          }
        }
      } else {
      const uint32_t modulus = p.k.modulus[m], magic = p.k.magic[m], bias = p.k.bias[m];
      uint8_t* out = p.residues + (size_t(m) * p.num_tiles + tile) * size_t(kTileY * kTileX) + size_t(row) * kTileX;
#pragma unroll 1
      for (int c = 0; c < kTileX / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(taddr + c * 32, v);
        uint4 old0 = make_uint4(0, 0, 0, 0), old1 = old0;
        if (p.accumulate) { old0 = *reinterpret_cast<const uint4*>(out + c * 32); old1 = *reinterpret_cast<const uint4*>(out + c * 32 + 16); }
        tmem_ld_wait();
        const uint32_t oldw[8] = {old0.x, old0.y, old0.z, old0.w, old1.x, old1.y, old1.z, old1.w};
        uint32_t packed[8];
#pragma unroll
        for (int w = 0; w < 8; ++w) {
          uint32_t word = 0;
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            // accumulator + bias is non-negative and congruent to the accumulator; add the previous residue,
            // estimate the quotient (at most one too small), correct once.
            uint32_t t = v[w * 4 + b] + bias + ((oldw[w] >> (8 * b)) & 0xFFu);
            uint32_t r = t - __umulhi(t, magic) * modulus;
            r = r >= modulus ? r - modulus : r;
            word |= r << (8 * b);
          }
          packed[w] = word;
        }
        *reinterpret_cast<uint4*>(out + c * 32) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        *reinterpret_cast<uint4*>(out + c * 32 + 16) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
      }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->acc_empty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  }

  // Teardown: every role ends up here, also after an expired wait, so TMEM is always released.
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

// Second half of the split limb mode: entry (y, x) of a tile gets sum_s scratch[tile][s][y][x] 2^(8 s) added to its
// packed 63-bit limbs (or stored, for the first chunk of a beta = 0 call).  One thread per Gram row of the tile, as in
// the epilogue above, so the limb words of consecutive threads are contiguous.
__global__ void __launch_bounds__(kTileY) limb_combine_kernel(const GramParams p) {
  int ty, tx; tile_of(p, blockIdx.x, &ty, &tx);
  const int y = ty * kTileY + threadIdx.x, shifts = 2 * p.order - 1;
  if (y >= p.n) return;
  const int32_t* src = p.scratch + (size_t(blockIdx.x) * shifts * kTileY + threadIdx.x) * size_t(kTileX);
  for (int q = blockIdx.y * 32; q < blockIdx.y * 32 + 32; ++q) {      // 32 of the tile's columns per block
    const int x = tx * kTileX + q;
    if (x >= p.n || y > x) continue;
    uint64_t* dst = p.gram + y + (int64_t(x) * (x + 1)) / 2;
    U192 acc192; acc192.w[0] = acc192.w[1] = acc192.w[2] = 0;
    if (!p.overwrite) acc192 = limbs_to_u192(dst, p.tri, p.limb_panels);
    for (int sft = 0; sft < shifts; ++sft) add_i32_shifted(acc192, src[size_t(sft) * kTileY * kTileX + q], 8 * sft);
    store_limbs(acc192, dst, p.tri, p.limb_panels);
  }
}

// ---- two-CTA variant (residue Gram over the upper triangle) ---------------------------------------------------
// A CTA pair (cluster of two, the two SMs of a TPC) works on a 256 x 256 tile with tcgen05.mma.cta_group::2: each CTA
// stages its 128 rows of the A operand and its 128 columns of the B operand, the MMA issued by the even CTA reads
// both halves, and each CTA keeps the accumulator of its own 128 rows in its tensor memory.  Per MMA every SM
// fetches and reads 8 KiB of operands instead of 12, which is what matters when the step runs into the power cap.
// Loads are plain TMA tile loads of the CTA's own halves that signal the even CTA's barrier (no multicast);
// tcgen05.commit arrives on the barriers of both CTAs.  The output layout is unchanged: the pair tile (TY, TX)
// is the two ordinary tiles (2 TY, TX) and (2 TY + 1, TX).
constexpr int kStages2 = 6;
constexpr uint32_t kStageBytes2 = 2 * kABytes;               // 16 KiB of A rows + 16 KiB of B columns per CTA
constexpr size_t kSmemBytes2 = 1024 + size_t(kStages2) * kStageBytes2 + 256;
constexpr uint32_t kInstrDesc2 = (2u << 4) | (1u << 7) | (1u << 10) | (uint32_t(256 >> 3) << 17) | (uint32_t(256 >> 4) << 24);
struct Barriers2 {
  uint64_t full[kStages2], empty[kStages2], acc_full[2], acc_empty[2];
  uint32_t tmem_base; uint32_t abort_flag;
};
__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank)); return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
               ::"r"(smem_dst), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void umma_i8_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {      // arrives on this barrier in both CTAs of the pair
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(uint16_t(3)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void pair_tile_coords(int tiles_x, int t, int* TY, int* TX) {   // TY <= TX, column-block major
  int x = 0, base = 0;
  for (;;) { if (t < base + x + 1 || x + 1 >= tiles_x) { *TY = t - base; *TX = x; return; } base += x + 1; ++x; }
}
__device__ __forceinline__ int tile_index(int tiles_y, int ty, int tx) {                   // inverse of tile_coords
  int base = 0;
  for (int x = 0; x < tx; ++x) { int cnt = 2 * x + 2; base += cnt > tiles_y ? tiles_y : cnt; }
  return base + ty;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gram_pair_kernel(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ GramParams p, int tiles_x) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  Barriers2* bars = reinterpret_cast<Barriers2*>(aligned + size_t(kStages2) * kStageBytes2);
  volatile uint32_t* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  const int pair_rows = (p.tiles_y + 1) / 2;                            // pair tiles per column block when every tile is wanted
  const int pairs = p.full ? pair_rows * tiles_x : tiles_x * (tiles_x + 1) / 2;
  const int num_items = p.moduli * pairs;
  auto pair_of = [&](int t, int* TY, int* TX) {
    if (p.full) { *TX = t / pair_rows; *TY = t - *TX * pair_rows; } else pair_tile_coords(tiles_x, t, TY, TX);
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages2; ++s) { mbar_init(&bars->full[s], 1); mbar_init(&bars->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&bars->acc_full[a], 1); mbar_init(&bars->acc_empty[a], 2 * kEpilogueWarps); }
    bars->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                               // barriers and tensor memory of both CTAs exist from here on
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs: own halves, completion counted on the even CTA's barrier) ----------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0; bool ok = true;
      for (int item = cluster_id; item < num_items && ok; item += num_clusters) {
        const int m = item / pairs; int TY, TX; pair_of(item - m * pairs, &TY, &TX);
        const int y0 = (2 * TY + int(rank)) * kTileY, x0 = TX * kTileX + int(rank) * kTileY;
        for (int kb = 0; kb < p.num_kblocks; ++kb) {
          if (!(ok = mbar_wait(&bars->empty[stage], phase ^ 1u, abort_flag, p.status, 11u))) break;
          if (rank == 0) mbar_expect_tx(&bars->full[stage], 2 * kStageBytes2);
          const uint32_t sa = base + stage * kStageBytes2, sb = sa + kABytes;
          const uint32_t full0 = map_to_cta(smem_u32(&bars->full[stage]), 0);
          tma_load_3d_pair(sa, &tmap, full0, p.ka0 + kb * kStageK, y0, m);
          tma_load_3d_pair(sb, &tmap, full0, p.kb0 + kb * kStageK, x0, m);
          if (++stage == kStages2) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (even CTA only) ----------------
    if (lane == 0 && rank == 0) {
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0; bool ok = true;
      for (int item = cluster_id; item < num_items && ok; item += num_clusters) {
        if (!(ok = mbar_wait(&bars->acc_empty[acc], acc_phase ^ 1u, abort_flag, p.status, 12u))) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * kTileX;
        for (int kb = 0; kb < p.num_kblocks; ++kb) {
          if (!(ok = mbar_wait(&bars->full[stage], phase, abort_flag, p.status, 13u))) break;
          tc_fence_after();
          const uint32_t sa = base + stage * kStageBytes2, sb = sa + kABytes;
          const uint64_t adesc = smem_desc_k128(sa), bdesc = smem_desc_k128(sb);
#pragma unroll
          for (int k = 0; k < kStageK / kUmmaK; ++k)
            umma_i8_pair(tmem_d, adesc + uint64_t(2 * k), bdesc + uint64_t(2 * k), kInstrDesc2, (kb | k) != 0 ? 1u : 0u);
          umma_commit_pair(&bars->empty[stage]);
          if (++stage == kStages2) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit_pair(&bars->acc_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ---------------- epilogue warps (both CTAs: own 128 rows) ----------------
    const int lane_group = warp & 3;
    const int row = lane_group * 32 + lane;
    uint32_t acc = 0, acc_phase = 0; bool ok = true;
    for (int item = cluster_id; item < num_items && ok; item += num_clusters) {
      const int m = item / pairs; int TY, TX; pair_of(item - m * pairs, &TY, &TX);
      const int ty = 2 * TY + int(rank);
      ok = mbar_wait(&bars->acc_full[acc], acc_phase, abort_flag, p.status, 14u);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      if (ty < p.tiles_y) {
        const uint32_t taddr = tmem_base + (uint32_t(lane_group * 32) << 16) + acc * kTileX;
        const int tile = p.full ? ty + TX * p.tiles_y : tile_index(p.tiles_y, ty, TX);
        const uint32_t modulus = p.k.modulus[m], magic = p.k.magic[m], bias = p.k.bias[m];
        uint8_t* out = p.residues + (size_t(m) * p.num_tiles + tile) * size_t(kTileY * kTileX) + size_t(row) * kTileX;
#pragma unroll 1
        for (int c = 0; c < kTileX / 32; ++c) {
          uint32_t v[32];
          tmem_ld32(taddr + c * 32, v);
          uint4 old0 = make_uint4(0, 0, 0, 0), old1 = old0;
          if (p.accumulate) { old0 = *reinterpret_cast<const uint4*>(out + c * 32); old1 = *reinterpret_cast<const uint4*>(out + c * 32 + 16); }
          tmem_ld_wait();
          const uint32_t oldw[8] = {old0.x, old0.y, old0.z, old0.w, old1.x, old1.y, old1.z, old1.w};
          uint32_t packed[8];
#pragma unroll
          for (int w = 0; w < 8; ++w) {
            uint32_t word = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              uint32_t t = v[w * 4 + b] + bias + ((oldw[w] >> (8 * b)) & 0xFFu);
              uint32_t r = t - __umulhi(t, magic) * modulus;
              r = r >= modulus ? r - modulus : r;
              word |= r << (8 * b);
            }
            packed[w] = word;
          }
          *reinterpret_cast<uint4*>(out + c * 32) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          *reinterpret_cast<uint4*>(out + c * 32 + 16) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(map_to_cta(smem_u32(&bars->acc_empty[acc]), 0));
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  }

  // Teardown: every role of both CTAs ends up here, also after an expired wait.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
}

// ---- two-CTA variant on items of two neighbouring tiles (the default of the CRT route) ----------------------------
// A CTA pair works on the pair tiles (TY, TX) and (TY, TX + 1) at once: the 128 A rows a CTA stages are multiplied with
// both column blocks (two MMAs per K step, one accumulator each), so a CTA stages 48 KiB per 128-byte K block for two
// accumulators instead of 64 KiB.  The step runs against the power cap, so fewer bytes moved per MAC means a higher
// clock: 5 % on the step against gram_pair_kernel.  All 512 columns of tensor memory hold one item, so the accumulators
// are not double buffered: the epilogue (eight warps, both accumulators in parallel, the old residue bytes of the next
// 32 columns prefetched) runs between items, about 1 % of a 65536-row item.  A tile row with an odd number of tiles ends
// in an ordinary single-tile item.  Items of two sizes are dealt so that all pairs finish together: the double items
// round-robin, then the single ones first to the pairs that got one double item less (WideSchedule; the host mirror
// hyacinB200GramItem lets a CPU test check that every tile is covered once).  HYACIN_B200_GRAM_WIDE=0 selects
// gram_pair_kernel instead.
constexpr int kStagesW = 4;
constexpr uint32_t kStageBytesW = 3 * kABytes;               // A rows + two blocks of B columns per CTA
constexpr size_t kSmemBytesW = 1024 + size_t(kStagesW) * kStageBytesW + 256;
constexpr int kEpilogueWarpsW = 8;
constexpr int kThreadsW = 64 + 32 * kEpilogueWarpsW;
struct BarriersW {
  uint64_t full[kStagesW], empty[kStagesW], acc_full, acc_empty;
  uint32_t tmem_base; uint32_t abort_flag;
};

struct WideSchedule {
  int tiles_x, pair_rows, full, clusters, cluster;
  int doubles_per_plane, singles_per_plane, doubles, singles;
  int my_doubles, low_first, low_count, filled, my_filled;
  // full = 0: pair tiles TY <= TX of the upper triangle; full = 1: all pair_rows x tiles_x pair tiles
  __host__ __device__ void init(int tiles_x_, int pair_rows_, int full_, int moduli, int clusters_, int cluster_) {
    tiles_x = tiles_x_; pair_rows = pair_rows_; full = full_; clusters = clusters_; cluster = cluster_;
    doubles_per_plane = full ? pair_rows * (tiles_x / 2) : (tiles_x * tiles_x) / 4;
    singles_per_plane = full ? (tiles_x & 1) * pair_rows : (tiles_x + 1) / 2;
    doubles = moduli * doubles_per_plane; singles = moduli * singles_per_plane;
    const int r = doubles % clusters;
    my_doubles = doubles / clusters + (cluster < r ? 1 : 0);
    // pairs r .. clusters - 1 have one double item less: they take up to two single items each before the rest is dealt to all
    low_first = r; low_count = clusters - r;
    filled = r > 0 ? (singles < 2 * low_count ? singles : 2 * low_count) : 0;
    my_filled = 0;
    if (r > 0 && cluster >= r) my_filled = (cluster - r < filled ? 1 : 0) + (cluster - r + low_count < filled ? 1 : 0);
  }
  // k-th item of this pair: modulus, tile row, first tile column, number of tiles (1 or 2); false when there is none
  __host__ __device__ bool item(int k, int* m, int* TY, int* TX, int* width) const {
    if (k < my_doubles) {
      const int g = cluster + k * clusters;
      *m = g / doubles_per_plane; int w = g - *m * doubles_per_plane;
      if (full) { const int per_row = tiles_x / 2; *TY = w / per_row; *TX = 2 * (w - *TY * per_row); }
      else for (int ty = 0;; ++ty) { const int c = (tiles_x - ty) / 2; if (w < c) { *TY = ty; *TX = ty + 2 * w; break; } w -= c; }
      *width = 2; return true;
    }
    const int j = k - my_doubles;
    const int sidx = j < my_filled ? cluster - low_first + j * low_count : filled + cluster + (j - my_filled) * clusters;
    if (sidx >= singles) return false;
    *m = sidx / singles_per_plane; const int w = sidx - *m * singles_per_plane;
    *TY = full ? w : ((tiles_x - 1) & 1) + 2 * w; *TX = tiles_x - 1; *width = 1;
    return true;
  }
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreadsW, 1)
gram_wide_kernel(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ GramParams p, int tiles_x) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  BarriersW* bars = reinterpret_cast<BarriersW*>(aligned + size_t(kStagesW) * kStageBytesW);
  volatile uint32_t* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  WideSchedule sched; sched.init(tiles_x, (p.tiles_y + 1) / 2, p.full, p.moduli, gridDim.x >> 1, blockIdx.x >> 1);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStagesW; ++s) { mbar_init(&bars->full[s], 1); mbar_init(&bars->empty[s], 1); }
    mbar_init(&bars->acc_full, 1); mbar_init(&bars->acc_empty, 2 * kEpilogueWarpsW);
    bars->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs: own rows and own halves of the column blocks) ----------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0; bool ok = true;
      int m, TY, TX, width;
      for (int k = 0; ok && sched.item(k, &m, &TY, &TX, &width); ++k) {
        const int y0 = (2 * TY + int(rank)) * kTileY, x0 = TX * kTileX + int(rank) * kTileY;
        for (int kb = 0; kb < p.num_kblocks; ++kb) {
          if (!(ok = mbar_wait(&bars->empty[stage], phase ^ 1u, abort_flag, p.status, 21u))) break;
          if (rank == 0) mbar_expect_tx(&bars->full[stage], 2u * uint32_t(1 + width) * kABytes);
          const uint32_t sa = base + stage * kStageBytesW;
          const uint32_t full0 = map_to_cta(smem_u32(&bars->full[stage]), 0);
          tma_load_3d_pair(sa, &tmap, full0, p.ka0 + kb * kStageK, y0, m);
          tma_load_3d_pair(sa + kABytes, &tmap, full0, p.kb0 + kb * kStageK, x0, m);
          if (width == 2) tma_load_3d_pair(sa + 2 * kABytes, &tmap, full0, p.kb0 + kb * kStageK, x0 + kTileX, m);
          if (++stage == kStagesW) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (even CTA only) ----------------
    if (lane == 0 && rank == 0) {
      uint32_t stage = 0, phase = 0, acc_phase = 0; bool ok = true;
      int m, TY, TX, width;
      for (int k = 0; ok && sched.item(k, &m, &TY, &TX, &width); ++k) {
        if (!(ok = mbar_wait(&bars->acc_empty, acc_phase ^ 1u, abort_flag, p.status, 22u))) break;
        tc_fence_after();
        for (int kb = 0; kb < p.num_kblocks; ++kb) {
          if (!(ok = mbar_wait(&bars->full[stage], phase, abort_flag, p.status, 23u))) break;
          tc_fence_after();
          const uint32_t sa = base + stage * kStageBytesW;
          const uint64_t adesc = smem_desc_k128(sa), b0desc = smem_desc_k128(sa + kABytes), b1desc = smem_desc_k128(sa + 2 * kABytes);
#pragma unroll
          for (int q = 0; q < kStageK / kUmmaK; ++q) {
            umma_i8_pair(tmem_base, adesc + uint64_t(2 * q), b0desc + uint64_t(2 * q), kInstrDesc2, (kb | q) != 0 ? 1u : 0u);
            if (width == 2) umma_i8_pair(tmem_base + kTileX, adesc + uint64_t(2 * q), b1desc + uint64_t(2 * q), kInstrDesc2, (kb | q) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&bars->empty[stage]);
          if (++stage == kStagesW) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit_pair(&bars->acc_full);
        acc_phase ^= 1u;
      }
    }
  } else {
    // ---------------- epilogue warps (both CTAs: own 128 rows; warps 2-5 and 6-9 split the columns) ----------------
    const int lane_group = warp & 3, half = (warp - 2) >> 2;
    const int row = lane_group * 32 + lane;
    uint32_t acc_phase = 0; bool ok = true;
    int m, TY, TX, width;
    for (int k = 0; ok && sched.item(k, &m, &TY, &TX, &width); ++k) {
      const int ty = 2 * TY + int(rank);
      ok = mbar_wait(&bars->acc_full, acc_phase, abort_flag, p.status, 24u);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      if (ty < p.tiles_y) {
        // double item: this warp drains one accumulator (one tile); single item: half of the only accumulator
        const int col0 = width == 2 ? half * kTileX : half * (kTileX / 2), chunks = width == 2 ? kTileX / 32 : kTileX / 64;
        const int tx = width == 2 ? TX + half : TX, out_col0 = width == 2 ? 0 : col0;
        const uint32_t taddr = tmem_base + (uint32_t(lane_group * 32) << 16) + uint32_t(col0);
        const int tile = p.full ? ty + tx * p.tiles_y : tile_index(p.tiles_y, ty, tx);
        const uint32_t modulus = p.k.modulus[m], magic = p.k.magic[m], bias = p.k.bias[m];
        uint8_t* out = p.residues + (size_t(m) * p.num_tiles + tile) * size_t(kTileY * kTileX) + size_t(row) * kTileX + out_col0;
        uint4 old0 = make_uint4(0, 0, 0, 0), old1 = old0;
        if (p.accumulate) { old0 = *reinterpret_cast<const uint4*>(out); old1 = *reinterpret_cast<const uint4*>(out + 16); }
#pragma unroll 1
        for (int c = 0; c < chunks; ++c) {
          uint32_t v[32];
          tmem_ld32(taddr + c * 32, v);
          const uint32_t oldw[8] = {old0.x, old0.y, old0.z, old0.w, old1.x, old1.y, old1.z, old1.w};
          if (p.accumulate && c + 1 < chunks) {          // the bytes of the next chunk arrive while this one is reduced
            old0 = *reinterpret_cast<const uint4*>(out + (c + 1) * 32); old1 = *reinterpret_cast<const uint4*>(out + (c + 1) * 32 + 16);
          }
          tmem_ld_wait();
          uint32_t packed[8];
#pragma unroll
          for (int w = 0; w < 8; ++w) {
            uint32_t word = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              uint32_t t = v[w * 4 + b] + bias + ((oldw[w] >> (8 * b)) & 0xFFu);
              uint32_t r = t - __umulhi(t, magic) * modulus;
              r = r >= modulus ? r - modulus : r;
              word |= r << (8 * b);
            }
            packed[w] = word;
          }
          *reinterpret_cast<uint4*>(out + c * 32) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          *reinterpret_cast<uint4*>(out + c * 32 + 16) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(map_to_cta(smem_u32(&bars->acc_empty), 0));
      acc_phase ^= 1u;
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
}

// ---- host side ------------------------------------------------------------------------------------
}  // namespace

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr; cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q);
    if (e == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeTiledFn>(sym);
    else std::fprintf(stderr, "hyacin-b200: cuTensorMapEncodeTiled is not available from this driver\n");
  });
  return fn;
}

TilePlan make_tile_plan(int n) {
  TilePlan t; t.n = n;
  t.tiles_x = (n + kTileX - 1) / kTileX; t.tiles_y = (n + kTileY - 1) / kTileY;
  int count = 0;
  for (int x = 0; x < t.tiles_x; ++x) { int c = 2 * x + 2; count += c < t.tiles_y ? c : t.tiles_y; }
  t.num_tiles = count;
  return t;
}

namespace {
bool encode_planes(CUtensorMap* tmap, const int8_t* w, int64_t ldw, int n, int planes, int64_t plane_stride) {
  EncodeTiledFn encode = encode_tiled();
  if (!encode) return false;
  const cuuint64_t dims[3] = {cuuint64_t(ldw), cuuint64_t(n), cuuint64_t(planes)};
  const cuuint64_t strides[2] = {cuuint64_t(ldw), cuuint64_t(plane_stride)};
  const cuuint32_t box[3] = {cuuint32_t(kStageK), cuuint32_t(kTileY), 1};
  const cuuint32_t elem[3] = {1, 1, 1};
  CUresult r = encode(tmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<int8_t*>(w), dims, strides, box, elem,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { std::fprintf(stderr, "hyacin-b200: cuTensorMapEncodeTiled failed (%d)\n", int(r)); return false; }
  return true;
}
}  // namespace

void launch_gram_residues(cudaStream_t stream, const GramLaunch& g) {
  const TilePlan tp = make_tile_plan(g.n);
  CUtensorMap tmap;
  if (!encode_planes(&tmap, g.w, g.ldw, g.n, g.moduli, g.plane_stride)) return;
  GramParams p{};
  p.residues = g.residues; p.status = g.status;
  p.ka0 = g.ka0; p.kb0 = g.kb0; p.num_kblocks = g.k_rows / kStageK;
  p.full = g.full ? 1 : 0;
  p.num_tiles = p.full ? tp.tiles_y * tp.tiles_x : tp.num_tiles; p.tiles_y = tp.tiles_y; p.moduli = g.moduli; p.accumulate = g.accumulate;
  for (int i = 0; i < crt::kMaxModuli; ++i) {
    const bool have = g.table == 0 || i < crt2m::kMaxModuli;
    const uint32_t m = !have ? 1u : g.table == 0 ? crt::kModulus[i] : crt2m::kModulus[i];
    p.k.modulus[i] = m; p.k.magic[i] = !have ? 0u : g.table == 0 ? crt::kMagicFloor[i] : crt2m::kMagicFloor[i];
    p.k.bias[i] = (0x80000000u / m) * m;
  }
  static const bool single_cta = [] { const char* e = std::getenv("HYACIN_B200_GRAM_SINGLE_CTA"); return e && e[0] == '1'; }();   // diagnosis: A/B the two kernels
  static const bool narrow = [] { const char* e = std::getenv("HYACIN_B200_GRAM_WIDE"); return e && e[0] == '0'; }();        // diagnosis: items of one tile
  if (!narrow && !single_cta && p.num_kblocks > 0 && g.sm_count >= 2) {
    // CTA pairs on items of two neighbouring 256 x 256 tiles
    HYB_CUDA(cudaFuncSetAttribute(gram_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSmemBytesW)));
    const int units = g.moduli * (p.full ? ((tp.tiles_y + 1) / 2) * tp.tiles_x : tp.tiles_x * (tp.tiles_x + 1) / 2);
    int clusters = g.sm_count / 2; if (clusters > units) clusters = units;
    ProfileScope prof(stream, KernelKind::Gram);
    count_launch();
    gram_wide_kernel<<<2 * clusters, kThreadsW, kSmemBytesW, stream>>>(tmap, p, tp.tiles_x);
    const cudaError_t launched = cudaGetLastError();
    if (launched == cudaSuccess) return;
    std::fprintf(stderr, "hyacin-b200: cluster launch of the wide Gram kernel refused (%s); trying the pair kernel\n", cudaGetErrorString(launched));
  }
  if (!single_cta && p.num_kblocks > 0 && g.sm_count >= 2) {
    // CTA pairs on 256 x 256 tiles; the single-CTA kernel below remains for devices that report one SM
    HYB_CUDA(cudaFuncSetAttribute(gram_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSmemBytes2)));
    const int pairs = p.full ? ((tp.tiles_y + 1) / 2) * tp.tiles_x : tp.tiles_x * (tp.tiles_x + 1) / 2;
    int clusters = g.sm_count / 2; if (clusters > g.moduli * pairs) clusters = g.moduli * pairs;
    ProfileScope prof(stream, KernelKind::Gram);
    count_launch();
    gram_pair_kernel<<<2 * clusters, kThreads, kSmemBytes2, stream>>>(tmap, p, tp.tiles_x);
    const cudaError_t launched = cudaGetLastError();
    if (launched == cudaSuccess) return;
    std::fprintf(stderr, "hyacin-b200: cluster launch of the pair Gram kernel refused (%s); using the single-CTA kernel\n", cudaGetErrorString(launched));
  }
  HYB_CUDA(cudaFuncSetAttribute(gram_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSmemBytes)));
  const int items = g.moduli * p.num_tiles;
  int grid = g.sm_count > 0 ? g.sm_count : 148; if (grid > items) grid = items;
  if (grid <= 0 || p.num_kblocks <= 0) return;
  ProfileScope prof(stream, KernelKind::Gram);
  count_launch();
  gram_kernel<false><<<grid, kThreads, kSmemBytes, stream>>>(tmap, p);
  HYB_CUDA(cudaGetLastError());
}

void launch_gram_limbs(cudaStream_t stream, const GramLimbLaunch& g) {
  const TilePlan tp = make_tile_plan(g.n);
  CUtensorMap tmap;
  if (!encode_planes(&tmap, g.w, g.ldw, g.n, g.order, g.plane_stride)) return;
  GramParams p{};
  p.status = g.status; p.ka0 = g.ka0; p.kb0 = g.kb0; p.num_kblocks = g.k_rows / kStageK;
  p.num_tiles = tp.num_tiles; p.tiles_y = tp.tiles_y;
  p.gram = g.gram; p.tri = (int64_t(g.n) * g.n + g.n) / 2; p.n = g.n; p.order = g.order; p.limb_panels = g.limb_panels;
  p.overwrite = g.overwrite;
  HYB_CUDA(cudaFuncSetAttribute(gram_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSmemBytes)));
  const int sms = g.sm_count > 0 ? g.sm_count : 148;
  if (tp.num_tiles <= 0 || p.num_kblocks <= 0 || g.order <= 0) return;
  // fewer tiles than SMs: deal (tile, shift) pairs to the CTAs instead of tiles and sum the shifts afterwards
  p.split = (g.scratch != nullptr && tp.num_tiles < sms) ? 1 : 0;
  p.scratch = g.scratch;
  const int groups = p.split ? tp.num_tiles * (2 * g.order - 1) : tp.num_tiles;
  const int grid = groups < sms ? groups : sms;
  ProfileScope prof(stream, KernelKind::Gram);
  count_launch(p.split ? 2 : 1);
  gram_kernel<true><<<grid, kThreads, kSmemBytes, stream>>>(tmap, p);
  if (p.split) limb_combine_kernel<<<dim3(tp.num_tiles, kTileX / 32), kTileY, 0, stream>>>(p);
  HYB_CUDA(cudaGetLastError());
}

bool gram_schedule_item(int tiles_x, int pair_rows, int full, int moduli, int clusters, int cluster, int k, int* m, int* TY, int* TX, int* width) {
  if (tiles_x <= 0 || pair_rows <= 0 || moduli <= 0 || clusters <= 0 || cluster < 0 || cluster >= clusters || k < 0) return false;
  WideSchedule sched; sched.init(tiles_x, pair_rows, full ? 1 : 0, moduli, clusters, cluster);
  return sched.item(k, m, TY, TX, width);
}

size_t gram_limbs_scratch_bytes(int n, int order, int sm_count) {
  const TilePlan tp = make_tile_plan(n);
  const int sms = sm_count > 0 ? sm_count : 148;
  return tp.num_tiles < sms ? size_t(tp.num_tiles) * (2 * order - 1) * kTileY * kTileX * sizeof(int32_t) : 0;
}

}  // namespace hyb
