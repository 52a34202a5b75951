// Internal interfaces of the B200 Hyacin build (host side).  Nothing here is part of the public ABI.
#pragma once
#include <hyacin.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>

namespace hyb {

// ---------------------------------------------------------------------------------------------------
// Error reporting.  The public ABI has no error channel (the reference drops CUDA errors in release
// builds); this build keeps going as well but says so on stderr, once per call site.
// ---------------------------------------------------------------------------------------------------
void report_cuda_error(cudaError_t err, const char* what, const char* file, int line);
#define HYB_CUDA(call) do { cudaError_t hyb_err_ = (call); if (hyb_err_ != cudaSuccess) \
  ::hyb::report_cuda_error(hyb_err_, #call, __FILE__, __LINE__); } while (0)

inline int is_complex(hyacinPrecision_t t) { return int(t) & 1; }
inline int base_type(hyacinPrecision_t t) { return int(t) & ~1; }

// Status word of the bounded waits in the Gram kernel (pinned host memory mapped into the device).
uint32_t* status_word_device(int device);
uint32_t* status_word_if_ready(int device);      // never allocates: nullptr until status_word_device has run
uint32_t status_word_read(int device, bool clear);
void status_check(const hyacinHandle_t* handle, const char* where);

// Launch accounting: every kernel launch of this library is counted; with profiling switched on the Gram,
// quantise, pivoted-Cholesky and SVD launches are also bracketed by CUDA events on the launching stream (read back by hyacinB200Profile*).
enum class KernelKind : int { Other = 0, Quantize = 1, Gram = 2, Cholesky = 3, Svd = 4, Count = 5 };
void count_launch(int n = 1);
struct ProfileScope {                       // RAII: records start/stop events around one launch when enabled
  ProfileScope(cudaStream_t stream, KernelKind kind);
  ~ProfileScope();
  cudaStream_t stream; int slot;
};

// Timer classes of hyacinSync_TimerSegments ('D', 'R', 'C'; anything else untimed).
enum class Segment : unsigned char { Untimed, Distributed, Replicated, Comm };
void timer_mark(const hyacinHandle_t* handle, Segment seg);

// ---------------------------------------------------------------------------------------------------
// Geometry of the residue Gram kernel.
//   One work item = one (modulus, tile) pair; a tile is kTileY rows (y, the A operand) by kTileX columns
//   (x, the B operand) of the Gram matrix, kept only if it intersects the upper triangle y <= x.
//   Residues of a tile are stored as kTileY x kTileX bytes, x fastest, tiles in the order of tile_list().
// ---------------------------------------------------------------------------------------------------
constexpr int kTileY = 128;
constexpr int kTileX = 256;
constexpr int kStageK = 128;                       // bytes of K per pipeline stage (one 128-byte swizzle row)
constexpr int kMaxAccumRows = 130816;              // 128 * 128 * rows < 2^31 keeps the int32 accumulator exact

struct TilePlan {
  int n;            // Gram dimension
  int tiles_x;      // ceil(n / kTileX)
  int tiles_y;      // ceil(n / kTileY)
  int num_tiles;    // tiles that touch the upper triangle
};
TilePlan make_tile_plan(int n);
// Linear tile index -> (ty, tx).  Column-block major: all ty of tx = 0, then tx = 1, ...
__host__ __device__ inline void tile_coords(int n_tiles_y, int t, int* ty, int* tx) {
  // Tiles of column block tx: ty = 0 .. min(tiles_y, 2 tx + 2) - 1  (kTileX == 2 kTileY).
  int x = 0, base = 0;
  for (;;) {
    int cnt = 2 * x + 2; if (cnt > n_tiles_y) cnt = n_tiles_y;
    if (t < base + cnt) { *ty = t - base; *tx = x; return; }
    base += cnt; ++x;
  }
}

// Integer Gram of op(A): what hyacinXherkBatch does, for any of the three input layouts.
// batches / seg_m: the row segmentation vexp was built with (rows 1.. of vexp hold the per-segment exponents); with
// more than one segment the precision ladder may split the rows into runs of lower precision.
void herk_any(const hyacinHandle_t* handle, int64_t rows, int n, hyacinPrecision_t atype, const void* A, int64_t lda, char op,
              int u, const int32_t* vexp, int beta, int order_c, uint64_t* C, int batches = 1, int64_t seg_m = 0);

// Plan of one hyacinXherkBatch call: how many moduli, how rows are grouped and chunked.
struct CrtPlan {
  int moduli;          // number of CRT moduli (prefix of crt::kModulus)
  int value_bytes;     // bytes needed for a biased quantised value (1..12)
  int group_rows;      // rows reconstructed together (residues accumulate across the chunks of a group)
  int chunk_rows;      // rows quantised and multiplied per kernel launch (multiple of kStageK)
  int two_m;           // complex input through the moduli with a square root of -1 (crt2m tables, two planes p, q)
};
// u: quantisation bits of the call; cplx: 0/1; rows: rows of this call.  Returns moduli == 0 if impossible.
// allow_two_m: complex input may use the crt2m route when its moduli cover the whole call without grouping.
CrtPlan make_crt_plan(int u, int cplx, int64_t rows, bool allow_two_m = true);

// ---------------------------------------------------------------------------------------------------
// Kernel launchers (all asynchronous on `stream`).
// ---------------------------------------------------------------------------------------------------

// Column exponents: fills vexp[(batches+1) x N].  Reference behaviour: src/fp_exponent.cu:45-51.
// op 'N': A is rows x n column-major.  op 'T' / 'C': A is stored n x rows (the transposed input of a fit).
void launch_column_exponents(cudaStream_t stream, hyacinPrecision_t atype, int batches, int seg_m, int last_m, int n,
                             const void* A, int64_t lda, int u, int32_t* vexp, char op = 'N');
// Bits needed per row segment (segU[batches]).  Reference behaviour: src/fp_exponent.cu:67-76.
void launch_vector_range(cudaStream_t stream, int batches, int n, int u, const int32_t* vexp, int32_t* seg_u);

// Quantise rows [0, rows) of op(A) into centred int8 residue planes (op as for launch_column_exponents)
//   W[modulus][column][part * ldk + row]     (ldk a multiple of kStageK; rows in [rows, ldk) are zeroed)
// Real input has one part.  Complex input has three, stacked along K inside each column: real, imaginary,
// negated real -- so that rows [0, 2 ldk) are the operand (re; im) and rows [ldk, 3 ldk) the operand (im; -re).
// With plan.two_m complex input has two parts instead: p = re - iota im and q = re + iota im modulo each modulus of
// the crt2m set (reference counterpart: src/quantize_crt_complex.cu:30-42).
void launch_quantize_crt(cudaStream_t stream, hyacinPrecision_t atype, int rows, int n, const void* A, int64_t lda,
                         const int32_t* vexp, const CrtPlan& plan, int8_t* W, int64_t ldk, char op = 'N');

// Residue Gram of one chunk.  For every modulus m and every upper-triangle tile:
//   R[m][tile][y][x] = (accumulate ? R : 0) + sum_{k < k_rows} W[m][y][ka0 + k] * W[m][x][kb0 + k]  (mod m), a byte.
// W has column pitch ldw and plane pitch plane_stride (bytes); k_rows, ka0, kb0 are multiples of kStageK.
// status: device word that becomes non-zero if a bounded wait inside the kernel expired.
struct GramLaunch {
  const int8_t* w;
  int64_t ldw, plane_stride;
  int ka0, kb0, k_rows, n, moduli, accumulate, sm_count;
  uint8_t* residues;            // [moduli][num_tiles][kTileY * kTileX]
  uint32_t* status;
  int full;                     // 1: every tile (ty, tx) = index ty + tx tiles_y, for a product that is not symmetric
  int table;                    // 0: moduli of crt, 1: moduli of crt2m
};
void launch_gram_residues(cudaStream_t stream, const GramLaunch& g);
// crt2m: X = P^T Q over all tiles -> residues of the real and imaginary parts of the Hermitian Gram in the
// upper-triangle tile layout: re = (X_yx + X_xy) / 2, im = (X_yx - X_xy) / (2 iota) modulo each modulus.
// Reference counterpart: src/crt_rotate.cu.
void launch_crt2m_rotate(cudaStream_t stream, int n, int moduli, const uint8_t* full_residues, uint8_t* re_residues, uint8_t* im_residues);

// Limb Gram of one chunk, straight into the packed integer Gram (one panel: real or imaginary part):
//   gram[y <= x] (+)= sum_{i, j < order} 2^(8 (i + j)) sum_{k < k_rows} W[i][y][ka0 + k] * W[j][x][kb0 + k]
// W holds `order` planes of balanced base-256 digits.  order * k_rows * 2^14 must stay below 2^31 (digit pairs
// with the same i + j share one int32 accumulator).  overwrite: the call defines gram instead of adding to it.
// Reference counterpart: src/hyacin_herk.cpp:111-161 with src/limbs_diag.cu, limbs_cross_real.cu, limbs_cross_imag.cu.
struct GramLimbLaunch {
  const int8_t* w;
  int64_t ldw, plane_stride;
  int ka0, kb0, k_rows, n, order, limb_panels, overwrite, sm_count;
  uint64_t* gram;
  uint32_t* status;
  int32_t* scratch;             // gram_limbs_scratch_bytes() bytes, or nullptr: with it, a Gram of few tiles is split over (tile, shift)
};
void launch_gram_limbs(cudaStream_t stream, const GramLimbLaunch& g);
// Scratch that lets launch_gram_limbs fill the GPU when the Gram has fewer tiles than the device has SMs (0 otherwise).
size_t gram_limbs_scratch_bytes(int n, int order, int sm_count);
// k-th work item of CTA pair `cluster` in the residue Gram kernel (host mirror of the device schedule, for tests)
bool gram_schedule_item(int tiles_x, int pair_rows, int full, int moduli, int clusters, int cluster, int k, int* m, int* TY, int* TX, int* width);
// Quantise rows of A into `order` planes of balanced base-256 digits (same plane layout as launch_quantize_crt).
// Reference counterpart: src/quantize_limbs.cu:29-79.
void launch_quantize_limbs(cudaStream_t stream, hyacinPrecision_t atype, int rows, int n, const void* A, int64_t lda,
                           const int32_t* vexp, int order, int8_t* W, int64_t ldk, char op = 'N');

// CRT reconstruction of `moduli` residue planes into the packed 63-bit-limb Gram:
//   C[panel][order][tri] = (beta ? C : 0) + value.  Reference counterpart: src/crt_reconstruct_real.cu:51-92.
// table: 0 = moduli of crt, 1 = moduli of crt2m.
void launch_reconstruct(cudaStream_t stream, int n, int moduli, const uint8_t* residues, int beta, int order,
                        uint64_t* C_panel, int table = 0);

// The same two steps on the summed slices of a cross-rank reduction (S[panel][slice][tri], layout of slice_plan for
// `ranks` ranks): the limbs are re-assembled in registers, so the post-collective epilogue needs no pass that writes
// them back.  Reference counterpart of the fusion: src/allreduce_1drow.cu:112-131 + src/fp_i63tp_dequantize.cu.
void launch_gram_range_slices(cudaStream_t stream, int n, int order, int ranks, const uint64_t* S, const int32_t* vexp, int32_t* bits_out);
void launch_dequantize_slices(cudaStream_t stream, int n, int order, int ranks, const uint64_t* S, const int32_t* vexp,
                              hyacinPrecision_t gtype, void* G, int64_t ldg);
// Cut C into slices and sum them over the communicator; returns the pool-allocated slice buffer (the caller frees it
// on the handle's stream) and the communicator size, or nullptr when there is nothing to reduce.
uint64_t* allreduce_to_slices(const hyacinHandle_t* handle, int panels, int order, uint64_t count, const uint64_t* C, int* ranks_out);
// Gram format for a given bit length of the largest true-scale diagonal entry (src/fp_i63tp_dequantize.cu:46-54).
hyacinPrecision_t gram_type_from_bits(const hyacinHandle_t* handle, int bits, hyacinPrecision_t atype);

// Largest bit length among the true-scale diagonal entries (written to *bits_out, device or pinned).
void launch_gram_range(cudaStream_t stream, int n, int order, const uint64_t* C, const int32_t* vexp, int32_t* bits_out);
// Packed integer Gram -> full Hermitian floating-point matrix.
void launch_dequantize(cudaStream_t stream, int n, int order, const uint64_t* C, const int32_t* vexp,
                       hyacinPrecision_t gtype, void* G, int64_t ldg);

// Slices for the cross-rank sum: A[panels][order][count] -> S[panels][slice_count][count] and back.
int slice_count(int order, int ranks);
void slice_layout(int order, int ranks, int* slices, int* width);
void launch_limbs_to_slices(cudaStream_t stream, int panels, int order, int ranks, uint64_t count, const uint64_t* A, uint64_t* S);
void launch_slices_to_limbs(cudaStream_t stream, int panels, int order, int ranks, uint64_t count, const uint64_t* S, uint64_t* A);

}  // namespace hyb
