// Host orchestration of the quantized Gram: sizing, column exponents, the integer HERK and dequantisation.
//
// Entry points keep the reference's names, arguments and no-op rules (src/hyacin_herk.cpp:45-59, 386-407;
// src/fp_exponent.cu:53-65; src/fp_i63tp_dequantize.cu:29-54, 143-159).  The schedule behind
// hyacinXherkBatch is new.  The reference buckets row segments into a precision ladder, flushes the CRT
// accumulation every 8192 rows through cuBLAS GEMMs into an int32 scratch and reconstructs after every
// flush.  Here every row goes through one CRT pipeline sized for the whole call:
//     for each row chunk (<= 65536 rows):  quantize -> residue Gram (tcgen05), residues accumulate mod m
//     once per call (or per 2^k-row group when the bit budget demands it): Garner reconstruction into C
// The integer Gram C = sum_k q_ky q_kx is exact under either schedule, so results are bit-identical.
#include "hyb_internal.h"
#include "crt_tables.h"
#include <hyacin_b200.h>
#include <algorithm>
#include <vector>
#include <climits>
#include <cmath>

namespace hyb {

static int ceil_log2_u64(uint64_t v) { int l = 0; while (l < 64 && (uint64_t(1) << l) < v) ++l; return l; }

CrtPlan make_crt_plan(int u, int cplx, int64_t rows, bool allow_two_m) {
  CrtPlan p{}; if (u < 0 || rows <= 0) return p;
  p.value_bytes = (u + 9) / 8;                       // |q| <= 2^u must stay below the bias 2^(8 nb - 1)
  auto bits_for = [&](int64_t g) { return 2 * u + 1 + cplx + ceil_log2_u64(uint64_t(g)); };
  if (cplx && allow_two_m && bits_for(rows) <= crt2m::kRangeBits[crt2m::kMaxModuli - 1]) {
    // complex input whose whole call fits the moduli with a square root of -1: half the tensor work
    const int need = bits_for(rows);
    int k = 1; while (k < crt2m::kMaxModuli && crt2m::kRangeBits[k - 1] < need) ++k;
    p.moduli = k; p.group_rows = int(std::min<int64_t>(rows, int64_t(1) << 30)); p.two_m = 1;
    p.chunk_rows = int(std::min<int64_t>(65536, (rows + kStageK - 1) / kStageK * kStageK));
    if (rows <= (int64_t(1) << 30)) return p;
    p = CrtPlan{}; p.value_bytes = (u + 9) / 8;
  }
  int64_t group = rows;
  const int max_bits = crt::kRangeBits[crt::kMaxModuli - 1];
  if (bits_for(group) > max_bits) { group = 1; while (group * 2 <= rows && bits_for(group * 2) <= max_bits) group *= 2; }
  if (group > (int64_t(1) << 30)) group = int64_t(1) << 30;
  auto moduli_for = [&](int64_t g) { const int need = bits_for(g); int k = 1; while (k < crt::kMaxModuli && crt::kRangeBits[k - 1] < need) ++k; return k; };
  // Rows per kernel launch: bounded by the int32 accumulator (a complex operand stacks two parts along K)
  // and by a ~4 GiB residue-plane workspace.
  const int64_t chunk = cplx ? 32768 : 65536;
  // Smaller groups need fewer bits, hence sometimes one modulus less for every row, at the price of one more
  // reconstruction per group (FP32 input at eps 1e-5 over 2^17 rows: 8 moduli and two groups instead of 9 and one).
  // Both costs grow with N^2, so the choice does not depend on N: quantising and multiplying a row costs about
  // 1.25 k units, reconstructing a group as much as 700 k^2 such rows (Garner's k^2 / 2 steps per entry;
  // measured at N = 4096: 0.77 ms per reconstruction with 13 moduli, 6.8 ms of tensor time per modulus and 2^20 rows).
  auto cost = [&](int64_t g) { const int k = moduli_for(g); return 1.25 * k * double(rows) + 700.0 * double((rows + g - 1) / g) * k * k; };
  int64_t best = group;
  for (int64_t g = chunk; g < group; g *= 2)
    if (cost(g) < cost(best) || (g > best && cost(g) == cost(best))) best = g;
  group = best;
  p.moduli = moduli_for(group); p.group_rows = int(group);
  p.chunk_rows = int(std::min<int64_t>(chunk, (group + kStageK - 1) / kStageK * kStageK));
  return p;
}

// ---- status word shared with the kernels (pinned, mapped; written by a kernel only when a wait expires) ----
static uint32_t* g_status_host[64] = {};
static uint32_t* g_status_dev[64] = {};
uint32_t* status_word_device(int device) {
  if (device < 0 || device >= 64) return nullptr;
  if (!g_status_host[device]) {
    uint32_t* h = nullptr;
    if (cudaHostAlloc(reinterpret_cast<void**>(&h), 64, cudaHostAllocMapped) != cudaSuccess) return nullptr;
    *h = 0;
    void* d = nullptr; if (cudaHostGetDevicePointer(&d, h, 0) != cudaSuccess) { cudaFreeHost(h); return nullptr; }
    g_status_host[device] = h; g_status_dev[device] = static_cast<uint32_t*>(d);
  }
  return g_status_dev[device];
}
uint32_t* status_word_if_ready(int device) { return (device >= 0 && device < 64) ? g_status_dev[device] : nullptr; }
uint32_t status_word_read(int device, bool clear) {
  if (device < 0 || device >= 64 || !g_status_host[device]) return 0;
  volatile uint32_t* p = g_status_host[device]; uint32_t v = *p; if (clear) *p = 0; return v;
}
void status_check(const hyacinHandle_t* handle, const char* where) {
  uint32_t v = status_word_read(handle->DeviceID, false);
  if (v) std::fprintf(stderr, "hyacin-b200: ERROR: a bounded wait inside the Gram kernel expired (code %u), seen at %s; "
                              "the integer Gram of that call is invalid\n", v, where);
}

static void herk_crt(const hyacinHandle_t* handle, int64_t rows, int n, hyacinPrecision_t atype, const void* A, int64_t lda, char op,
                     int u, const int32_t* vexp, int beta, int order, uint64_t* C) {
  cudaStream_t stream = handle->cudaStream;
  const int cplx = is_complex(atype), parts = cplx ? 3 : 1;
  const int64_t tri = (int64_t(n) * n + n) / 2;
  CrtPlan plan = make_crt_plan(u, cplx, rows);
  if (plan.moduli == 0) return;
  {
    // keep the residue planes of one chunk within about 8 GiB whatever N and the number of moduli are
    const int64_t per_row = int64_t(plan.two_m ? 2 : parts) * n * plan.moduli;
    const int64_t cap_rows = std::max<int64_t>(8 * kStageK, ((int64_t(8) << 30) / per_row) / kStageK * kStageK);
    plan.chunk_rows = int(std::min<int64_t>(plan.chunk_rows, cap_rows));
  }
  const TilePlan tp = make_tile_plan(n);
  const size_t elem = (base_type(atype) == HYACIN_F64 ? 8 : base_type(atype) == HYACIN_F32 ? 4 : 2) * size_t(cplx ? 2 : 1);
  if (plan.two_m) {
    // X = P^T Q over all tiles, accumulated modulo m across the row chunks; then one pass turns X into the residues
    // of the real and imaginary parts over the upper-triangle tiles, and each is reconstructed into its panel.
    const size_t tile_bytes = size_t(kTileY) * kTileX;
    const size_t full_bytes = size_t(plan.moduli) * tp.tiles_y * tp.tiles_x * tile_bytes, tri_bytes = size_t(plan.moduli) * tp.num_tiles * tile_bytes;
    const size_t wb = size_t(plan.chunk_rows) * 2 * size_t(n) * plan.moduli;
    int8_t* W = nullptr; uint8_t* X = nullptr; uint8_t* R = nullptr;
    HYB_CUDA(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&W), wb, handle->mempool, stream));
    HYB_CUDA(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&X), full_bytes, handle->mempool, stream));
    HYB_CUDA(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&R), 2 * tri_bytes, handle->mempool, stream));
    uint32_t* status = status_word_device(handle->DeviceID);
    if (W && X && R && status) {
      bool first = true;
      for (int64_t c0 = 0; c0 < rows; c0 += plan.chunk_rows) {
        const int rc = int(std::min<int64_t>(plan.chunk_rows, rows - c0));
        const int64_t ldk = (rc + kStageK - 1) / kStageK * kStageK;
        const char* src = static_cast<const char*>(A) + size_t(c0) * elem * (op == 'N' ? 1 : size_t(lda));
        launch_quantize_crt(stream, atype, rc, n, src, lda, vexp, plan, W, ldk, op);
        GramLaunch gl{};
        gl.w = W; gl.ldw = ldk * 2; gl.plane_stride = gl.ldw * n;
        gl.ka0 = 0; gl.kb0 = int(ldk); gl.k_rows = int(ldk); gl.n = n; gl.moduli = plan.moduli;
        gl.accumulate = first ? 0 : 1; gl.sm_count = handle->DeviceSMs; gl.residues = X; gl.status = status;
        gl.full = 1; gl.table = 1;
        launch_gram_residues(stream, gl);
        first = false;
      }
      launch_crt2m_rotate(stream, n, plan.moduli, X, R, R + tri_bytes);
      launch_reconstruct(stream, n, plan.moduli, R, beta, order, C, 1);
      launch_reconstruct(stream, n, plan.moduli, R + tri_bytes, beta, order, C + size_t(order) * tri, 1);
    }
    if (W) HYB_CUDA(cudaFreeAsync(W, stream));
    if (X) HYB_CUDA(cudaFreeAsync(X, stream));
    if (R) HYB_CUDA(cudaFreeAsync(R, stream));
    if (handle->logger) std::fprintf(static_cast<FILE*>(handle->logger), "I8I32-GEMM-COMPLEX [algo=TN,crt-2m,tcgen05] [M=N=%d] [K=%lld] [Order=%d]\n",
                                     n, (long long)rows, plan.moduli);
    return;
  }
  const size_t w_bytes = size_t(plan.chunk_rows) * parts * size_t(n) * plan.moduli;
  const size_t r_bytes = size_t(plan.moduli) * tp.num_tiles * size_t(kTileY) * kTileX;
  int8_t* W = nullptr; uint8_t* R = nullptr;
  HYB_CUDA(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&W), w_bytes, handle->mempool, stream));
  HYB_CUDA(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&R), r_bytes * (cplx ? 2 : 1), handle->mempool, stream));
  uint32_t* status = status_word_device(handle->DeviceID);
  if (!W || !R || !status) { if (W) cudaFreeAsync(W, stream); if (R) cudaFreeAsync(R, stream); return; }

  for (int64_t row = 0; row < rows; row += plan.group_rows) {
    const int64_t g = std::min<int64_t>(plan.group_rows, rows - row);
    bool first = true;
    for (int64_t c0 = 0; c0 < g; c0 += plan.chunk_rows) {
      const int rc = int(std::min<int64_t>(plan.chunk_rows, g - c0));
      const int64_t ldk = (rc + kStageK - 1) / kStageK * kStageK;
      const char* src = static_cast<const char*>(A) + size_t(row + c0) * elem * (op == 'N' ? 1 : size_t(lda));
      launch_quantize_crt(stream, atype, rc, n, src, lda, vexp, plan, W, ldk, op);
      GramLaunch gl{};
      gl.w = W; gl.ldw = ldk * parts; gl.plane_stride = gl.ldw * n;
      gl.ka0 = 0; gl.kb0 = 0; gl.k_rows = int(ldk) * (cplx ? 2 : 1); gl.n = n; gl.moduli = plan.moduli;
      gl.accumulate = first ? 0 : 1; gl.sm_count = handle->DeviceSMs; gl.residues = R; gl.status = status;
      launch_gram_residues(stream, gl);               // real part: (re; im)^T (re; im)
      if (cplx) { gl.kb0 = int(ldk); gl.residues = R + r_bytes; launch_gram_residues(stream, gl); }   // (re; im)^T (im; -re)
      first = false;
    }
    launch_reconstruct(stream, n, plan.moduli, R, beta, order, C);
    if (cplx) launch_reconstruct(stream, n, plan.moduli, R + r_bytes, beta, order, C + size_t(order) * tri);
    beta = 1;
  }
  HYB_CUDA(cudaFreeAsync(W, stream));
  HYB_CUDA(cudaFreeAsync(R, stream));
  if (handle->logger) std::fprintf(static_cast<FILE*>(handle->logger), "I8I32-GEMM-%s [algo=TN,crt,tcgen05] [M=N=%d] [K=%lld] [Order=%d]\n",
                                   cplx ? "COMPLEX" : "REAL", n, (long long)rows, plan.moduli);
}

// Limb route: the quantised values are split into `order` balanced base-256 digits and every digit pair is
// multiplied on the tensor cores; pairs with the same shift share a TMEM accumulator and the epilogue adds it
// into the packed integer Gram at bit 8 (i + j).  order^2 tile products per row chunk against `moduli` for the
// CRT route, so it is the cheaper one only for small bit budgets (and whenever the caller forces it).
static void herk_limbs(const hyacinHandle_t* handle, int64_t rows, int n, hyacinPrecision_t atype, const void* A, int64_t lda, char op,
                       int u, const int32_t* vexp, int beta, int order_c, uint64_t* C) {
  cudaStream_t stream = handle->cudaStream;
  const int cplx = is_complex(atype), parts = cplx ? 3 : 1, kmul = cplx ? 2 : 1;
  const int order = (u + 9) / 8;
  const int64_t tri = (int64_t(n) * n + n) / 2;
  const size_t elem = (base_type(atype) == HYACIN_F64 ? 8 : base_type(atype) == HYACIN_F32 ? 4 : 2) * size_t(cplx ? 2 : 1);
  // order * k_rows * 2^14 < 2^31 for the shared int32 accumulators (k_rows counts both stacked parts of a complex operand)
  int64_t chunk = (131071 / (int64_t(order) * kmul)) / kStageK * kStageK;
  chunk = std::min<int64_t>(chunk, (rows + kStageK - 1) / kStageK * kStageK);
  int8_t* W = nullptr;
  HYB_CUDA(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&W), size_t(chunk) * parts * size_t(n) * order, handle->mempool, stream));
  uint32_t* status = status_word_device(handle->DeviceID);
  if (!W || !status) { if (W) cudaFreeAsync(W, stream); return; }
  int32_t* scratch = nullptr;
  const size_t scratch_bytes = gram_limbs_scratch_bytes(n, order, handle->DeviceSMs);
  if (scratch_bytes) HYB_CUDA(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&scratch), scratch_bytes, handle->mempool, stream));
  bool first = true;
  for (int64_t c0 = 0; c0 < rows; c0 += chunk) {
    const int rc = int(std::min<int64_t>(chunk, rows - c0));
    const int64_t ldk = (rc + kStageK - 1) / kStageK * kStageK;
    const char* src = static_cast<const char*>(A) + size_t(c0) * elem * (op == 'N' ? 1 : size_t(lda));
    launch_quantize_limbs(stream, atype, rc, n, src, lda, vexp, order, W, ldk, op);
    GramLimbLaunch gl{};
    gl.w = W; gl.ldw = ldk * parts; gl.plane_stride = gl.ldw * n; gl.ka0 = 0; gl.kb0 = 0; gl.k_rows = int(ldk) * kmul;
    gl.n = n; gl.order = order; gl.limb_panels = order_c; gl.overwrite = (first && beta == 0) ? 1 : 0;
    gl.sm_count = handle->DeviceSMs; gl.gram = C; gl.status = status; gl.scratch = scratch;
    launch_gram_limbs(stream, gl);
    if (cplx) { gl.kb0 = int(ldk); gl.gram = C + size_t(order_c) * tri; launch_gram_limbs(stream, gl); }
    first = false;
  }
  HYB_CUDA(cudaFreeAsync(W, stream));
  if (scratch) HYB_CUDA(cudaFreeAsync(scratch, stream));
  if (handle->logger) std::fprintf(static_cast<FILE*>(handle->logger), "I8I32-GEMM-%s [algo=TN,limbs,tcgen05] [M=N=%d] [K=%lld] [Order=%d]\n",
                                   cplx ? "COMPLEX" : "REAL", n, (long long)rows, order);
}

// 'L' forces limbs, 'C' forces CRT; otherwise the route with fewer tile products per row chunk is taken.
static bool use_limb_route(char algorithm, int u, int cplx, int64_t rows);

// Integer Gram of op(A) (rows x n): the body of hyacinXherkBatch, with the transposed layouts the fits pass in.
static bool use_limb_route(char algorithm, int u, int cplx, int64_t rows);

static void herk_rows(const hyacinHandle_t* handle, int64_t rows, int n, hyacinPrecision_t atype, const void* A, int64_t lda, char op,
                      int u, const int32_t* vexp, int beta, int order_c, uint64_t* C) {
  const int cplx = is_complex(atype);
  if (use_limb_route(handle->GramMatrixAlgorithm, u, cplx, rows)) herk_limbs(handle, rows, n, atype, A, lda, op, u, vexp, beta ? 1 : 0, order_c, C);
  else herk_crt(handle, rows, n, atype, A, lda, op, u, vexp, beta ? 1 : 0, order_c, C);
}

// Precision ladder over row segments (reference: src/fp_exponent.cu:67-76 and the bucketing of
// src/hyacin_herk.cpp:316-338): a segment whose column maxima all lie d bits below the global ones only holds
// values |q| <= 2^(u - d), so its share of the Gram needs fewer moduli (or digit planes) and fewer bytes per value;
// a segment of zeros needs nothing.  The bits per segment come back through one small device-to-host copy (the
// reference has the same pipeline bubble).  Consecutive segments of one precision level form a run; every run
// is an independent exact contribution added with beta = 1, so the result does not depend on the split.
// Returns false when there is nothing to gain (every segment at the top level), and the caller runs the plain path.
static bool herk_ladder(const hyacinHandle_t* handle, int64_t rows, int batches, int64_t seg_m, int n, hyacinPrecision_t atype,
                        const void* A, int64_t lda, char op, int u, const int32_t* vexp, int beta, int order_c, uint64_t* C) {
  const int cplx = is_complex(atype);
  cudaStream_t stream = handle->cudaStream;
  int32_t* seg_dev = nullptr;
  HYB_CUDA(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&seg_dev), size_t(batches) * sizeof(int32_t), handle->mempool, stream));
  if (!seg_dev) return false;
  std::vector<int32_t> seg_u(batches);
  launch_vector_range(stream, batches, n, u, vexp, seg_dev);
  HYB_CUDA(cudaMemcpyAsync(seg_u.data(), seg_dev, size_t(batches) * sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
  HYB_CUDA(cudaStreamSynchronize(stream));
  HYB_CUDA(cudaFreeAsync(seg_dev, stream));
  // precision level of a segment: 0 = nothing to do, otherwise the bit budget rounded up to a multiple of 8 (one
  // value byte, about one modulus per 4 bits); the top level is that of u itself
  auto level_of = [&](int32_t bits) { return bits < 0 ? 0 : std::min((bits + 8) / 8, (u + 8) / 8); };
  const int top = level_of(u);
  struct Run { int64_t row0, rows; int level, bits; };
  std::vector<Run> runs;
  bool gain = false;
  for (int b = 0; b < batches; ++b) {
    const int64_t r0 = int64_t(b) * seg_m, r1 = std::min<int64_t>(rows, r0 + seg_m);
    if (r1 <= r0) break;
    const int32_t bits = seg_u[b] == INT_MIN ? -1 : std::min<int32_t>(seg_u[b], u);
    const int level = level_of(bits);
    if (level < top) gain = true;
    if (!runs.empty() && runs.back().level == level) { runs.back().rows += r1 - r0; runs.back().bits = std::max(runs.back().bits, int(bits)); }
    else runs.push_back(Run{r0, r1 - r0, level, int(bits)});
  }
  if (!gain || runs.size() > 16) return false;               // nothing to save, or too fragmented to be worth a reconstruction per run
  {
    // Worth it?  Work is counted in rows x moduli; every extra run costs one more reconstruction, about as much as
    // 100 000 row-moduli of quantisation and Gram.
    const int k_top = make_crt_plan(u, cplx, rows).moduli;
    int64_t saved = 0; int executed = 0;
    for (const Run& r : runs) {
      const int k_run = r.level == 0 ? 0 : make_crt_plan(std::max(r.bits, 0), cplx, r.rows).moduli;
      saved += r.rows * int64_t(std::max(0, k_top - k_run));
      executed += r.level != 0;
    }
    if (saved <= int64_t(100000) * std::max(0, executed - 1)) return false;
  }
  const size_t elem = (base_type(atype) == HYACIN_F64 ? 8 : base_type(atype) == HYACIN_F32 ? 4 : 2) * size_t(cplx ? 2 : 1);
  bool any = false;
  for (const Run& r : runs) {
    if (r.level == 0) continue;
    const char* src = static_cast<const char*>(A) + size_t(r.row0) * elem * (op == 'N' ? 1 : size_t(lda));
    herk_rows(handle, r.rows, n, atype, src, lda, op, std::max(r.bits, 0), vexp, (beta || any) ? 1 : 0, order_c, C);
    any = true;
  }
  if (!any && beta == 0) {
    const uint64_t tri = (uint64_t(n) * n + n) / 2;
    HYB_CUDA(cudaMemsetAsync(C, 0, tri * uint64_t(order_c) * (1 + cplx) * sizeof(uint64_t), stream));
  }
  if (handle->logger) std::fprintf(static_cast<FILE*>(handle->logger), "I8I32-LADDER [segments=%d] [runs=%d] [top-bits=%d]\n", batches, int(runs.size()), u);
  return true;
}

void herk_any(const hyacinHandle_t* handle, int64_t rows, int n, hyacinPrecision_t atype, const void* A, int64_t lda, char op,
              int u, const int32_t* vexp, int beta, int order_c, uint64_t* C, int batches, int64_t seg_m) {
  const int cplx = is_complex(atype);
  if (n > 65535) {
    // launch grids index columns with a 16-bit block coordinate; a Gram of that size (> 68 GB of limbs) is out of reach anyway
    std::fprintf(stderr, "hyacin-b200: N = %d exceeds the supported 65535 columns; nothing computed\n", n);
    return;
  }
  if (rows <= 0 || u < 0) {
    // Nothing to add: an overwrite still has to define C (src/hyacin_herk.cpp:287).
    if (beta == 0) {
      const uint64_t tri = (uint64_t(n) * n + n) / 2;
      HYB_CUDA(cudaMemsetAsync(C, 0, tri * uint64_t(order_c) * (1 + cplx) * sizeof(uint64_t), handle->cudaStream));
    }
    return;
  }
  if (batches > 1 && seg_m > 0 && herk_ladder(handle, rows, batches, seg_m, n, atype, A, lda, op, u, vexp, beta, order_c, C)) return;
  herk_rows(handle, rows, n, atype, A, lda, op, u, vexp, beta, order_c, C);
}

static bool use_limb_route(char algorithm, int u, int cplx, int64_t rows) {
  if (algorithm == 'L' || algorithm == 'l') return true;
  if (algorithm == 'C' || algorithm == 'c') return false;
  const int order = (u + 9) / 8;
  return order * order < make_crt_plan(u, cplx, rows, false).moduli;
}

}  // namespace hyb

extern "C" void hyacinXherkBatchInit(const hyacinHandle_t* handle, double eps, uint64_t M, int32_t N, hyacinPrecision_t Atype,
                                     int32_t* uA, int32_t* cPanels, int32_t* lPanels, uint64_t* stride) {
  if (stride) { const uint64_t n = uint64_t(std::max(0, N)); *stride = (n * n + n) >> 1; }
  if (!uA && !cPanels && !lPanels) return;
  if (int(Atype) < 0 || int(Atype) > 11) return;
  static const int mantissa[12] = {52, 52, 23, 23, 10, 10, 105, 105, 71, 71, 95, 95};
  const int log2m = M > 1 ? hyb::ceil_log2_u64(M) : 0;       // log2 of the row count rounded up to a power of two
  int e = 0; const double f = std::frexp(std::fabs(eps), &e);
  const int u = std::min(std::max((f == 0.5 ? 1 : 0) - e, 0), mantissa[int(Atype)]);
  const int cplx = hyb::is_complex(Atype);
  const int u_corr = std::max(-1, std::min(80, handle->QuantizeBitCorrection + u));
  if (uA) *uA = u_corr;
  if (cPanels) *cPanels = 1 + cplx;
  if (lPanels) *lPanels = u_corr >= 0 ? (63 + std::max(0, 2 * (u_corr + cplx)) + log2m) / 63 : 0;
}

extern "C" void hyacinXquantizeScaleBatch(const hyacinHandle_t* handle, int32_t batches, int32_t segM, int32_t lastM, int32_t N,
                                          hyacinPrecision_t Atype, const void* A, int32_t lda, int32_t uA, int32_t* vexp) {
  if (N <= 0 || int(Atype) < 0 || int(Atype) > int(HYACIN_F16_COMPLEX)) return;
  hyb::timer_mark(handle, hyb::Segment::Distributed);
  hyb::launch_column_exponents(handle->cudaStream, Atype, batches, segM, lastM, N, A, lda, uA, vexp);
}

extern "C" void hyacinXherkBatch(const hyacinHandle_t* handle, int32_t batches, int32_t segM, int32_t lastM, int32_t N,
                                 hyacinPrecision_t Atype, const void* A, int32_t lda, int32_t u, const int32_t* vexp,
                                 int32_t beta, int32_t orderC, uint64_t* C) {
  if (N <= 0 || orderC <= 0 || orderC > 3) return;
  if (int(Atype) < 0 || int(Atype) > int(HYACIN_F16_COMPLEX)) return;
  hyb::timer_mark(handle, hyb::Segment::Distributed);
  const int64_t rows = batches <= 1 ? int64_t(lastM) : int64_t(batches - 1) * segM + lastM;
  hyb::herk_any(handle, rows, N, Atype, A, lda, 'N', u, vexp, beta, orderC, C, batches, segM);
}

namespace hyb {
hyacinPrecision_t gram_type_from_bits(const hyacinHandle_t* handle, int raw_bits, hyacinPrecision_t atype) {
  const int bits = raw_bits - 2 * handle->QuantizeBitCorrection;
  const bool wide_fp64 = handle->DeviceIsF64Capable != 0;
  hyacinPrecision_t g = bits <= 23 ? HYACIN_F32_COMPLEX
                      : bits <= 52 ? HYACIN_F64_COMPLEX
                      : (bits <= 71 && !wide_fp64) ? HYACIN_TF_COMPLEX
                      : (bits <= 95 && !wide_fp64) ? HYACIN_QF_COMPLEX : HYACIN_DD_COMPLEX;
  if (!is_complex(atype)) g = hyacinPrecision_t(int(g) - 1);
  return g;
}
}  // namespace hyb

extern "C" void hyacinXdequantizeInit(const hyacinHandle_t* handle, int32_t N, int32_t orderC, const uint64_t* C, const int32_t* vexp,
                                      hyacinPrecision_t Atype, hyacinPrecision_t* Gtype, int32_t* gElemBytes) {
  if (N <= 0 && (Gtype != nullptr || gElemBytes != nullptr)) return;
  if (int(Atype) < 0 || int(Atype) > 11) return;
  hyb::timer_mark(handle, hyb::Segment::Replicated);
  int32_t* bits_host = static_cast<int32_t*>(handle->pinnedWorkspace);
  *bits_host = 0;
  hyb::launch_gram_range(handle->cudaStream, N, orderC, C, vexp, bits_host);
  HYB_CUDA(cudaStreamSynchronize(handle->cudaStream));
  hyb::status_check(handle, "hyacinXdequantizeInit");
  static const int bytes[12] = {8, 16, 4, 8, 2, 4, 16, 32, 12, 24, 16, 32};
  const hyacinPrecision_t g = hyb::gram_type_from_bits(handle, *bits_host, Atype);
  if (Gtype) *Gtype = g;
  if (gElemBytes) *gElemBytes = bytes[int(g)];
}

extern "C" void hyacinXdequantize(const hyacinHandle_t* handle, int32_t N, int32_t orderC, const uint64_t* C, const int32_t* vexp,
                                  hyacinPrecision_t Gtype, void* G, int32_t ldg) {
  if (N <= 0) return;
  hyb::timer_mark(handle, hyb::Segment::Replicated);
  hyb::launch_dequantize(handle->cudaStream, N, orderC, C, vexp, Gtype, G, ldg);
}

// ---- stage-level entry points of this build (declared in hyacin_b200.h) ---------------------------------
extern "C" uint32_t hyacinB200Status(int32_t clear) {
  int dev = 0; if (cudaGetDevice(&dev) != cudaSuccess) return 0xFFFFFFFFu;
  return hyb::status_word_read(dev, clear != 0);
}

extern "C" void hyacinB200CrtPlan(int32_t u, int32_t Complex, int64_t rows, int32_t* moduli, int32_t* valueBytes,
                                  int32_t* groupRows, int32_t* chunkRows) {
  const hyb::CrtPlan p = hyb::make_crt_plan(u, Complex ? 1 : 0, rows, false);     // the stage hooks keep the three-part complex layout
  if (moduli) *moduli = p.moduli; if (valueBytes) *valueBytes = p.value_bytes;
  if (groupRows) *groupRows = p.group_rows; if (chunkRows) *chunkRows = p.chunk_rows;
}

extern "C" void hyacinB200VectorRange(const hyacinHandle_t* handle, int32_t batches, int32_t N, int32_t u, const int32_t* vexp, int32_t* segU) {
  if (batches <= 0 || N <= 0) return;
  hyb::launch_vector_range(handle->cudaStream, batches, N, u, vexp, segU);
}

extern "C" int32_t hyacinB200GramItem(int32_t tilesX, int32_t pairRows, int32_t full, int32_t moduli, int32_t pairs, int32_t pair, int32_t k,
                                      int32_t* modulus, int32_t* tileRow, int32_t* tileCol, int32_t* width) {
  int m = 0, ty = 0, tx = 0, w = 0;
  if (!hyb::gram_schedule_item(tilesX, pairRows, full, moduli, pairs, pair, k, &m, &ty, &tx, &w)) return 0;
  if (modulus) *modulus = m; if (tileRow) *tileRow = ty; if (tileCol) *tileCol = tx; if (width) *width = w;
  return 1;
}

extern "C" void hyacinB200TileInfo(int32_t N, int32_t* tileY, int32_t* tileX, int32_t* tilesY, int32_t* numTiles) {
  const hyb::TilePlan tp = hyb::make_tile_plan(N);
  if (tileY) *tileY = hyb::kTileY; if (tileX) *tileX = hyb::kTileX;
  if (tilesY) *tilesY = tp.tiles_y; if (numTiles) *numTiles = tp.num_tiles;
}

extern "C" void hyacinB200QuantizeCrt(const hyacinHandle_t* handle, hyacinPrecision_t Atype, int32_t rows, int32_t N, const void* A,
                                      int32_t lda, const int32_t* vexp, int32_t moduli, int32_t valueBytes, int8_t* W, int64_t ldk) {
  if (N <= 0 || rows < 0 || moduli <= 0 || moduli > hyb::crt::kMaxModuli || valueBytes < 1 || valueBytes > hyb::crt::kMaxBytes) return;
  if (int(Atype) < 0 || int(Atype) > int(HYACIN_F16_COMPLEX) || ldk % hyb::kStageK) return;
  hyb::CrtPlan p{}; p.moduli = moduli; p.value_bytes = valueBytes;
  hyb::launch_quantize_crt(handle->cudaStream, Atype, rows, N, A, lda, vexp, p, W, ldk);
}

extern "C" void hyacinB200GramResidues(const hyacinHandle_t* handle, int32_t N, int32_t moduli, const int8_t* W, int64_t ldw,
                                       int64_t planeStride, int32_t ka0, int32_t kb0, int32_t kRows, int32_t accumulate,
                                       uint8_t* residues) {
  if (N <= 0 || moduli <= 0 || moduli > hyb::crt::kMaxModuli || kRows <= 0) return;
  if (kRows % hyb::kStageK || ka0 % hyb::kStageK || kb0 % hyb::kStageK || ldw % 16 || planeStride % 16 || kRows > hyb::kMaxAccumRows) return;
  hyb::GramLaunch g{};
  g.w = W; g.ldw = ldw; g.plane_stride = planeStride; g.ka0 = ka0; g.kb0 = kb0; g.k_rows = kRows; g.n = N; g.moduli = moduli;
  g.accumulate = accumulate ? 1 : 0; g.sm_count = handle->DeviceSMs; g.residues = residues;
  g.status = hyb::status_word_device(handle->DeviceID);
  if (!g.status) return;
  hyb::launch_gram_residues(handle->cudaStream, g);
}

extern "C" void hyacinB200Reconstruct(const hyacinHandle_t* handle, int32_t N, int32_t moduli, const uint8_t* residues, int32_t beta,
                                      int32_t orderC, uint64_t* Cpanel) {
  if (N <= 0 || moduli <= 0 || moduli > hyb::crt::kMaxModuli || orderC <= 0 || orderC > 3) return;
  hyb::launch_reconstruct(handle->cudaStream, N, moduli, residues, beta ? 1 : 0, orderC, Cpanel);
}

extern "C" void hyacinB200DequantizeViaSlices(const hyacinHandle_t* handle, int32_t N, int32_t orderC, const uint64_t* C, const int32_t* vexp,
                                             hyacinPrecision_t Atype, int32_t ranks, hyacinPrecision_t* Gtype, void* G, int32_t ldg) {
  if (N <= 0 || orderC <= 0 || orderC > 3 || ranks < 1 || int(Atype) < 0 || int(Atype) > 11 || !Gtype) return;
  cudaStream_t stream = handle->cudaStream;
  const int panels = 1 + hyb::is_complex(Atype);
  const uint64_t tri = (uint64_t(N) * N + N) / 2;
  int slices = 0, width = 0; hyb::slice_layout(orderC, ranks, &slices, &width);
  uint64_t* S = nullptr;
  HYB_CUDA(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&S), uint64_t(panels) * slices * tri * sizeof(uint64_t), handle->mempool, stream));
  if (!S) return;
  hyb::launch_limbs_to_slices(stream, panels, orderC, ranks, tri, C, S);
  int32_t* bits_host = static_cast<int32_t*>(handle->pinnedWorkspace);
  *bits_host = 0;
  hyb::launch_gram_range_slices(stream, N, orderC, ranks, S, vexp, bits_host);
  HYB_CUDA(cudaStreamSynchronize(stream));
  *Gtype = hyb::gram_type_from_bits(handle, *bits_host, Atype);
  if (G) hyb::launch_dequantize_slices(stream, N, orderC, ranks, S, vexp, *Gtype, G, ldg);
  HYB_CUDA(cudaFreeAsync(S, stream));
}

extern "C" void hyacinB200QuantizeLimbs(const hyacinHandle_t* handle, hyacinPrecision_t Atype, int32_t rows, int32_t N, const void* A,
                                        int32_t lda, const int32_t* vexp, int32_t order, int8_t* W, int64_t ldk) {
  if (N <= 0 || rows < 0 || order < 1 || order > hyb::crt::kMaxBytes || ldk % hyb::kStageK) return;
  if (int(Atype) < 0 || int(Atype) > int(HYACIN_F16_COMPLEX)) return;
  hyb::launch_quantize_limbs(handle->cudaStream, Atype, rows, N, A, lda, vexp, order, W, ldk);
}

extern "C" void hyacinB200GramLimbs(const hyacinHandle_t* handle, int32_t N, int32_t order, const int8_t* W, int64_t ldw,
                                    int64_t planeStride, int32_t ka0, int32_t kb0, int32_t kRows, int32_t beta, int32_t orderC,
                                    uint64_t* Cpanel) {
  if (N <= 0 || order < 1 || order > hyb::crt::kMaxBytes || kRows <= 0 || orderC < 1 || orderC > 3) return;
  if (kRows % hyb::kStageK || ka0 % hyb::kStageK || kb0 % hyb::kStageK || ldw % 16 || planeStride % 16) return;
  if (int64_t(order) * kRows > 131071) return;
  hyb::GramLimbLaunch g{};
  g.w = W; g.ldw = ldw; g.plane_stride = planeStride; g.ka0 = ka0; g.kb0 = kb0; g.k_rows = kRows; g.n = N; g.order = order;
  g.limb_panels = orderC; g.overwrite = beta ? 0 : 1; g.sm_count = handle->DeviceSMs; g.gram = Cpanel;
  g.status = hyb::status_word_device(handle->DeviceID);
  if (!g.status) return;
  hyb::launch_gram_limbs(handle->cudaStream, g);
}
