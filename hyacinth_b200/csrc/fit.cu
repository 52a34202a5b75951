// Fitting drivers and the replicated factorisation of the Gram matrix.
//
// The call sequences are the reference's (src/lra.cpp:18-156 for the three fits, src/gram_evd.cu:94-194 for
// Gram -> SVD basis, src/gram_id.cpp:28-101 for Gram -> interpolation basis, src/lra.cpp:158-208 for the
// projection-error check); cuSOLVER and cuBLAS do the dense linear algebra exactly as there.  What differs is
// the plumbing around this build's Cholesky factor layout (tail.h) and that library status codes are checked.
#include "hyb_internal.h"
#include "tail.h"
#include <cuda_fp16.h>
#include <algorithm>
#include <cfloat>
#include <cmath>
#include <numeric>
#include <vector>

namespace hyb {
namespace {

void report_status(int status, const char* what) { if (status != 0) std::fprintf(stderr, "hyacin-b200: %s failed with status %d\n", what, status); }
#define HYB_LIB(call) ::hyb::report_status(int(call), #call)

template <typename T> T* pool_alloc(const hyacinHandle_t* h, size_t count) {
  T* p = nullptr; HYB_CUDA(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&p), std::max<size_t>(count, 1) * sizeof(T), h->mempool, h->cudaStream)); return p;
}
void pool_free(const hyacinHandle_t* h, void* p) { if (p) HYB_CUDA(cudaFreeAsync(p, h->cudaStream)); }

// Library element type of a storage type: double stays double, float and half compute in float.
hyacinPrecision_t lib_type(hyacinPrecision_t t) { return hyacinPrecision_t((base_type(t) == HYACIN_F64 ? HYACIN_F64 : HYACIN_F32) | is_complex(t)); }
hyacinPrecision_t real_of(hyacinPrecision_t t) { return hyacinPrecision_t(base_type(t)); }
size_t elem_bytes(hyacinPrecision_t t) { return gram_elem_bytes(t); }

// ---- typed cuSOLVER / cuBLAS front ends ------------------------------------------------------------------
int gesvdj(const hyacinHandle_t* h, hyacinPrecision_t lt, int m, int n, void* A, void* S, void* U, void* V, int sweeps, double tol) {
  cusolverDnHandle_t s = h->cusolverHandle; gesvdjInfo_t params = nullptr; int lwork = 0;
  HYB_LIB(cusolverDnCreateGesvdjInfo(&params));
  HYB_LIB(cusolverDnXgesvdjSetTolerance(params, tol));
  HYB_LIB(cusolverDnXgesvdjSetMaxSweeps(params, sweeps));
  int* info = pool_alloc<int>(h, 1); void* work = nullptr;
  const cusolverEigMode_t jobz = CUSOLVER_EIG_MODE_VECTOR;
  switch (int(lt)) {
    case HYACIN_F64:
      HYB_LIB(cusolverDnDgesvdj_bufferSize(s, jobz, 1, m, n, (double*)A, m, (double*)S, (double*)U, m, (double*)V, n, &lwork, params));
      work = pool_alloc<double>(h, lwork);
      HYB_LIB(cusolverDnDgesvdj(s, jobz, 1, m, n, (double*)A, m, (double*)S, (double*)U, m, (double*)V, n, (double*)work, lwork, info, params)); break;
    case HYACIN_F32:
      HYB_LIB(cusolverDnSgesvdj_bufferSize(s, jobz, 1, m, n, (float*)A, m, (float*)S, (float*)U, m, (float*)V, n, &lwork, params));
      work = pool_alloc<float>(h, lwork);
      HYB_LIB(cusolverDnSgesvdj(s, jobz, 1, m, n, (float*)A, m, (float*)S, (float*)U, m, (float*)V, n, (float*)work, lwork, info, params)); break;
    case HYACIN_F64_COMPLEX:
      HYB_LIB(cusolverDnZgesvdj_bufferSize(s, jobz, 1, m, n, (cuDoubleComplex*)A, m, (double*)S, (cuDoubleComplex*)U, m, (cuDoubleComplex*)V, n, &lwork, params));
      work = pool_alloc<cuDoubleComplex>(h, lwork);
      HYB_LIB(cusolverDnZgesvdj(s, jobz, 1, m, n, (cuDoubleComplex*)A, m, (double*)S, (cuDoubleComplex*)U, m, (cuDoubleComplex*)V, n, (cuDoubleComplex*)work, lwork, info, params)); break;
    case HYACIN_F32_COMPLEX:
      HYB_LIB(cusolverDnCgesvdj_bufferSize(s, jobz, 1, m, n, (cuComplex*)A, m, (float*)S, (cuComplex*)U, m, (cuComplex*)V, n, &lwork, params));
      work = pool_alloc<cuComplex>(h, lwork);
      HYB_LIB(cusolverDnCgesvdj(s, jobz, 1, m, n, (cuComplex*)A, m, (float*)S, (cuComplex*)U, m, (cuComplex*)V, n, (cuComplex*)work, lwork, info, params)); break;
    default: break;
  }
  pool_free(h, work); pool_free(h, info);
  HYB_LIB(cusolverDnDestroyGesvdjInfo(params));
  return 0;
}

int gesvd(const hyacinHandle_t* h, hyacinPrecision_t lt, int m, int n, void* A, void* S, void* U) {
  cusolverDnHandle_t s = h->cusolverHandle; int lwork = 0; int* info = pool_alloc<int>(h, 1); void* work = nullptr; void* rwork = nullptr;
  switch (int(lt)) {
    case HYACIN_F64:
      HYB_LIB(cusolverDnDgesvd_bufferSize(s, m, n, &lwork)); work = pool_alloc<double>(h, lwork); rwork = pool_alloc<double>(h, n);
      HYB_LIB(cusolverDnDgesvd(s, 'S', 'N', m, n, (double*)A, m, (double*)S, (double*)U, m, nullptr, n, (double*)work, lwork, (double*)rwork, info)); break;
    case HYACIN_F32:
      HYB_LIB(cusolverDnSgesvd_bufferSize(s, m, n, &lwork)); work = pool_alloc<float>(h, lwork); rwork = pool_alloc<float>(h, n);
      HYB_LIB(cusolverDnSgesvd(s, 'S', 'N', m, n, (float*)A, m, (float*)S, (float*)U, m, nullptr, n, (float*)work, lwork, (float*)rwork, info)); break;
    case HYACIN_F64_COMPLEX:
      HYB_LIB(cusolverDnZgesvd_bufferSize(s, m, n, &lwork)); work = pool_alloc<cuDoubleComplex>(h, lwork); rwork = pool_alloc<double>(h, n);
      HYB_LIB(cusolverDnZgesvd(s, 'S', 'N', m, n, (cuDoubleComplex*)A, m, (double*)S, (cuDoubleComplex*)U, m, nullptr, n, (cuDoubleComplex*)work, lwork, (double*)rwork, info)); break;
    case HYACIN_F32_COMPLEX:
      HYB_LIB(cusolverDnCgesvd_bufferSize(s, m, n, &lwork)); work = pool_alloc<cuComplex>(h, lwork); rwork = pool_alloc<float>(h, n);
      HYB_LIB(cusolverDnCgesvd(s, 'S', 'N', m, n, (cuComplex*)A, m, (float*)S, (cuComplex*)U, m, nullptr, n, (cuComplex*)work, lwork, (float*)rwork, info)); break;
    default: break;
  }
  pool_free(h, work); pool_free(h, rwork); pool_free(h, info);
  return 0;
}

void trsm_upper_left(const hyacinHandle_t* h, hyacinPrecision_t lt, int m, int n, void* R, int ldr) {
  cublasHandle_t b = h->cublasHandle; const size_t off = size_t(m) * ldr;
  switch (int(lt)) {
    case HYACIN_F64: { double one = 1.; HYB_LIB(cublasDtrsm(b, CUBLAS_SIDE_LEFT, CUBLAS_FILL_MODE_UPPER, CUBLAS_OP_N, CUBLAS_DIAG_NON_UNIT, m, n, &one, (double*)R, ldr, (double*)R + off, ldr)); break; }
    case HYACIN_F32: { float one = 1.f; HYB_LIB(cublasStrsm(b, CUBLAS_SIDE_LEFT, CUBLAS_FILL_MODE_UPPER, CUBLAS_OP_N, CUBLAS_DIAG_NON_UNIT, m, n, &one, (float*)R, ldr, (float*)R + off, ldr)); break; }
    case HYACIN_F64_COMPLEX: { cuDoubleComplex one = make_cuDoubleComplex(1., 0.); HYB_LIB(cublasZtrsm(b, CUBLAS_SIDE_LEFT, CUBLAS_FILL_MODE_UPPER, CUBLAS_OP_N, CUBLAS_DIAG_NON_UNIT, m, n, &one, (cuDoubleComplex*)R, ldr, (cuDoubleComplex*)R + off, ldr)); break; }
    case HYACIN_F32_COMPLEX: { cuComplex one = make_cuComplex(1.f, 0.f); HYB_LIB(cublasCtrsm(b, CUBLAS_SIDE_LEFT, CUBLAS_FILL_MODE_UPPER, CUBLAS_OP_N, CUBLAS_DIAG_NON_UNIT, m, n, &one, (cuComplex*)R, ldr, (cuComplex*)R + off, ldr)); break; }
    default: break;
  }
}

// C (m x n) = op(A) (m x k) * B (k x n) in the storage type t, compute modes as in src/lra.cpp:86-110.
bool stage_gemm(const hyacinHandle_t* h, hyacinPrecision_t t, char op, int m, int n, int k, const void* A, int lda, const void* B, int ldb, void* C, int ldc) {
  cublasHandle_t b = h->cublasHandle;
  const cublasOperation_t opa = op == 'C' ? (is_complex(t) ? CUBLAS_OP_C : CUBLAS_OP_T) : op == 'T' ? CUBLAS_OP_T : CUBLAS_OP_N;
  switch (int(t)) {
    case HYACIN_F64: { double one = 1., zero = 0.; HYB_LIB(cublasDgemm(b, opa, CUBLAS_OP_N, m, n, k, &one, (const double*)A, lda, (const double*)B, ldb, &zero, (double*)C, ldc)); return true; }
    case HYACIN_F32: {
      // The emulated mode is the reference's (src/lra.cpp:92); the library refuses it for some leading dimensions and
      // offsets (status NOT_SUPPORTED), where the reference carries on with an unwritten product.  Plain FP32 then.
      float one = 1.f, zero = 0.f;
      if (cublasGemmEx(b, opa, CUBLAS_OP_N, m, n, k, &one, A, CUDA_R_32F, lda, B, CUDA_R_32F, ldb, &zero, C, CUDA_R_32F, ldc, CUBLAS_COMPUTE_32F_EMULATED_16BFX9, CUBLAS_GEMM_DEFAULT) != CUBLAS_STATUS_SUCCESS)
        HYB_LIB(cublasGemmEx(b, opa, CUBLAS_OP_N, m, n, k, &one, A, CUDA_R_32F, lda, B, CUDA_R_32F, ldb, &zero, C, CUDA_R_32F, ldc, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT));
      return true;
    }
    case HYACIN_F16: { __half one = __float2half(1.f), zero = __float2half(0.f); HYB_LIB(cublasGemmEx(b, opa, CUBLAS_OP_N, m, n, k, &one, A, CUDA_R_16F, lda, B, CUDA_R_16F, ldb, &zero, C, CUDA_R_16F, ldc, CUBLAS_COMPUTE_16F, CUBLAS_GEMM_DEFAULT)); return true; }
    case HYACIN_F64_COMPLEX: { cuDoubleComplex one = make_cuDoubleComplex(1., 0.), zero = make_cuDoubleComplex(0., 0.); HYB_LIB(cublasZgemm(b, opa, CUBLAS_OP_N, m, n, k, &one, (const cuDoubleComplex*)A, lda, (const cuDoubleComplex*)B, ldb, &zero, (cuDoubleComplex*)C, ldc)); return true; }
    case HYACIN_F32_COMPLEX: {
      cuComplex one = make_cuComplex(1.f, 0.f), zero = make_cuComplex(0.f, 0.f);
      if (cublasGemmEx(b, opa, CUBLAS_OP_N, m, n, k, &one, A, CUDA_C_32F, lda, B, CUDA_C_32F, ldb, &zero, C, CUDA_C_32F, ldc, CUBLAS_COMPUTE_32F_EMULATED_16BFX9, CUBLAS_GEMM_DEFAULT) != CUBLAS_STATUS_SUCCESS)
        HYB_LIB(cublasGemmEx(b, opa, CUBLAS_OP_N, m, n, k, &one, A, CUDA_C_32F, lda, B, CUDA_C_32F, ldb, &zero, C, CUDA_C_32F, ldc, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT));
      return true;
    }
    case HYACIN_F16_COMPLEX: {
      // The library has no complex-half GEMM: split into planes and use two real GEMMs per block of 8192 rows,
      //   [C_re | C_im] = A_re [B_re | B_im] + A_im [-B_im | B_re].
      // Operand layouts, padding of K to a multiple of 8, leading dimensions and the half-precision compute type are
      // those of src/matmul_fp16_complex.cu (planes of a stored-transposed A stay K-major and enter with op T), so that
      // cuBLAS is asked for the very same products and returns the same bits.
      const int block = 8192, ak = (k + 7) & ~7;
      const bool stored_t = op == 'T' || op == 'C';
      const size_t plane_a = size_t(block) * ak, plane_b = size_t(ak) * n, plane_c = size_t(block) * n;
      __half* bp = pool_alloc<__half>(h, 3 * plane_b);
      __half* ap = pool_alloc<__half>(h, 2 * plane_a);
      __half* cp = pool_alloc<__half>(h, 2 * plane_c);
      HYB_CUDA(cudaMemsetAsync(bp, 0, 3 * plane_b * sizeof(__half), h->cudaStream));       // the padding rows K .. ak - 1 stay zero
      HYB_CUDA(cudaMemsetAsync(ap, 0, 2 * plane_a * sizeof(__half), h->cudaStream));
      split_complex_half_b(h->cudaStream, k, n, B, ldb, bp, ak);
      const __half one = __float2half(1.f), zero = __float2half(0.f);
      for (int i = 0; i < m; i += block) {
        const int rows = std::min(block, m - i);
        if (stored_t) {
          // stored K x M: columns i .. i + rows - 1, planes [kk + r ak]
          split_complex_half_stored(h->cudaStream, op == 'C', k, rows, static_cast<const char*>(A) + size_t(i) * lda * 4, lda, ap, ap + plane_a, ak);
          HYB_LIB(cublasGemmEx(b, CUBLAS_OP_T, CUBLAS_OP_N, rows, 2 * n, ak, &one, ap, CUDA_R_16F, ak, bp + plane_b, CUDA_R_16F, ak, &zero, cp, CUDA_R_16F, block, CUBLAS_COMPUTE_16F, CUBLAS_GEMM_DEFAULT));
          HYB_LIB(cublasGemmEx(b, CUBLAS_OP_T, CUBLAS_OP_N, rows, 2 * n, ak, &one, ap + plane_a, CUDA_R_16F, ak, bp, CUDA_R_16F, ak, &one, cp, CUDA_R_16F, block, CUBLAS_COMPUTE_16F, CUBLAS_GEMM_DEFAULT));
        } else {
          // stored M x K: rows i .. i + rows - 1, planes [r + kk block]
          split_complex_half_stored(h->cudaStream, false, rows, k, static_cast<const char*>(A) + size_t(i) * 4, lda, ap, ap + plane_a, block);
          HYB_LIB(cublasGemmEx(b, CUBLAS_OP_N, CUBLAS_OP_N, rows, 2 * n, ak, &one, ap, CUDA_R_16F, block, bp + plane_b, CUDA_R_16F, ak, &zero, cp, CUDA_R_16F, block, CUBLAS_COMPUTE_16F, CUBLAS_GEMM_DEFAULT));
          HYB_LIB(cublasGemmEx(b, CUBLAS_OP_N, CUBLAS_OP_N, rows, 2 * n, ak, &one, ap + plane_a, CUDA_R_16F, block, bp, CUDA_R_16F, ak, &one, cp, CUDA_R_16F, block, CUBLAS_COMPUTE_16F, CUBLAS_GEMM_DEFAULT));
        }
        merge_complex_half(h->cudaStream, rows, n, cp, cp + plane_c, block, static_cast<char*>(C) + size_t(i) * 4, ldc);
      }
      pool_free(h, bp); pool_free(h, ap); pool_free(h, cp);
      return true;
    }
    default: return false;
  }
}

// ---- Gram -> factor -> basis ------------------------------------------------------------------------------
struct GramProblem { int32_t* vexp; uint64_t* C; void* G; hyacinPrecision_t gtype; };

// Everything from the input matrix to the floating-point Gram (src/lra.cpp:55-81).
bool build_gram(const hyacinHandle_t* h, double eps, char op, int M, int N, hyacinPrecision_t type, const void* A, int lda, int64_t globalM, GramProblem* out) {
  const int seg = h->GramSegmentK <= 0 ? M : std::min(h->GramSegmentK, M);
  const int batches = seg > 0 ? (M + seg - 1) / seg : 0, lastM = (seg > 0 && M % seg) ? M % seg : seg;
  int32_t u = 0, cp = 0, lp = 0, gbytes = 0; uint64_t tri = 0;
  hyacinXherkBatchInit(h, eps, uint64_t(globalM), N, type, &u, &cp, &lp, &tri);
  int32_t* vexp = pool_alloc<int32_t>(h, size_t(batches + 1) * N);
  uint64_t* C = pool_alloc<uint64_t>(h, size_t(cp) * lp * tri);
  if (op == 'T' || op == 'C') {
    // The reference first writes a transposed copy of the whole input (src/lra.cpp:63-65); here the exponent
    // pass and the quantisers read the stored layout directly (transposing 64 x 32 tiles through shared
    // memory), which saves M x N elements of workspace and two passes over them.  Same integers either way.
    timer_mark(h, Segment::Distributed);
    launch_column_exponents(h->cudaStream, type, batches, seg, lastM, N, A, lda, u, vexp, op);
    hyacinAllReduceVExp(h, uint64_t(N), vexp);
    timer_mark(h, Segment::Distributed);
    if (lp > 0) herk_any(h, M, N, type, A, lda, op, u, vexp, 0, lp, C, batches, seg);
  } else {
    hyacinXquantizeScaleBatch(h, batches, seg, lastM, N, type, A, lda, u, vexp);
    hyacinAllReduceVExp(h, uint64_t(N), vexp);
    hyacinXherkBatch(h, batches, seg, lastM, N, type, A, lda, u, vexp, 0, lp, C);
  }
  hyacinPrecision_t gtype = HYACIN_F64;
  void* G = nullptr;
  int ranks = 1;
  uint64_t* slices = lp > 0 ? allreduce_to_slices(h, cp, lp, tri, C, &ranks) : nullptr;
  if (slices) {
    // Post-collective epilogue in one pass: the summed slices are never written back as limbs; the format scan and
    // the conversion to floating point re-assemble each integer in registers.
    timer_mark(h, Segment::Replicated);
    int32_t* bits_host = static_cast<int32_t*>(h->pinnedWorkspace);
    *bits_host = 0;
    launch_gram_range_slices(h->cudaStream, N, lp, ranks, slices, vexp, bits_host);
    HYB_CUDA(cudaStreamSynchronize(h->cudaStream));
    gtype = gram_type_from_bits(h, *bits_host, type);
    gbytes = int(gram_elem_bytes(gtype));
    G = pool_alloc<char>(h, size_t(N) * N * size_t(gbytes));
    launch_dequantize_slices(h->cudaStream, N, lp, ranks, slices, vexp, gtype, G, N);
    pool_free(h, slices);
  } else {
    hyacinXdequantizeInit(h, N, lp, C, vexp, type, &gtype, &gbytes);
    G = pool_alloc<char>(h, size_t(N) * N * size_t(gbytes));
    hyacinXdequantize(h, N, lp, C, vexp, gtype, G, N);
  }
  pool_free(h, vexp); pool_free(h, C);
  out->vexp = nullptr; out->C = nullptr; out->G = G; out->gtype = gtype;
  return true;
}

int svd_fit(const hyacinHandle_t* h, double eps, char op, int M, int N, int K, hyacinPrecision_t type, const void* A, int lda, void* S, void* V, int ldv, int64_t globalM) {
  K = std::min(N, K); if (K <= 0) return 0;
  GramProblem gp{};
  build_gram(h, eps, op, M, N, type, A, lda, globalM, &gp);
  const int rank = hyacinXGevd(h, eps, N, K, type, V, ldv, S, gp.gtype, gp.G, N);
  pool_free(h, gp.G);
  return rank;
}

int interp_fit(const hyacinHandle_t* h, double eps, char op, int M, int N, int K, hyacinPrecision_t type, const void* A, int lda, int32_t* jpvt, void* V, int ldv, int64_t globalM) {
  K = std::min(N, K); if (K <= 0) return 0;
  GramProblem gp{};
  build_gram(h, eps, op, M, N, type, A, lda, globalM, &gp);
  const int rank = hyacinXGinterp(h, eps, N, K, type, V, ldv, jpvt, gp.gtype, gp.G, N);
  pool_free(h, gp.G);
  return rank;
}

// Two-stage column-segmented SVD fit (src/lra.cpp:112-156).
int svd_fit_segmented(const hyacinHandle_t* h, double eps, char op, int M, int N, int K, hyacinPrecision_t type, const void* A, int lda, void* S, void* V, int ldv, int64_t globalM) {
  K = std::min(N, K); if (K <= 0) return 0;
  const int segments = N >= 512 ? int(std::floor(std::sqrt(double(N) / double(K)))) : 1;
  if (segments <= 1) return svd_fit(h, eps, op, M, N, K, type, A, lda, S, V, ldv, globalM);
  eps *= std::sqrt(0.5);
  const size_t eb = elem_bytes(type), rb = elem_bytes(real_of(type));
  const int quot = N / segments, rem = N % segments, n1 = quot + (rem ? 1 : 0);
  const size_t v1_stride = size_t(n1) * n1;
  const bool trans = op == 'T' || op == 'C';
  char* V1 = pool_alloc<char>(h, v1_stride * segments * eb);
  char* S1 = pool_alloc<char>(h, size_t(n1) * rb);
  std::vector<int> ranks;
  const char* a = static_cast<const char*>(A); size_t loc = 0;
  for (int i = 0; i < segments; ++i) {
    const int cols = quot + (i < rem ? 1 : 0);
    ranks.push_back(svd_fit(h, eps, op, M, cols, cols, type, a + loc * eb, lda, S1, V1 + size_t(i) * v1_stride * eb, n1, globalM));
    loc += trans ? size_t(cols) : size_t(cols) * lda;
  }
  pool_free(h, S1);
  const int n2 = std::accumulate(ranks.begin(), ranks.end(), 0);
  char* A2 = pool_alloc<char>(h, size_t(M) * n2 * eb);
  timer_mark(h, Segment::Distributed);
  loc = 0; size_t loc2 = 0;
  if (M > 0) for (int i = 0; i < segments; ++i) {
    const int cols = quot + (i < rem ? 1 : 0);
    if (ranks[i] > 0) stage_gemm(h, type, op, M, ranks[i], cols, a + loc * eb, lda, V1 + size_t(i) * v1_stride * eb, n1, A2 + loc2 * eb, M);
    loc += trans ? size_t(cols) : size_t(cols) * lda; loc2 += size_t(ranks[i]) * M;
  }
  K = std::min(n2, K);
  char* V2 = pool_alloc<char>(h, size_t(n2) * std::max(K, 1) * eb);
  const int rank = n2 > 0 ? svd_fit(h, eps, 'N', M, n2, K, type, A2, M, S, V2, n2, globalM) : 0;
  pool_free(h, A2);
  timer_mark(h, Segment::Replicated);
  int row = 0, row_v = 0;
  for (int i = 0; i < segments; ++i) {
    const int cols = quot + (i < rem ? 1 : 0);
    if (rank > 0 && ranks[i] > 0) stage_gemm(h, type, 'N', cols, rank, ranks[i], V1 + size_t(i) * v1_stride * eb, n1, V2 + size_t(row_v) * eb, n2, static_cast<char*>(V) + size_t(row) * eb, ldv);
    else if (rank > 0) for (int c = 0; c < rank; ++c) HYB_CUDA(cudaMemsetAsync(static_cast<char*>(V) + (size_t(row) + size_t(c) * ldv) * eb, 0, size_t(cols) * eb, h->cudaStream));
    row += cols; row_v += ranks[i];
  }
  pool_free(h, V1); pool_free(h, V2);
  return rank;
}

// || op(A) - op(A) Q Q^H ||_F^2 in double precision, 2048-row blocks (src/lra.cpp:158-208).
double projection_residual(const hyacinHandle_t* h, char op, int M, int N, hyacinPrecision_t type, const void* A, int lda, int rank, const void* V, int ldv) {
  if (M <= 0 || N <= 0) return 0.;
  timer_mark(h, Segment::Untimed);
  const int cplx = is_complex(type), block = 2048;
  const hyacinPrecision_t wide = hyacinPrecision_t(HYACIN_F64 | cplx);
  const size_t wb = elem_bytes(wide), eb = elem_bytes(type);
  const bool trans = op == 'T' || op == 't' || op == 'C' || op == 'c';
  const char opn = (op == 't') ? 'T' : (op == 'c') ? 'C' : op;
  const char* a = static_cast<const char*>(A);
  double err = 0.;
  cublasHandle_t b = h->cublasHandle; cusolverDnHandle_t s = h->cusolverHandle;
  if (rank <= 0) {
    char* blk = pool_alloc<char>(h, size_t(block) * block * wb);
    for (int i = 0; i < M; i += block) { const int rows = std::min(M - i, block);
      for (int j = 0; j < N; j += block) { const int cols = std::min(N - j, block);
        const char* src = trans ? a + (size_t(j) + size_t(i) * lda) * eb : a + (size_t(i) + size_t(j) * lda) * eb;
        convert_copy(h->cudaStream, trans ? opn : 'N', rows, cols, type, src, lda, wide, blk, rows);
        double nrm = 0.; HYB_LIB(cublasDnrm2_64(b, int64_t(rows) * cols * (cplx + 1), reinterpret_cast<const double*>(blk), 1, &nrm)); err += nrm * nrm;
      } }
    pool_free(h, blk);
    return err;
  }
  char* Q = pool_alloc<char>(h, size_t(N) * rank * wb); char* tau = pool_alloc<char>(h, size_t(N) * wb); int* info = pool_alloc<int>(h, 1);
  convert_copy(h->cudaStream, 'N', N, rank, type, V, ldv, wide, Q, N);
  int lw0 = 0, lw1 = 0; void* work = nullptr;
  if (cplx) {
    HYB_LIB(cusolverDnZgeqrf_bufferSize(s, N, rank, (cuDoubleComplex*)Q, N, &lw0));
    HYB_LIB(cusolverDnZungqr_bufferSize(s, N, rank, rank, (cuDoubleComplex*)Q, N, (cuDoubleComplex*)tau, &lw1)); lw0 = std::max(lw0, lw1);
    work = pool_alloc<cuDoubleComplex>(h, lw0);
    HYB_LIB(cusolverDnZgeqrf(s, N, rank, (cuDoubleComplex*)Q, N, (cuDoubleComplex*)tau, (cuDoubleComplex*)work, lw0, info));
    HYB_LIB(cusolverDnZungqr(s, N, rank, rank, (cuDoubleComplex*)Q, N, (cuDoubleComplex*)tau, (cuDoubleComplex*)work, lw0, info));
  } else {
    HYB_LIB(cusolverDnDgeqrf_bufferSize(s, N, rank, (double*)Q, N, &lw0));
    HYB_LIB(cusolverDnDorgqr_bufferSize(s, N, rank, rank, (double*)Q, N, (double*)tau, &lw1)); lw0 = std::max(lw0, lw1);
    work = pool_alloc<double>(h, lw0);
    HYB_LIB(cusolverDnDgeqrf(s, N, rank, (double*)Q, N, (double*)tau, (double*)work, lw0, info));
    HYB_LIB(cusolverDnDorgqr(s, N, rank, rank, (double*)Q, N, (double*)tau, (double*)work, lw0, info));
  }
  pool_free(h, tau); pool_free(h, work); pool_free(h, info);
  char* blkA = pool_alloc<char>(h, size_t(block) * N * wb); char* blkU = pool_alloc<char>(h, size_t(block) * rank * wb);
  const cuDoubleComplex z_one = make_cuDoubleComplex(1., 0.), z_zero = make_cuDoubleComplex(0., 0.), z_minus = make_cuDoubleComplex(-1., 0.);
  const cudaDataType dt = cplx ? CUDA_C_64F : CUDA_R_64F; const cublasOperation_t opt = cplx ? CUBLAS_OP_C : CUBLAS_OP_T;
  for (int i = 0; i < M; i += block) {
    const int rows = std::min(M - i, block);
    const char* src = trans ? a + size_t(i) * lda * eb : a + size_t(i) * eb;
    convert_copy(h->cudaStream, trans ? opn : 'N', rows, N, type, src, lda, wide, blkA, rows);
    // a real alpha/beta is read from the leading double of the complex constant
    HYB_LIB(cublasGemmEx(b, CUBLAS_OP_N, CUBLAS_OP_N, rows, rank, N, &z_one, blkA, dt, rows, Q, dt, N, &z_zero, blkU, dt, block, CUBLAS_COMPUTE_64F_PEDANTIC, CUBLAS_GEMM_DEFAULT));
    HYB_LIB(cublasGemmEx(b, CUBLAS_OP_N, opt, rows, N, rank, &z_minus, blkU, dt, block, Q, dt, N, &z_one, blkA, dt, rows, CUBLAS_COMPUTE_64F_PEDANTIC, CUBLAS_GEMM_DEFAULT));
    double nrm = 0.; HYB_LIB(cublasDnrm2_64(b, int64_t(rows) * N * (cplx + 1), reinterpret_cast<const double*>(blkA), 1, &nrm)); err += nrm * nrm;
  }
  pool_free(h, blkA); pool_free(h, blkU); pool_free(h, Q);
  return err;
}

bool input_type_ok(hyacinPrecision_t t) { return int(t) >= 0 && int(t) <= int(HYACIN_F16_COMPLEX); }
char canon_op(char op) { return op == 't' ? 'T' : op == 'c' ? 'C' : op; }

}  // namespace
}  // namespace hyb

using namespace hyb;

extern "C" int32_t hyacinXGevd(const hyacinHandle_t* handle, double eps, int32_t N, int32_t K, hyacinPrecision_t Atype, void* X, int32_t ldx,
                               void* S, hyacinPrecision_t Gtype, void* G, int32_t ldg) {
  if (N <= 0 || !input_type_ok(Atype)) return 0;
  if (is_complex(Atype) != is_complex(Gtype)) return 0;
  K = K <= 0 ? N : std::min(N, K);
  timer_mark(handle, Segment::Replicated);
  cudaStream_t stream = handle->cudaStream;
  const int lrqr = handle->QRCPTruncateRank;
  const int jacobi = std::abs(handle->JacobiSVDSweeps), bidiag = std::abs(std::min(0, handle->JacobiSVDSweeps));
  const int sweeps = base_type(Atype) == HYACIN_F64 ? ((lrqr && handle->DeviceIsF64Capable) ? jacobi : bidiag) : (lrqr ? jacobi : bidiag);
  const hyacinPrecision_t lt = lib_type(Atype);
  const double machine_eps = base_type(lt) == HYACIN_F64 ? DBL_EPSILON : double(FLT_EPSILON);
  eps = std::min(std::max(std::fabs(eps), machine_eps), 1.);

  const size_t gb = gram_elem_bytes(Gtype);
  const int64_t ldc = factor_col_pitch(N);
  char* Rc = pool_alloc<char>(handle, size_t(N) * ldc * gb);
  int32_t* jpiv = pool_alloc<int32_t>(handle, size_t(2) * N);
  int32_t* pos = jpiv + N;
  int rank = potrfp(handle, lrqr ? eps : 0., N, N, Gtype, G, ldg, Rc, ldc, jpiv, pos);
  if (rank <= 0) { pool_free(handle, jpiv); pool_free(handle, Rc); return 0; }

  const size_t lb = gram_elem_bytes(lt), rb = gram_elem_bytes(real_of(lt));
  char* A = pool_alloc<char>(handle, size_t(N) * rank * lb);
  factor_to_columns(stream, N, rank, Gtype, Rc, ldc, pos, lt, A, N);
  pool_free(handle, jpiv); pool_free(handle, Rc);
  char* sigma = pool_alloc<char>(handle, size_t(rank) * rb);
  char* U = pool_alloc<char>(handle, size_t(N) * rank * lb);
  {
    ProfileScope scope(stream, KernelKind::Svd);
    if (sweeps > 0) {
      char* Vr = pool_alloc<char>(handle, size_t(rank) * rank * lb);
      gesvdj(handle, lt, N, rank, A, sigma, U, Vr, sweeps, machine_eps);
      pool_free(handle, Vr);
    } else gesvd(handle, lt, N, rank, A, sigma, U);
  }
  pool_free(handle, A);
  double* suffix = pool_alloc<double>(handle, size_t(std::max(K, rank)));
  int32_t* r_host = static_cast<int32_t*>(handle->pinnedWorkspace);
  find_rank(stream, eps * eps, rank, K, real_of(lt), sigma, real_of(Atype), S, r_host, suffix);
  HYB_CUDA(cudaStreamSynchronize(stream));
  const int svd_rank = *r_host;
  rank = std::min(rank, svd_rank);
  pool_free(handle, sigma); pool_free(handle, suffix);
  // Same storage and library type: the copy goes through cuBLAS geam as in the reference (src/matcopy.cu:100-108).  For
  // complex data that is a multiplication by (1, 0), which turns an imaginary part of -0 into +0: part of the bits of V.
  if (lt == Atype && rank > 0) {
    cublasHandle_t b = handle->cublasHandle;
    switch (int(lt)) {
      case HYACIN_F64: { const double one = 1., zero = 0.; HYB_LIB(cublasDgeam(b, CUBLAS_OP_N, CUBLAS_OP_N, N, rank, &one, (const double*)U, N, &zero, (const double*)X, ldx, (double*)X, ldx)); break; }
      case HYACIN_F32: { const float one = 1.f, zero = 0.f; HYB_LIB(cublasSgeam(b, CUBLAS_OP_N, CUBLAS_OP_N, N, rank, &one, (const float*)U, N, &zero, (const float*)X, ldx, (float*)X, ldx)); break; }
      case HYACIN_F64_COMPLEX: { const cuDoubleComplex one = make_cuDoubleComplex(1., 0.), zero = make_cuDoubleComplex(0., 0.);
        HYB_LIB(cublasZgeam(b, CUBLAS_OP_N, CUBLAS_OP_N, N, rank, &one, (const cuDoubleComplex*)U, N, &zero, (const cuDoubleComplex*)X, ldx, (cuDoubleComplex*)X, ldx)); break; }
      default: { const cuComplex one = make_cuComplex(1.f, 0.f), zero = make_cuComplex(0.f, 0.f);
        HYB_LIB(cublasCgeam(b, CUBLAS_OP_N, CUBLAS_OP_N, N, rank, &one, (const cuComplex*)U, N, &zero, (const cuComplex*)X, ldx, (cuComplex*)X, ldx)); break; }
    }
  } else convert_copy(stream, 'N', N, rank, lt, U, N, Atype, X, ldx);
  pool_free(handle, U);
  if (handle->logger) {
    static const char* names[4] = {"FP64", "FP64-COMPLEX", "FP32", "FP32-COMPLEX"};
    if (sweeps > 0) std::fprintf(static_cast<FILE*>(handle->logger), "GESVJ-%s [eps=%.1le] [M=%d] [N=%d] [K=%d] [sweeps=%d] [SVD-rank=%d]\n", names[int(lt)], eps, N, rank, K, sweeps, svd_rank);
    else std::fprintf(static_cast<FILE*>(handle->logger), "GESVD-%s [eps=%.1le] [M=%d] [N=%d] [K=%d] [SVD-rank=%d]\n", names[int(lt)], eps, N, rank, K, svd_rank);
  }
  return rank;
}

extern "C" int32_t hyacinXGinterp(const hyacinHandle_t* handle, double eps, int32_t N, int32_t K, hyacinPrecision_t Atype, void* X, int32_t ldx,
                                  int32_t* jpiv, hyacinPrecision_t Gtype, void* G, int32_t ldg) {
  if (N <= 0 || !input_type_ok(Atype)) return 0;
  if (is_complex(Atype) != is_complex(Gtype)) return 0;
  K = K <= 0 ? N : std::min(N, K);
  timer_mark(handle, Segment::Replicated);
  cudaStream_t stream = handle->cudaStream;
  const hyacinPrecision_t lt = lib_type(Atype);
  const double machine_eps = base_type(lt) == HYACIN_F64 ? DBL_EPSILON : double(FLT_EPSILON);
  eps = std::min(std::max(std::fabs(eps), machine_eps), 1.);
  const size_t gb = gram_elem_bytes(Gtype);
  const int64_t ldc = factor_col_pitch(K);
  char* Rc = pool_alloc<char>(handle, size_t(N) * ldc * gb);
  int32_t* pos = pool_alloc<int32_t>(handle, N);
  const int rank = potrfp(handle, eps, K, N, Gtype, G, ldg, Rc, ldc, jpiv, pos);
  pool_free(handle, pos);
  if (rank == N) interp_scatter(stream, N, N, jpiv, lt, nullptr, N, Atype, X, ldx);
  else if (rank > 0) {
    const size_t lb = gram_elem_bytes(lt);
    char* B = pool_alloc<char>(handle, size_t(rank) * N * lb);
    factor_to_pivoted(stream, N, rank, Gtype, Rc, ldc, jpiv, lt, B, rank);
    trsm_upper_left(handle, lt, rank, N - rank, B, rank);
    interp_scatter(stream, N, rank, jpiv, lt, B, rank, Atype, X, ldx);
    pool_free(handle, B);
    if (handle->logger) { static const char* names[4] = {"FP64", "FP64-COMPLEX", "FP32", "FP32-COMPLEX"};
      std::fprintf(static_cast<FILE*>(handle->logger), "TRSM-LEFT-%s [M=%d] [N=%d]\n", names[int(lt)], rank, N - rank); }
  }
  pool_free(handle, Rc);
  return rank;
}

// Test hook: the pivoted Cholesky alone.  R comes out as the reference leaves it in the upper triangle of its
// (overwritten) Gram matrix: R[k + x ldr] = R[k, column jpiv[x] - 1] for k <= x, zero below, in the Gram's format.
extern "C" int32_t hyacinB200PivotedCholesky(const hyacinHandle_t* handle, double eps, int32_t N, int32_t K, hyacinPrecision_t Gtype, const void* G,
                                             int32_t ldg, int32_t* jpiv, void* R, int32_t ldr) {
  const size_t gb = gram_elem_bytes(Gtype);
  if (N <= 0 || gb == 0) return 0;
  K = K <= 0 ? N : std::min(N, K);
  const int64_t ldc = factor_col_pitch(K);
  char* Rc = pool_alloc<char>(handle, size_t(N) * ldc * gb);
  int32_t* pos = pool_alloc<int32_t>(handle, N);
  const int rank = potrfp(handle, eps, K, N, Gtype, G, ldg, Rc, ldc, jpiv, pos);
  if (rank > 0 && R) factor_copy_pivoted(handle->cudaStream, N, std::min(rank, K), Gtype, Rc, ldc, jpiv, R, ldr);
  pool_free(handle, pos); pool_free(handle, Rc);
  HYB_CUDA(cudaStreamSynchronize(handle->cudaStream));
  return rank;
}

extern "C" int32_t hyacinInterpolateFit(const hyacinHandle_t* handle, double eps, char opA, int32_t M, int32_t N, int32_t K, const void* A,
                                        int32_t lda, int32_t* jpvt, void* V, int32_t ldv, int64_t globalM, hyacinPrecision_t ComputeType) {
  if (!input_type_ok(ComputeType)) return 0;
  return interp_fit(handle, eps, canon_op(opA), M, N, K, ComputeType, A, lda, jpvt, V, ldv, globalM <= 0 ? int64_t(M) : globalM);
}

extern "C" int32_t hyacinTsvdFit(const hyacinHandle_t* handle, double eps, char opA, int32_t M, int32_t N, int32_t K, const void* A, int32_t lda,
                                 void* S, void* V, int32_t ldv, int64_t globalM, hyacinPrecision_t ComputeType) {
  if (!input_type_ok(ComputeType)) return 0;
  return svd_fit(handle, eps, canon_op(opA), M, N, K, ComputeType, A, lda, S, V, ldv, globalM <= 0 ? int64_t(M) : globalM);
}

extern "C" int32_t hyacinTsvdFitSegmentN(const hyacinHandle_t* handle, double eps, char opA, int32_t M, int32_t N, int32_t K, const void* A,
                                         int32_t lda, void* S, void* V, int32_t ldv, int64_t globalM, hyacinPrecision_t ComputeType) {
  if (!input_type_ok(ComputeType)) return 0;
  return svd_fit_segmented(handle, eps, canon_op(opA), M, N, K, ComputeType, A, lda, S, V, ldv, globalM <= 0 ? int64_t(M) : globalM);
}

extern "C" double hyacinCheckNorm(const hyacinHandle_t* handle, char opA, int32_t M, int32_t N, const void* A, int32_t lda, int32_t rank,
                                  const void* V, int32_t ldv, hyacinPrecision_t ComputeType) {
  if (!input_type_ok(ComputeType)) return 0.;
  return projection_residual(handle, opA, M, N, ComputeType, A, lda, rank, V, ldv);
}
