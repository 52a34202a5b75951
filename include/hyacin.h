/*
 * hyacin.h -- public C ABI of the B200-native Hyacin build.
 *
 * Binary-compatible with the reference header (include/hyacin.h in QxGbM/hyacinth): same enum values,
 * same handle layout, same 16 entry points with the same argument order.  An application linked against
 * the reference library can be relinked (or LD_PRELOADed) against this one unchanged.
 *
 * Conventions shared by every entry point:
 *   - all matrix arguments are DEVICE pointers in column-major storage;
 *   - M and N describe op(A), the matrix whose right basis is fitted (stored shape M x N for opA 'N',
 *     N x M for 'T' / 'C');
 *   - work is enqueued on handle->cudaStream; temporaries come from handle->mempool (stream ordered);
 *   - there is no error channel: unsupported arguments make a call a no-op (or return rank 0).
 */
#ifndef HYACIN_H_
#define HYACIN_H_

#include <stdint.h>
#include <cublas_v2.h>
#include <cusolverDn.h>

#ifndef HYACIN_BUILD_NO_NCCL
#include <nccl.h>
#endif

/* Storage / compute precisions.  Even values are real, odd values the complex counterpart.
 * Only the first six are accepted as input types; DD (double-double), TF (triple-float) and
 * QF (quad-float) are Gram-matrix formats chosen by hyacinXdequantizeInit.
 * Reference: include/hyacin.h:11-18. */
typedef enum {
  HYACIN_F64 = 0,
  HYACIN_F64_COMPLEX = 1,
  HYACIN_F32 = 2,
  HYACIN_F32_COMPLEX = 3,
  HYACIN_F16 = 4,
  HYACIN_F16_COMPLEX = 5,
  HYACIN_DD = 6,
  HYACIN_DD_COMPLEX = 7,
  HYACIN_TF = 8,
  HYACIN_TF_COMPLEX = 9,
  HYACIN_QF = 10,
  HYACIN_QF_COMPLEX = 11
} hyacinPrecision_t;

/* Per-GPU, per-host-thread context.  Zero-initialise before hyacinCreate(); resource fields that are
 * non-zero at that point are borrowed from the caller, the others are created and owned by the handle.
 * Reference: include/hyacin.h:20-53 (field order and types are part of the ABI). */
typedef struct {
  /* Scheduling knobs (environment: HYACIN_GRAM_ALGORITHM, HYACIN_STRIDE_BATCH_PERF_PENALTY,
   * HYACIN_GRAM_SEGMENT_K, HYACIN_TCGEMM_TARGET_K).  The integer Gram is exact whatever they say;
   * GramSegmentK also sets the row-segment length of the per-segment column exponents. */
  char GramMatrixAlgorithm;      /* 'L' limbs only, 'C' CRT only, anything else automatic; default 'A' */
  double StrideBatchPerfPenalty; /* default 1.3 */
  int32_t GramSegmentK;          /* default 8192 */
  int32_t TCGemmTargetK;         /* default 8192 */

  /* Spectral knobs (HYACIN_QUANTIZE_BITS_CORR, HYACIN_QRCP_TRUNCATE_RANK, HYACIN_JACOBI_SVD_SWEEPS). */
  int32_t QuantizeBitCorrection; /* extra quantisation bits on top of those derived from eps; default 7 */
  int32_t QRCPTruncateRank;      /* 1: stop the pivoted Cholesky at the numerical rank; default 1 */
  int32_t JacobiSVDSweeps;       /* >0 Jacobi sweeps, 0 bidiagonalisation SVD, <0 force Jacobi; default 3 */

  /* Device description and resources. */
  int32_t DeviceID, DeviceSMs, DeviceIsF64Capable;
  uint32_t HandleOwnedResource;  /* internal ownership bits; leave zero */
  cudaStream_t cudaStream;
  cublasHandle_t cublasHandle;
  cusolverDnHandle_t cusolverHandle;
  cudaMemPool_t mempool;
  void *pinnedWorkspace, *timer, *logger;
#ifndef HYACIN_BUILD_NO_NCCL
  ncclComm_t ncclComm;           /* borrowed; NULL selects single-GPU operation */
#endif
} hyacinHandle_t;

#ifdef __cplusplus
extern "C" {
#endif

/* Fill the tuning fields from the environment and create whatever resource fields are still zero.
 * Reference: src/utils.cpp:56-90. */
void hyacinCreate(hyacinHandle_t* handle);

/* Synchronise the device, release owned resources, zero the handle.  Reference: src/utils.cpp:92-101. */
void hyacinDestroy(hyacinHandle_t* handle);

/* Interpolative fit: V (N x rank) = [I; T^H] scattered by the pivots, jpvt (N, 1-based) on the device.
 * Returns the rank (stops at K or at eps).  Reference: src/lra.cpp:18-50, 210-220. */
int32_t hyacinInterpolateFit(const hyacinHandle_t* handle, double eps, char opA, int32_t M, int32_t N, int32_t K,
                             const void* A, int32_t lda, int32_t* jpvt, void* V, int32_t ldv, int64_t globalM,
                             hyacinPrecision_t ComputeType);

/* Truncated-SVD fit: S (K reals in the storage precision) and V (N x rank).  Returns the rank.
 * globalM <= 0 means M.  Reference: src/lra.cpp:52-84, 222-232. */
int32_t hyacinTsvdFit(const hyacinHandle_t* handle, double eps, char opA, int32_t M, int32_t N, int32_t K,
                      const void* A, int32_t lda, void* S, void* V, int32_t ldv, int64_t globalM,
                      hyacinPrecision_t ComputeType);

/* As hyacinTsvdFit, with the two-stage column-segmented scheme when floor(sqrt(N / K)) > 1 and N >= 512.
 * Reference: src/lra.cpp:112-156, 234-244. */
int32_t hyacinTsvdFitSegmentN(const hyacinHandle_t* handle, double eps, char opA, int32_t M, int32_t N, int32_t K,
                              const void* A, int32_t lda, void* S, void* V, int32_t ldv, int64_t globalM,
                              hyacinPrecision_t ComputeType);

/* Host-only sizing of the integer Gram: quantisation bits uA, complex panels (1 or 2), 63-bit limb panels
 * (<= 3, from the GLOBAL row count M) and the packed-triangle stride N(N+1)/2.  Any output may be NULL.
 * Reference: src/hyacin_herk.cpp:45-59. */
void hyacinXherkBatchInit(const hyacinHandle_t* handle, double eps, uint64_t M, int32_t N, hyacinPrecision_t Atype,
                          int32_t* uA, int32_t* cPanels, int32_t* lPanels, uint64_t* stride);

/* Exact integer Gram of the quantised matrix: C (+)= Q^H Q with Q = rint(A * 2^vexp[col]), stored as packed
 * upper triangle in 63-bit limbs, [cPanels][orderC][N(N+1)/2].  A is already in 'N' orientation with
 * (batches-1)*segM + lastM rows; vexp is the (batches+1) x N array from hyacinXquantizeScaleBatch.
 * beta: 0 overwrite, 1 accumulate.  Reference: src/hyacin_herk.cpp:386-407. */
void hyacinXherkBatch(const hyacinHandle_t* handle, int32_t batches, int32_t segM, int32_t lastM, int32_t N,
                      hyacinPrecision_t Atype, const void* A, int32_t lda, int32_t u, const int32_t* vexp,
                      int32_t beta, int32_t orderC, uint64_t* C);

/* Per-column power-of-two scales: vexp[0][j] = uA - e_j with max_i |a_ij| in [2^(e_j-1), 2^e_j); rows 1..batches
 * hold the same quantity per row segment.  INT32_MAX marks an all-zero column.
 * Reference: src/fp_exponent.cu:53-65. */
void hyacinXquantizeScaleBatch(const hyacinHandle_t* handle, int32_t batches, int32_t segM, int32_t lastM, int32_t N,
                               hyacinPrecision_t Atype, const void* A, int32_t lda, int32_t uA, int32_t* vexp);

/* Pick the floating format of the dequantised Gram from the bit length of its largest scaled diagonal entry.
 * Blocks the host.  Reference: src/fp_i63tp_dequantize.cu:29-54. */
void hyacinXdequantizeInit(const hyacinHandle_t* handle, int32_t N, int32_t orderC, const uint64_t* C,
                           const int32_t* vexp, hyacinPrecision_t Atype, hyacinPrecision_t* Gtype,
                           int32_t* gElemBytes);

/* Packed integer Gram -> full Hermitian N x N matrix G[y,x] = C[y,x] * 2^-(vexp[x]+vexp[y]).
 * Reference: src/fp_i63tp_dequantize.cu:143-159. */
void hyacinXdequantize(const hyacinHandle_t* handle, int32_t N, int32_t orderC, const uint64_t* C,
                       const int32_t* vexp, hyacinPrecision_t Gtype, void* G, int32_t ldg);

/* Gram matrix -> singular values S and right basis X via pivoted Cholesky + small SVD.  Returns the rank.
 * Reference: src/gram_evd.cu:144-194. */
int32_t hyacinXGevd(const hyacinHandle_t* handle, double eps, int32_t N, int32_t K, hyacinPrecision_t Atype,
                    void* X, int32_t ldx, void* S, hyacinPrecision_t Gtype, void* G, int32_t ldg);

/* Gram matrix -> interpolation basis X and 1-based pivots jpiv via pivoted Cholesky + triangular solve.
 * Returns the rank.  Reference: src/gram_id.cpp:53-101. */
int32_t hyacinXGinterp(const hyacinHandle_t* handle, double eps, int32_t N, int32_t K, hyacinPrecision_t Atype,
                       void* X, int32_t ldx, int32_t* jpiv, hyacinPrecision_t Gtype, void* G, int32_t ldg);

/* || op(A) - op(A) Q Q^H ||_F^2 with Q = orth(V[:, :rank]); rank <= 0 gives || op(A) ||_F^2 (V untouched).
 * Local value on distributed inputs.  Reference: src/lra.cpp:158-208, 246-256. */
double hyacinCheckNorm(const hyacinHandle_t* handle, char opA, int32_t M, int32_t N, const void* A, int32_t lda,
                       int32_t rank, const void* V, int32_t ldv, hyacinPrecision_t ComputeType);

/* Exact cross-rank sum of the packed integer Gram (Complex = cPanels, orderA = limb panels, N = packed
 * stride).  No-op without a communicator or with one rank.  Reference: src/allreduce_1drow.cu:145-169. */
void hyacinAllReduce1Drow(const hyacinHandle_t* handle, int32_t Complex, int32_t orderA, uint64_t N, uint64_t* A);

/* Cross-rank minimum of the N global column exponents.  Reference: src/allreduce_1drow.cu:171-178. */
void hyacinAllReduceVExp(const hyacinHandle_t* handle, uint64_t N, int32_t* vexp);

/* Wait for the stream; when the handle has a timer, answer each entry of eventMs that holds 'D', 'R' or 'C'
 * (as a double) with the milliseconds spent in distributed kernels, replicated kernels or communication
 * since the previous call, then clear the recorded events.  Reference: src/utils.cpp:116-141. */
void hyacinSync_TimerSegments(const hyacinHandle_t* handle, double* eventMs, int32_t lenMs);

#ifdef __cplusplus
}
#endif

#endif /* HYACIN_H_ */
