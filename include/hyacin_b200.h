/*
 * hyacin_b200.h -- entry points that exist only in the B200-native build.
 *
 * None of them has a counterpart in the reference library; applications that stay within hyacin.h never
 * need this header.  They expose the individual kernels of the quantized-Gram path (so that each stage can
 * be checked in isolation) and the status word of the bounded waits inside the tensor-core kernel.
 * Pointers are device pointers unless stated otherwise; work is enqueued on handle->cudaStream.
 */
#ifndef HYACIN_B200_H_
#define HYACIN_B200_H_

#include <hyacin.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Non-zero if a bounded wait inside the Gram kernel expired on the current device since the word was last
 * cleared (the integer Gram of that call is then invalid).  Call after synchronising the stream.
 * No counterpart in the reference (its kernels have no waits). */
uint32_t hyacinB200Status(int32_t clear);

/* Self-test of the bounded waits: runs a one-block kernel that waits, for pollLimit polls (1 .. 65536), on a
 * barrier that nothing ever completes, so the wait expires the way it would inside the Gram or Cholesky kernels:
 * the kernel returns, `code` (non-zero) appears in the status word, and the device stays usable.  Returns 0 if
 * both waiting roles of the kernel reported that they gave up, -1 for bad arguments, -2 otherwise.  Blocks the
 * host.  No counterpart in the reference. */
int32_t hyacinB200SelfTestWait(const hyacinHandle_t* handle, uint32_t pollLimit, uint32_t code);

/* Schedule of one hyacinXherkBatch call with `rows` local rows and quantisation bits u: number of CRT
 * moduli, bytes per biased quantised value, rows reconstructed together, rows per kernel launch.
 * Takes over the role of the reference's cost model (src/hyacin_herk.cpp:11-43) for this build.
 * Describes the schedule these stage hooks work with; for complex input hyacinXherkBatch itself prefers a
 * second moduli set with a square root of -1 (two planes per column, one product over all tiles) whenever
 * that set covers the bit budget, which this query does not report. */
void hyacinB200CrtPlan(int32_t u, int32_t Complex, int64_t rows, int32_t* moduli, int32_t* valueBytes,
                       int32_t* groupRows, int32_t* chunkRows);

/* Bits each row segment really needs: segU[b] = u + max_j (vexp[0][j] - vexp[b + 1][j]) over the columns that are not
 * zero in the segment, INT32_MIN for an all-zero segment; vexp is the (batches + 1) x N table of
 * hyacinXquantizeScaleBatch, segU a device array of `batches` words.  Asynchronous on the handle's stream.
 * Stage counterpart in the reference: src/fp_exponent.cu:67-76 (internal::int8::vector_range). */
void hyacinB200VectorRange(const hyacinHandle_t* handle, int32_t batches, int32_t N, int32_t u, const int32_t* vexp, int32_t* segU);

/* Tile geometry of the residue buffers for an N x N Gram: tile height / width, tile rows, and the number of
 * tiles that touch the upper triangle.  A residue buffer holds moduli * numTiles * tileY * tileX bytes. */
void hyacinB200TileInfo(int32_t N, int32_t* tileY, int32_t* tileX, int32_t* tilesY, int32_t* numTiles);

/* Work schedule of the residue Gram kernel (host mirror, no GPU needed): the k-th item of CTA pair `pair` out of `pairs`
 * when `moduli` planes of tilesX column blocks of 256 are multiplied.  An item is `width` (1 or 2) neighbouring 256 x 256
 * tiles of one tile row: (tileRow, tileCol) and, for width 2, (tileRow, tileCol + 1).  full = 0: tiles tileRow <= tileCol of
 * the upper triangle (pairRows is ignored); full = 1: all pairRows x tilesX tiles.  Returns 0 when the pair has fewer than
 * k + 1 items.  Over all pairs every tile of every plane appears exactly once. */
int32_t hyacinB200GramItem(int32_t tilesX, int32_t pairRows, int32_t full, int32_t moduli, int32_t pairs, int32_t pair, int32_t k,
                           int32_t* modulus, int32_t* tileRow, int32_t* tileCol, int32_t* width);

/* Quantise `rows` rows of A (column-major, lda in elements) into int8 residue planes
 * W[modulus][column][part * ldk + row]; ldk is a multiple of 128 and rows [rows, ldk) are zero-filled.
 * Real input: one part.  Complex input: three parts (re, im, -re).
 * Stage counterpart in the reference: src/quantize_crt_real.cu:63-99, src/quantize_crt_complex.cu:72-110. */
void hyacinB200QuantizeCrt(const hyacinHandle_t* handle, hyacinPrecision_t Atype, int32_t rows, int32_t N,
                           const void* A, int32_t lda, const int32_t* vexp, int32_t moduli, int32_t valueBytes,
                           int8_t* W, int64_t ldk);

/* Residue Gram: residues[m][tile][y][x] (+)= sum_k W[m][y][ka0 + k] * W[m][x][kb0 + k] mod modulus m.
 * kRows, ka0, kb0 multiples of 128; kRows <= 130816.
 * Stage counterpart in the reference: src/hyacin_herk.cpp:163-189 with src/crt_diag_real.cu:13-29. */
void hyacinB200GramResidues(const hyacinHandle_t* handle, int32_t N, int32_t moduli, const int8_t* W, int64_t ldw,
                            int64_t planeStride, int32_t ka0, int32_t kb0, int32_t kRows, int32_t accumulate,
                            uint8_t* residues);

/* Residues -> packed 63-bit-limb integers, Cpanel[orderC][N(N+1)/2] (+)= value.
 * Stage counterpart in the reference: src/crt_reconstruct_real.cu:94-99. */
void hyacinB200Reconstruct(const hyacinHandle_t* handle, int32_t N, int32_t moduli, const uint8_t* residues,
                           int32_t beta, int32_t orderC, uint64_t* Cpanel);

/* Limb route, stage by stage.  hyacinB200QuantizeLimbs writes `order` planes of balanced base-256 digits of
 * rint(a 2^vexp), laid out like the residue planes of hyacinB200QuantizeCrt (order = (u + 9) / 8 digits hold
 * |q| <= 2^u).  hyacinB200GramLimbs adds sum_{i,j} 2^(8(i+j)) W_i^T W_j (rows ka0.. of the A operand, kb0.. of the
 * B operand, kRows rows, order * kRows <= 131071) into one panel of the packed integer Gram (beta = 0 overwrites).
 * Stage counterparts in the reference: src/quantize_limbs.cu:60-79; src/hyacin_herk.cpp:148-161 with
 * src/limbs_diag.cu, src/limbs_cross_real.cu and src/limbs_cross_imag.cu. */
void hyacinB200QuantizeLimbs(const hyacinHandle_t* handle, hyacinPrecision_t Atype, int32_t rows, int32_t N, const void* A,
                             int32_t lda, const int32_t* vexp, int32_t order, int8_t* W, int64_t ldk);
void hyacinB200GramLimbs(const hyacinHandle_t* handle, int32_t N, int32_t order, const int8_t* W, int64_t ldw,
                         int64_t planeStride, int32_t ka0, int32_t kb0, int32_t kRows, int32_t beta, int32_t orderC,
                         uint64_t* Cpanel);

/* hyacinXherkBatch for callers that cannot allocate: same arguments, same exact integer Gram in C, but all
 * scratch (int8 residue planes, residue accumulators) lives in a fixed 64 MiB array that is part of the loaded
 * module instead of coming from handle->mempool.  It is meant for hosts that have handed the whole device to
 * their own arena, or that call from a latency-bound loop where an allocator call is not acceptable.
 * Returns 0 on success; -1 for unsupported arguments or a handle that belongs to another device than the current
 * one; -2 (with a message on stderr) when residues(N, moduli) + one 128-row chunk of planes exceed the array --
 * roughly N > 2000 for FP64 at eps 1e-10; -3 if the array's device address or the handle's status word could
 * not be obtained (the handle must come from hyacinCreate on this device).
 * The first call on a device looks the array's address up, which with lazy module loading is also the moment the
 * driver reserves the 64 MiB: make one call -- zero rows is enough, it launches nothing -- before the host takes
 * the rest of the device memory, and outside any stream capture; from then on the array costs 64 MiB of that
 * device until the process exits.  Calls on one device share the array: keep them on one stream or order them
 * with events; calls whose kernels overlap on the GPU race.  Complex input always uses the three-part schedule;
 * handle->GramMatrixAlgorithm is not consulted.
 * This entry point has no counterpart in the reference, whose hyacinXherkBatch always allocates from the pool. */
int32_t hyacinB200HerkBatchStatic(const hyacinHandle_t* handle, int32_t batches, int32_t segM, int32_t lastM, int32_t N,
                                  hyacinPrecision_t Atype, const void* A, int32_t lda, int32_t u, const int32_t* vexp,
                                  int32_t beta, int32_t orderC, uint64_t* C);

/* Wire format of hyacinAllReduce1Drow for a value of orderA 63-bit limbs summed over `ranks` ranks: the value
 * is cut into `slices` words, the first slices-1 holding widthBits unsigned bits each and the last the signed
 * remainder, so that a plain unsigned 64-bit sum over all ranks cannot overflow.  Host only.
 * Takes over the role of the reference's table of limb counts (src/allreduce_1drow.cu:151). */
void hyacinB200SlicePlan(int32_t orderA, int32_t ranks, int32_t* slices, int32_t* widthBits);

/* Format choice and conversion to floating point straight from the slices of a cross-rank sum: C is cut into the
 * slices that `ranks` ranks would exchange, and the Gram matrix is produced from those without re-assembling the
 * limbs in memory (the route the fits take after their all-reduce).  Gives the bits of hyacinXdequantizeInit +
 * hyacinXdequantize.  Stage counterparts in the reference: src/allreduce_1drow.cu:112-131,
 * src/fp_i63tp_dequantize.cu:17-26,121-129. */
void hyacinB200DequantizeViaSlices(const hyacinHandle_t* handle, int32_t N, int32_t orderC, const uint64_t* C, const int32_t* vexp,
                                   hyacinPrecision_t Atype, int32_t ranks, hyacinPrecision_t* Gtype, void* G, int32_t ldg);

/* Number of kernels this library has launched in the calling process (optionally reset to zero).
 * No counterpart in the reference. */
int64_t hyacinB200LaunchCount(int32_t reset);

/* In-situ kernel timing: while enabled, every quantise and Gram launch, the pivoted-Cholesky kernel and the
 * SVD call of hyacinXGevd are bracketed by CUDA events on their own stream; hyacinB200ProfileRead waits for
 * them, returns total milliseconds and launch counts of the quantise and Gram kernels, and clears the record;
 * hyacinB200ProfileReadTail does the same for the Cholesky kernel and the SVD call (what either call finds of the
 * other's kinds is kept for the other).  Enabling or disabling also clears everything.  No counterpart in the
 * reference (its timer, hyacinSync_TimerSegments, groups work by class, not by kernel). */
void hyacinB200ProfileEnable(int32_t enable);
void hyacinB200ProfileRead(double* gramMs, int32_t* gramLaunches, double* quantizeMs, int32_t* quantizeLaunches);
void hyacinB200ProfileReadTail(double* choleskyMs, int32_t* choleskyLaunches, double* svdMs, int32_t* svdCalls);

/* The truncated pivoted Cholesky of hyacinXGevd / hyacinXGinterp on its own: G (N x N, format Gtype, read only)
 * -> rank, the one-based pivot order jpiv[N], and the factor R[k + x * ldr] = R(k, column jpiv[x] - 1) for
 * k <= x, zero below the diagonal, rank rows, in the Gram's own format.  That is the content the reference's
 * src/hyacin_potrfp.cu:214-272 leaves in the upper triangle of the Gram matrix it overwrites, so the two can be
 * compared bit for bit.  Blocks the host. */
int32_t hyacinB200PivotedCholesky(const hyacinHandle_t* handle, double eps, int32_t N, int32_t K, hyacinPrecision_t Gtype,
                                  const void* G, int32_t ldg, int32_t* jpiv, void* R, int32_t ldr);

#ifdef __cplusplus
}
#endif

#endif /* HYACIN_B200_H_ */
