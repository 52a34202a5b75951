// Interfaces of the replicated tail of a fit (everything after the Gram matrix exists in floating point).
#pragma once
#include "hyb_internal.h"

namespace hyb {

size_t gram_elem_bytes(hyacinPrecision_t gtype);

// Truncated pivoted Cholesky.  G: n x n Hermitian Gram in format gtype (F32 / F64 / DD, real or complex), read
// only.  Rc: the factor in the same format, column-major by ORIGINAL column: Rc[i * ldc + k] = R[k, column i],
// defined for k <= (position of column i in the pivot order) and k < rank; entries below that diagonal are not
// written.  ldc = factor_col_pitch(cap) rows per column.  jpiv: n one-based column indices, chosen columns first;
// pos: its inverse, pos[i] = zero-based position of column i.  Stops at `cap` rows or when the remaining trace is
// <= eps^2 * initial trace.  Blocks the host; returns the rank.
int potrfp(const hyacinHandle_t* handle, double eps, int cap, int n, hyacinPrecision_t gtype, const void* G, int64_t ldg,
           void* Rc, int64_t ldc, int32_t* jpiv, int32_t* pos);
// Rows to allocate per column of Rc: cap + 1 rounded up to whole 128-row stages.
int64_t factor_col_pitch(int cap);

// dst (column-major, ldd) <- op(src) with element conversion.  op: 'N' copy, 'T' transpose, 'C' conjugate
// transpose.  rows / cols describe dst.  Types are hyacinPrecision_t values 0..5 (F64, F32, F16, real/complex).
void convert_copy(cudaStream_t stream, char op, int rows, int cols, hyacinPrecision_t src_type, const void* src, int64_t lds,
                  hyacinPrecision_t dst_type, void* dst, int64_t ldd);

// A (n x rank, column-major, lda) <- R^H with rows in original order: A[i, k] = conj(R[k, column i]) for
// k <= pos[i], 0 beyond.  dst_type: F64 / F32 (real or complex, matching the Gram).
void factor_to_columns(cudaStream_t stream, int n, int rank, hyacinPrecision_t gtype, const void* Rc, int64_t ldc, const int32_t* pos,
                       hyacinPrecision_t dst_type, void* A, int64_t lda);
// B (rank x n, column-major, ldb) <- R in PIVOTED column order: B[k, x] = R[k, column jpiv[x] - 1], zero below the diagonal.
void factor_to_pivoted(cudaStream_t stream, int n, int rank, hyacinPrecision_t gtype, const void* Rc, int64_t ldc, const int32_t* jpiv,
                       hyacinPrecision_t dst_type, void* B, int64_t ldb);
// The same in the Gram's own format, bit for bit (what the reference leaves in the upper triangle of G).
void factor_copy_pivoted(cudaStream_t stream, int n, int rank, hyacinPrecision_t gtype, const void* Rc, int64_t ldc, const int32_t* jpiv,
                         void* B, int64_t ldb);
// X (n x rank, ldx, type xtype) <- P [I; T^H]: row jpiv[x]-1 gets e_x for x < rank and conj(B[:, x]) otherwise.
void interp_scatter(cudaStream_t stream, int n, int rank, const int32_t* jpiv, hyacinPrecision_t b_type, const void* B, int64_t ldb,
                    hyacinPrecision_t xtype, void* X, int64_t ldx);

// Planar views of complex-half matrices for the segmented fit (the library has no complex-half GEMM).
// split: re, im (rows x cols, column-major, ld) <- op(src) rows [row0, row0 + rows); op 'N': src is stored rows x cols,
//        'T' / 'C': src is stored cols x rows (and conjugated for 'C').
// split_b: three panels of cols columns each, (-im, re, im), so that [re | im] and [-im | re] are contiguous
//        (rows x 2 cols) operands.  merge: dst complex <- (re, im).
void split_complex_half(cudaStream_t stream, char op, int64_t row0, int rows, int cols, const void* src, int64_t lds, void* re, void* im, int64_t ld);
void split_complex_half_stored(cudaStream_t stream, bool conj, int rows, int cols, const void* src, int64_t lds, void* re, void* im, int64_t ld);
void split_complex_half_b(cudaStream_t stream, int rows, int cols, const void* src, int64_t lds, void* panels, int64_t ld);
void merge_complex_half(cudaStream_t stream, int rows, int cols, const void* re, const void* im, int64_t ld, void* dst, int64_t ldd);

// Tail-energy rank rule on `n` singular values (descending); writes K values to `out`, the new rank to *rank.
// suffix: scratch of max(n, 1) doubles.
void find_rank(cudaStream_t stream, double eps_sq, int n, int K, hyacinPrecision_t sigma_type, const void* sigma, hyacinPrecision_t out_type,
               void* out, int32_t* rank, double* suffix);

}  // namespace hyb
