// Small data-movement kernels of the replicated tail: type-converting copies / transposes, unpacking of the
// Cholesky factor for cuSOLVER and cuBLAS, the interpolation scatter and the tail-energy rank rule.
// Behaviour follows the reference's src/matcopy.cu (conversion rules :4-21, transposes :36-43, pivot scatter
// :51-56) and src/gram_evd.cu:44-70 (rank rule); the kernels are written for this build's factor layout.
#include "tail.h"
#include <cuda_fp16.h>
#include <cuComplex.h>

namespace hyb {
namespace {

struct DD { double x, y; };

// ---- element access by hyacinPrecision_t base type ---------------------------------------------------------
template <typename T> struct Num;       // real scalar types that can be stored in matrices handed to libraries
template <> struct Num<double> { static __device__ double load(const double* p) { return *p; } static __device__ void store(double* p, double v) { *p = v; } };
template <> struct Num<float> { static __device__ double load(const float* p) { return double(*p); } static __device__ void store(float* p, double v) { *p = float(v); } };
template <> struct Num<__half> { static __device__ double load(const __half* p) { return double(__half2float(*p)); } static __device__ void store(__half* p, double v) { *p = __double2half(v); } };
template <> struct Num<DD> { static __device__ double load(const DD* p) { return p->x; } static __device__ void store(DD* p, double v) { p->x = v; p->y = 0.; } };

// dst[r + c ldd] = op(src)[r, c]; one 32 x 32 tile per block of 32 x 8 threads, transposes through shared memory.
template <typename S, typename D, int CP>   // CP: reals per element (1 real, 2 complex)
__global__ void __launch_bounds__(256)
convert_copy_kernel(char op, int rows, int cols, const S* __restrict__ src, int64_t lds, D* __restrict__ dst, int64_t ldd) {
  __shared__ double tile[CP][32][33];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int r0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
  if (op == 'N') {
    const int r = r0 + tx;
    for (int j = ty; j < 32; j += 8) {
      const int c = c0 + j;
      if (r < rows && c < cols)
        for (int q = 0; q < CP; ++q) Num<D>::store(dst + (r + int64_t(c) * ldd) * CP + q, Num<S>::load(src + (r + int64_t(c) * lds) * CP + q));
    }
    return;
  }
  // source element (c, r): read with the source's fast index (c) on threadIdx.x
  const int sc = c0 + tx;
  for (int j = ty; j < 32; j += 8) {
    const int sr = r0 + j;
    if (sc < cols && sr < rows)
      for (int q = 0; q < CP; ++q) {
        double v = Num<S>::load(src + (sc + int64_t(sr) * lds) * CP + q);
        tile[q][j][tx] = (op == 'C' && q == 1) ? -v : v;
      }
  }
  __syncthreads();
  const int r = r0 + tx;
  for (int j = ty; j < 32; j += 8) {
    const int c = c0 + j;
    if (r < rows && c < cols)
      for (int q = 0; q < CP; ++q) Num<D>::store(dst + (r + int64_t(c) * ldd) * CP + q, tile[q][tx][j]);
  }
}

template <typename S, typename D>
void launch_convert(cudaStream_t stream, char op, int rows, int cols, int cplx, const void* src, int64_t lds, void* dst, int64_t ldd) {
  dim3 grid((rows + 31) / 32, (cols + 31) / 32), block(32, 8);
  if (cplx) convert_copy_kernel<S, D, 2><<<grid, block, 0, stream>>>(op, rows, cols, static_cast<const S*>(src), lds, static_cast<D*>(dst), ldd);
  else convert_copy_kernel<S, D, 1><<<grid, block, 0, stream>>>(op, rows, cols, static_cast<const S*>(src), lds, static_cast<D*>(dst), ldd);
}

template <typename S>
void dispatch_dst(cudaStream_t stream, char op, int rows, int cols, int cplx, const void* src, int64_t lds, int dst_base, void* dst, int64_t ldd) {
  switch (dst_base) {
    case HYACIN_F64: launch_convert<S, double>(stream, op, rows, cols, cplx, src, lds, dst, ldd); break;
    case HYACIN_F32: launch_convert<S, float>(stream, op, rows, cols, cplx, src, lds, dst, ldd); break;
    case HYACIN_F16: launch_convert<S, __half>(stream, op, rows, cols, cplx, src, lds, dst, ldd); break;
    default: break;
  }
}

// A[i + k lda] = conj(R[k, column i]) for k <= pos[i], else 0 -- the factor as an n x rank matrix in original row
// order.  The factor is stored with k fastest, A with i fastest: 32 x 32 tiles through shared memory.
template <typename S, typename D, int CP>
__global__ void __launch_bounds__(256)
factor_to_columns_kernel(int n, int rank, const S* __restrict__ Rc, int64_t ldc, const int32_t* __restrict__ pos, D* __restrict__ A, int64_t lda) {
  __shared__ double tile[CP][32][33];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int i0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
  for (int jj = ty; jj < 32; jj += 8) {
    const int i = i0 + jj, k = k0 + tx;
    if (i < n && k < rank) {
      const bool upper = k <= pos[i];
      for (int q = 0; q < CP; ++q) {
        const double v = upper ? Num<S>::load(Rc + (size_t(i) * ldc + k) * CP + q) : 0.;
        tile[q][jj][tx] = q == 1 ? -v : v;
      }
    }
  }
  __syncthreads();
  for (int jj = ty; jj < 32; jj += 8) {
    const int k = k0 + jj, i = i0 + tx;
    if (i < n && k < rank)
      for (int q = 0; q < CP; ++q) Num<D>::store(A + (i + int64_t(k) * lda) * CP + q, tile[q][tx][jj]);
  }
}

// B[k + x ldb] = R[k, column jpiv[x] - 1] for k <= x (upper trapezoid in pivoted column order), 0 below the diagonal.
template <typename S, typename D, int CP>
__global__ void __launch_bounds__(256)
factor_to_pivoted_kernel(int n, int rank, const S* __restrict__ Rc, int64_t ldc, const int32_t* __restrict__ jpiv, D* __restrict__ B, int64_t ldb) {
  const int k = blockIdx.x * 256 + threadIdx.x, x = blockIdx.y;
  if (k >= rank || x >= n) return;
  const int i = jpiv[x] - 1;
  for (int q = 0; q < CP; ++q) {
    double v = k <= x ? Num<S>::load(Rc + (size_t(i) * ldc + k) * CP + q) : 0.;
    Num<D>::store(B + (k + int64_t(x) * ldb) * CP + q, v);
  }
}

// The same without conversion: 4-byte words of the Gram's own element format.
__global__ void __launch_bounds__(256)
factor_copy_pivoted_kernel(int n, int rank, int words, const uint32_t* __restrict__ Rc, int64_t ldc, const int32_t* __restrict__ jpiv,
                           uint32_t* __restrict__ B, int64_t ldb) {
  const int k = blockIdx.x * 256 + threadIdx.x, x = blockIdx.y;
  if (k >= rank || x >= n) return;
  const int i = jpiv[x] - 1;
  for (int q = 0; q < words; ++q) B[(k + int64_t(x) * ldb) * words + q] = k <= x ? Rc[(size_t(i) * ldc + k) * words + q] : 0u;
}

// X[(jpiv[x] - 1) + y ldx] = (x < rank) ? [x == y] : conj(B[y + x ldb]),  y < rank, x < n.
template <typename S, typename D, int CP>
__global__ void __launch_bounds__(256)
interp_scatter_kernel(int n, int rank, const int32_t* __restrict__ jpiv, const S* __restrict__ B, int64_t ldb, D* __restrict__ X, int64_t ldx) {
  const int y = blockIdx.x * 256 + threadIdx.x, x = blockIdx.y;
  if (y >= rank || x >= n) return;
  D* dst = X + (int64_t(jpiv[x] - 1) + int64_t(y) * ldx) * CP;
  for (int q = 0; q < CP; ++q) {
    double v;
    if (x < rank) v = (x == y && q == 0) ? 1. : 0.;
    else { v = Num<S>::load(B + (y + int64_t(x) * ldb) * CP + q); if (q == 1) v = -v; }
    Num<D>::store(dst + q, v);
  }
}

// Tail-energy rank rule (reference: src/gram_evd.cu:44-70): keep index i while sum_{j >= i} sigma_j^2 exceeds
// eps^2 * sum_j sigma_j^2; S receives the kept singular values in the output precision and zeros up to K.
template <typename R, typename S>
__global__ void find_rank_kernel(double eps_sq, int n, int K, const R* __restrict__ sigma, S* __restrict__ out, int32_t* __restrict__ rank,
                                 double* __restrict__ suffix) {
  __shared__ double s_total;
  if (threadIdx.x == 0) {
    double acc = 0.;
    for (int i = n - 1; i >= 0; --i) { const double x = double(sigma[i]); acc = fma(x, x, acc); suffix[i] = acc; }
    s_total = acc;
  }
  __syncthreads();
  const double limit = s_total * eps_sq; const bool keep_all = eps_sq == 0.;
  __shared__ int s_count;
  if (threadIdx.x == 0) s_count = 0;
  __syncthreads();
  int mine = 0;
  for (int i = threadIdx.x; i < K; i += blockDim.x) {
    const bool keep = keep_all || (i < n && limit < suffix[i]);
    mine += keep ? 1 : 0;
    Num<S>::store(out + i, keep ? double(sigma[i]) : 0.);
  }
  atomicAdd(&s_count, mine);
  __syncthreads();
  if (threadIdx.x == 0) *rank = s_count;
}


// ---- planar complex half ------------------------------------------------------------------------------------
__global__ void split_complex_half_kernel(int trans, int conj, int64_t row0, int rows, int cols, const __half2* __restrict__ src, int64_t lds,
                                          __half* __restrict__ re, __half* __restrict__ im, int64_t ld) {
  // 32 x 32 tile through shared memory so that both the read and the write run along the fast index
  __shared__ __half2 tile[32][33];
  const int r0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
  if (!trans) {
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
      const int r = r0 + threadIdx.x, c = c0 + j;
      if (r < rows && c < cols) { const __half2 v = src[row0 + r + int64_t(c) * lds]; re[r + int64_t(c) * ld] = v.x; im[r + int64_t(c) * ld] = conj ? __hneg(v.y) : v.y; }
    }
    return;
  }
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int c = c0 + threadIdx.x, r = r0 + j;                   // stored cols x rows: element (c, row0 + r)
    if (r < rows && c < cols) tile[j][threadIdx.x] = src[c + (row0 + r) * lds];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int r = r0 + threadIdx.x, c = c0 + j;
    if (r < rows && c < cols) { const __half2 v = tile[threadIdx.x][j]; re[r + int64_t(c) * ld] = v.x; im[r + int64_t(c) * ld] = conj ? __hneg(v.y) : v.y; }
  }
}
__global__ void split_complex_half_b_kernel(int rows, int cols, const __half2* __restrict__ src, int64_t lds, __half* __restrict__ panels, int64_t ld) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x, c = blockIdx.y;
  if (r >= rows) return;
  const __half2 v = src[r + int64_t(c) * lds];
  const int64_t panel = ld * cols, at = r + int64_t(c) * ld;
  panels[at] = __hneg(v.y); panels[at + panel] = v.x; panels[at + 2 * panel] = v.y;
}
__global__ void merge_complex_half_kernel(int rows, int cols, const __half* __restrict__ re, const __half* __restrict__ im, int64_t ld,
                                          __half2* __restrict__ dst, int64_t ldd) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x, c = blockIdx.y;
  if (r < rows) dst[r + int64_t(c) * ldd] = __halves2half2(re[r + int64_t(c) * ld], im[r + int64_t(c) * ld]);
}
}  // namespace

void convert_copy(cudaStream_t stream, char op, int rows, int cols, hyacinPrecision_t src_type, const void* src, int64_t lds,
                  hyacinPrecision_t dst_type, void* dst, int64_t ldd) {
  if (rows <= 0 || cols <= 0) return;
  count_launch();
  const int cplx = is_complex(src_type);
  switch (base_type(src_type)) {
    case HYACIN_F64: dispatch_dst<double>(stream, op, rows, cols, cplx, src, lds, base_type(dst_type), dst, ldd); break;
    case HYACIN_F32: dispatch_dst<float>(stream, op, rows, cols, cplx, src, lds, base_type(dst_type), dst, ldd); break;
    case HYACIN_F16: dispatch_dst<__half>(stream, op, rows, cols, cplx, src, lds, base_type(dst_type), dst, ldd); break;
    default: break;
  }
  HYB_CUDA(cudaGetLastError());
}

void factor_to_columns(cudaStream_t stream, int n, int rank, hyacinPrecision_t gtype, const void* Rc, int64_t ldc, const int32_t* pos,
                       hyacinPrecision_t dst_type, void* A, int64_t lda) {
  if (n <= 0 || rank <= 0) return;
  count_launch();
  dim3 grid((n + 31) / 32, (rank + 31) / 32), block(32, 8);
#define ARGS(S, D) n, rank, static_cast<const S*>(Rc), ldc, pos, static_cast<D*>(A), lda
  const int cplx = is_complex(gtype); const bool to_f64 = base_type(dst_type) == HYACIN_F64;
  switch (base_type(gtype)) {
    case HYACIN_F32:
      if (cplx) { if (to_f64) factor_to_columns_kernel<float, double, 2><<<grid, block, 0, stream>>>(ARGS(float, double)); else factor_to_columns_kernel<float, float, 2><<<grid, block, 0, stream>>>(ARGS(float, float)); }
      else { if (to_f64) factor_to_columns_kernel<float, double, 1><<<grid, block, 0, stream>>>(ARGS(float, double)); else factor_to_columns_kernel<float, float, 1><<<grid, block, 0, stream>>>(ARGS(float, float)); }
      break;
    case HYACIN_F64:
      if (cplx) { if (to_f64) factor_to_columns_kernel<double, double, 2><<<grid, block, 0, stream>>>(ARGS(double, double)); else factor_to_columns_kernel<double, float, 2><<<grid, block, 0, stream>>>(ARGS(double, float)); }
      else { if (to_f64) factor_to_columns_kernel<double, double, 1><<<grid, block, 0, stream>>>(ARGS(double, double)); else factor_to_columns_kernel<double, float, 1><<<grid, block, 0, stream>>>(ARGS(double, float)); }
      break;
    case HYACIN_DD:
      if (cplx) { if (to_f64) factor_to_columns_kernel<DD, double, 2><<<grid, block, 0, stream>>>(ARGS(DD, double)); else factor_to_columns_kernel<DD, float, 2><<<grid, block, 0, stream>>>(ARGS(DD, float)); }
      else { if (to_f64) factor_to_columns_kernel<DD, double, 1><<<grid, block, 0, stream>>>(ARGS(DD, double)); else factor_to_columns_kernel<DD, float, 1><<<grid, block, 0, stream>>>(ARGS(DD, float)); }
      break;
    default: break;
  }
#undef ARGS
  HYB_CUDA(cudaGetLastError());
}

void factor_copy_pivoted(cudaStream_t stream, int n, int rank, hyacinPrecision_t gtype, const void* Rc, int64_t ldc, const int32_t* jpiv,
                         void* B, int64_t ldb) {
  if (n <= 0 || rank <= 0) return;
  count_launch();
  factor_copy_pivoted_kernel<<<dim3((rank + 255) / 256, n), 256, 0, stream>>>(n, rank, int(gram_elem_bytes(gtype) / 4), static_cast<const uint32_t*>(Rc), ldc,
                                                                            jpiv, static_cast<uint32_t*>(B), ldb);
  HYB_CUDA(cudaGetLastError());
}

void factor_to_pivoted(cudaStream_t stream, int n, int rank, hyacinPrecision_t gtype, const void* Rc, int64_t ldc, const int32_t* jpiv,
                       hyacinPrecision_t dst_type, void* B, int64_t ldb) {
  if (n <= 0 || rank <= 0) return;
  count_launch();
  dim3 grid((rank + 255) / 256, n);
#define ARGS(S, D) n, rank, static_cast<const S*>(Rc), ldc, jpiv, static_cast<D*>(B), ldb
  const int cplx = is_complex(gtype); const bool to_f64 = base_type(dst_type) == HYACIN_F64;
  switch (base_type(gtype)) {
    case HYACIN_F32:
      if (cplx) { if (to_f64) factor_to_pivoted_kernel<float, double, 2><<<grid, 256, 0, stream>>>(ARGS(float, double)); else factor_to_pivoted_kernel<float, float, 2><<<grid, 256, 0, stream>>>(ARGS(float, float)); }
      else { if (to_f64) factor_to_pivoted_kernel<float, double, 1><<<grid, 256, 0, stream>>>(ARGS(float, double)); else factor_to_pivoted_kernel<float, float, 1><<<grid, 256, 0, stream>>>(ARGS(float, float)); }
      break;
    case HYACIN_F64:
      if (cplx) { if (to_f64) factor_to_pivoted_kernel<double, double, 2><<<grid, 256, 0, stream>>>(ARGS(double, double)); else factor_to_pivoted_kernel<double, float, 2><<<grid, 256, 0, stream>>>(ARGS(double, float)); }
      else { if (to_f64) factor_to_pivoted_kernel<double, double, 1><<<grid, 256, 0, stream>>>(ARGS(double, double)); else factor_to_pivoted_kernel<double, float, 1><<<grid, 256, 0, stream>>>(ARGS(double, float)); }
      break;
    case HYACIN_DD:
      if (cplx) { if (to_f64) factor_to_pivoted_kernel<DD, double, 2><<<grid, 256, 0, stream>>>(ARGS(DD, double)); else factor_to_pivoted_kernel<DD, float, 2><<<grid, 256, 0, stream>>>(ARGS(DD, float)); }
      else { if (to_f64) factor_to_pivoted_kernel<DD, double, 1><<<grid, 256, 0, stream>>>(ARGS(DD, double)); else factor_to_pivoted_kernel<DD, float, 1><<<grid, 256, 0, stream>>>(ARGS(DD, float)); }
      break;
    default: break;
  }
#undef ARGS
  HYB_CUDA(cudaGetLastError());
}

void interp_scatter(cudaStream_t stream, int n, int rank, const int32_t* jpiv, hyacinPrecision_t b_type, const void* B, int64_t ldb,
                    hyacinPrecision_t xtype, void* X, int64_t ldx) {
  if (n <= 0 || rank <= 0) return;
  count_launch();
  dim3 grid((rank + 255) / 256, n);
  const int cplx = is_complex(xtype);
#define RUN(S, D) do { if (cplx) interp_scatter_kernel<S, D, 2><<<grid, 256, 0, stream>>>(n, rank, jpiv, static_cast<const S*>(B), ldb, static_cast<D*>(X), ldx); \
                       else interp_scatter_kernel<S, D, 1><<<grid, 256, 0, stream>>>(n, rank, jpiv, static_cast<const S*>(B), ldb, static_cast<D*>(X), ldx); } while (0)
  const bool b64 = base_type(b_type) == HYACIN_F64;
  switch (base_type(xtype)) {
    case HYACIN_F64: if (b64) RUN(double, double); else RUN(float, double); break;
    case HYACIN_F32: if (b64) RUN(double, float); else RUN(float, float); break;
    case HYACIN_F16: if (b64) RUN(double, __half); else RUN(float, __half); break;
    default: break;
  }
#undef RUN
  HYB_CUDA(cudaGetLastError());
}

void find_rank(cudaStream_t stream, double eps_sq, int n, int K, hyacinPrecision_t sigma_type, const void* sigma, hyacinPrecision_t out_type,
               void* out, int32_t* rank, double* suffix) {
  const bool s64 = base_type(sigma_type) == HYACIN_F64;
  count_launch();
#define RUN(R, S) find_rank_kernel<R, S><<<1, 256, 0, stream>>>(eps_sq, n, K, static_cast<const R*>(sigma), static_cast<S*>(out), rank, suffix)
  switch (base_type(out_type)) {
    case HYACIN_F64: if (s64) RUN(double, double); else RUN(float, double); break;
    case HYACIN_F32: if (s64) RUN(double, float); else RUN(float, float); break;
    case HYACIN_F16: if (s64) RUN(double, __half); else RUN(float, __half); break;
    default: break;
  }
#undef RUN
  HYB_CUDA(cudaGetLastError());
}

void split_complex_half(cudaStream_t stream, char op, int64_t row0, int rows, int cols, const void* src, int64_t lds, void* re, void* im, int64_t ld) {
  if (rows <= 0 || cols <= 0) return;
  const int trans = op == 'T' || op == 'C';
  split_complex_half_kernel<<<dim3((rows + 31) / 32, (cols + 31) / 32), dim3(32, 8), 0, stream>>>(
      trans, op == 'C', row0, rows, cols, static_cast<const __half2*>(src), lds, static_cast<__half*>(re), static_cast<__half*>(im), ld);
  HYB_CUDA(cudaGetLastError());
}
// The planes in the stored layout (no transposition): element (r, c) of the stored matrix to re / im [r + c ld], the
// imaginary plane negated when conj is set.
void split_complex_half_stored(cudaStream_t stream, bool conj, int rows, int cols, const void* src, int64_t lds, void* re, void* im, int64_t ld) {
  if (rows <= 0 || cols <= 0) return;
  split_complex_half_kernel<<<dim3((rows + 31) / 32, (cols + 31) / 32), dim3(32, 8), 0, stream>>>(
      0, conj ? 1 : 0, 0, rows, cols, static_cast<const __half2*>(src), lds, static_cast<__half*>(re), static_cast<__half*>(im), ld);
  HYB_CUDA(cudaGetLastError());
}
void split_complex_half_b(cudaStream_t stream, int rows, int cols, const void* src, int64_t lds, void* panels, int64_t ld) {
  if (rows <= 0 || cols <= 0) return;
  split_complex_half_b_kernel<<<dim3((rows + 127) / 128, cols), 128, 0, stream>>>(rows, cols, static_cast<const __half2*>(src), lds, static_cast<__half*>(panels), ld);
  HYB_CUDA(cudaGetLastError());
}
void merge_complex_half(cudaStream_t stream, int rows, int cols, const void* re, const void* im, int64_t ld, void* dst, int64_t ldd) {
  if (rows <= 0 || cols <= 0) return;
  merge_complex_half_kernel<<<dim3((rows + 127) / 128, cols), 128, 0, stream>>>(rows, cols, static_cast<const __half*>(re), static_cast<const __half*>(im), ld, static_cast<__half2*>(dst), ldd);
  HYB_CUDA(cudaGetLastError());
}

}  // namespace hyb
