/*
 * oracle_gram.c -- CPU restatement of Hyacin's quantized-Gram path.  TEST INFRASTRUCTURE ONLY.
 *
 * Nothing in the product library links, loads or calls this file.  It exists so that tests, the smoke
 * check and the benchmark's CPU leg have an independent statement of what the GPU path must produce.
 *
 * Parity status: the reference ships no tests, golden vectors or known-answer files for this path, so this
 * restatement is pinned against outputs of the reference's own CUDA library (built from its sources by
 * oracle/Makefile and run on a B200) that are committed as fixtures under tests/golden/.
 *
 * Every function cites the reference source it follows (paths relative to the reference project root).
 * Integer results (exponents, quantised values, the packed integer Gram) are exact; the floating-point
 * dequantisation repeats the reference's operation order so that its results are bit-identical.
 *
 * Build: gcc -O2 -std=c11 -ffp-contract=off -fPIC -shared oracle_gram.c -o liboracle.so -lm
 */
#include <limits.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <float.h>

typedef __int128 i128;
typedef unsigned __int128 u128;

enum { ORC_F64 = 0, ORC_F32 = 2 };   /* element kinds understood here; complex = interleaved pairs */

/* ---------------------------------------------------------------------------------------------------
 * Sizing of the integer Gram.  Follows src/hyacin_herk.cpp:45-59.
 *   u       = clamp([frac(eps)==0.5] - exp(eps), 0, mantissa(type))       (frexp convention)
 *   u_corr  = max(-1, min(80, corr + u))
 *   cPanels = 1 + complex
 *   lPanels = (63 + max(0, 2 (u_corr + complex)) + ceil(log2(pow2ceil(globalM)))) / 63, 0 when u_corr < 0
 * atype is the hyacinPrecision_t value (0..11).
 * ------------------------------------------------------------------------------------------------- */
void orc_herk_init(double eps, uint64_t globalM, int32_t N, int32_t atype, int32_t corr,
                   int32_t* u_out, int32_t* cpanels, int32_t* lpanels, uint64_t* stride) {
  static const int mantissa[12] = {52, 52, 23, 23, 10, 10, 105, 105, 71, 71, 95, 95};
  uint64_t n = N > 0 ? (uint64_t)N : 0;
  if (stride) *stride = (n * n + n) >> 1;
  uint64_t m = globalM;
  int log2m = 0;
  if (m > 1) { m -= 1; while (m) { log2m++; m >>= 1; } }     /* ceil(log2(M)) for M >= 2, 0 otherwise */
  int e; double f = frexp(fabs(eps), &e);
  int u = (f == 0.5 ? 1 : 0) - e;
  if (u < 0) u = 0;
  if (u > mantissa[atype]) u = mantissa[atype];
  int cplx = atype & 1;
  int ucorr = corr + u; if (ucorr > 80) ucorr = 80; if (ucorr < -1) ucorr = -1;
  if (u_out) *u_out = ucorr;
  if (cpanels) *cpanels = 1 + cplx;
  if (lpanels) {
    int t = (ucorr + cplx) * 2; if (t < 0) t = 0;
    *lpanels = ucorr >= 0 ? (63 + t + log2m) / 63 : 0;
  }
}

/* ---------------------------------------------------------------------------------------------------
 * Column exponents.  Follows src/fp_exponent.cu:20-51.
 *   mexp[b][j] = u - e   with  max_i |a_ij| = f * 2^e, f in [1/2, 1)   over the rows of segment b
 *   a maximum below the smallest normal number of the element type gives INT_MAX (zero column)
 *   vexp[0][j] = min_b mexp[b][j];   rows 1..batches of vexp are mexp
 *   batches <= 0 or u < 0: vexp[0][*] = INT_MAX and nothing else is written
 * Complex columns use max(|re|, |im|) (fp_exponent.cu:32).  `kind` is ORC_F64 or ORC_F32; half inputs are
 * widened to float by the caller (exact).  lda counts elements (complex elements for complex input).
 * ------------------------------------------------------------------------------------------------- */
static double elem_abs(const void* A, int kind, int cplx, int64_t idx) {
  if (kind == ORC_F64) {
    const double* p = (const double*)A;
    if (cplx) { double r = fabs(p[2 * idx]), i = fabs(p[2 * idx + 1]); return fmax(r, i); }
    return fabs(p[idx]);
  } else {
    const float* p = (const float*)A;
    if (cplx) { float r = fabsf(p[2 * idx]), i = fabsf(p[2 * idx + 1]); return (double)fmaxf(r, i); }
    return (double)fabsf(p[idx]);
  }
}

void orc_column_exponents(int32_t kind, int32_t cplx, int32_t batches, int32_t segM, int32_t lastM, int32_t N,
                          const void* A, int64_t lda, int32_t u, int32_t* vexp) {
  if (N <= 0) return;
  if (batches <= 0 || u < 0) { for (int j = 0; j < N; ++j) vexp[j] = INT_MAX; return; }
  const double tiny = kind == ORC_F64 ? DBL_MIN : (double)FLT_MIN;
  for (int j = 0; j < N; ++j) {
    int32_t best = INT_MAX;
    for (int b = 0; b < batches; ++b) {
      int rows = (b + 1 == batches) ? lastM : segM;
      double mx = 0.0;
      for (int i = 0; i < rows; ++i) {
        double a = elem_abs(A, kind, cplx, (int64_t)b * segM + i + (int64_t)j * lda);
        mx = fmax(mx, a);
      }
      int32_t m;
      if (mx < tiny) m = INT_MAX; else { int e; frexp(mx, &e); m = u - e; }
      vexp[(int64_t)(1 + b) * N + j] = m;
      if (m < best) best = m;
    }
    vexp[j] = best;
  }
}

/* Bits a row segment really needs: segU[b] = u + max_j (vexp[0][j] - vexp[1+b][j]) over non-zero columns
 * of the segment, INT_MIN when the segment is all zero.  Follows src/fp_exponent.cu:67-73. */
void orc_vector_range(int32_t batches, int32_t N, int32_t u, const int32_t* vexp, int32_t* segU) {
  for (int b = 0; b < batches; ++b) {
    int32_t best = INT_MIN;
    for (int j = 0; j < N; ++j) {
      int32_t e = vexp[(int64_t)(1 + b) * N + j];
      if (e < INT_MAX) { int32_t d = vexp[j] - e; if (d > best) best = d; }
    }
    segU[b] = best == INT_MIN ? INT_MIN : u + best;
  }
}

/* ---------------------------------------------------------------------------------------------------
 * Quantiser.  Follows src/quantize_limbs.cu:14-27 (round_i95) and :46-58:
 *   q = rint_ties_to_even(a * 2^expon), formed as  llrint(scalbn(a, expon - e)) << e  with
 *   e = max(ilogb(a) + expon - 62, 0);  a zero-marked column (expon == INT_MAX) quantises to 0.
 * The shift only engages when |a 2^expon| >= 2^62, where the scaled value is already an integer, so the
 * result equals the correctly rounded product in every case.  ftz != 0 treats single-precision
 * subnormal inputs as zero, which is what the reference's fast-math build does to them.
 * Output layout: q[(part * N + j) * M + i], part 0 = real, part 1 = imaginary.
 * ------------------------------------------------------------------------------------------------- */
static i128 quantize_one(double a, int32_t expon) {
  if (a == 0.0 || expon == INT_MAX) return 0;
  int il = ilogb(a);
  long e = (long)il + (long)expon - 62; if (e < 0) e = 0;
  double s = scalbn(a, (int)((long)expon - e));
  long long i = llrint(s);                     /* default rounding mode: ties to even */
  return (i128)i << e;
}

void orc_quantize(int32_t kind, int32_t cplx, int32_t ftz, int32_t M, int32_t N, const void* A, int64_t lda,
                  const int32_t* vexp, i128* q) {
  for (int j = 0; j < N; ++j) for (int i = 0; i < M; ++i) {
    int64_t idx = i + (int64_t)j * lda;
    for (int part = 0; part <= cplx; ++part) {
      double a;
      if (kind == ORC_F64) a = ((const double*)A)[cplx ? 2 * idx + part : idx];
      else {
        float f = ((const float*)A)[cplx ? 2 * idx + part : idx];
        if (ftz && fabsf(f) < FLT_MIN) f = 0.f;
        a = (double)f;
      }
      q[((int64_t)part * N + j) * M + i] = quantize_one(a, vexp[j]);
    }
  }
}

/* ---------------------------------------------------------------------------------------------------
 * 256-bit two's-complement helpers for the exact accumulation.
 * ------------------------------------------------------------------------------------------------- */
typedef struct { uint64_t w[4]; } big_t;

static void big_add_i128_shifted(big_t* x, i128 v, int shift) {
  uint64_t t[4]; uint64_t ext = v < 0 ? ~(uint64_t)0 : 0;
  t[0] = (uint64_t)(u128)v; t[1] = (uint64_t)((u128)v >> 64); t[2] = ext; t[3] = ext;
  int ws = shift / 64, bs = shift % 64;
  uint64_t s[4];
  for (int k = 3; k >= 0; --k) {
    uint64_t lo = (k - ws >= 0) ? t[k - ws] : 0, below = (k - ws - 1 >= 0) ? t[k - ws - 1] : 0;
    s[k] = bs ? (lo << bs) | (below >> (64 - bs)) : lo;
  }
  unsigned carry = 0;
  for (int k = 0; k < 4; ++k) {
    u128 a = (u128)x->w[k] + s[k] + carry; x->w[k] = (uint64_t)a; carry = (unsigned)(a >> 64);
  }
}

static void big_sar63(big_t* x) {   /* arithmetic shift right by 63 */
  uint64_t ext = (x->w[3] >> 63) ? ~(uint64_t)0 : 0;
  uint64_t n0 = (x->w[0] >> 63) | (x->w[1] << 1), n1 = (x->w[1] >> 63) | (x->w[2] << 1);
  uint64_t n2 = (x->w[2] >> 63) | (x->w[3] << 1), n3 = (x->w[3] >> 63) | (ext << 1);
  x->w[0] = n0; x->w[1] = n1; x->w[2] = n2; x->w[3] = n3;
}

/* Packed limb format of the integer Gram (src/limbs_diag.cu:24, include/internal.hpp:116-159):
 *   value = a0 + a1 2^63 (+ a2 2^126); all limbs but the last lie in [0, 2^63); the last is a signed int64.
 *   plane stride between limbs = tri = N(N+1)/2; element (y <= x) sits at y + x(x+1)/2. */
static void big_to_limbs(big_t x, int order, uint64_t* out, int64_t stride) {
  const uint64_t m63 = ~(uint64_t)0 >> 1;
  for (int l = 0; l < order; ++l) {
    if (l + 1 == order) out[l * stride] = x.w[0];
    else { out[l * stride] = x.w[0] & m63; big_sar63(&x); }
  }
}

static big_t limbs_to_big(int order, const uint64_t* in, int64_t stride) {
  big_t x; memset(&x, 0, sizeof x);
  for (int l = 0; l < order; ++l) big_add_i128_shifted(&x, (i128)(int64_t)in[l * stride], 63 * l);
  return x;
}

/* ---------------------------------------------------------------------------------------------------
 * Exact integer Gram of the quantised matrix in the packed limb format.
 *   real:     C[y,x]    = sum_k q[k,y] q[k,x]
 *   complex:  Cre[y,x]  = sum_k (re_y re_x + im_y im_x),  Cim[y,x] = sum_k (re_y im_x - im_y re_x)
 * The reference reaches the same integers through int8 limb products (src/limbs_diag.cu,
 * src/limbs_cross_real.cu, src/limbs_cross_imag.cu:41-42) or CRT residues (src/crt_diag_real.cu,
 * src/crt_rotate.cu:10-11, src/crt_reconstruct_real.cu); both are exact, so the sum of products is the
 * contract.  Panel order is [re limbs][im limbs] (src/fp_i63tp_dequantize.cu:100-102).  beta != 0 adds
 * to the existing C (src/hyacin_herk.cpp:306).
 * ------------------------------------------------------------------------------------------------- */
static void split40(i128 q, i128* hi, i128* lo) {
  const i128 mask = (((i128)1) << 40) - 1;
  *lo = q & mask; *hi = q >> 40;    /* arithmetic shift: q = hi 2^40 + lo, 0 <= lo < 2^40 */
}

void orc_gram_exact(int32_t cplx, int32_t M, int32_t N, const i128* q, int32_t order, int32_t beta, uint64_t* C) {
  int64_t tri = ((int64_t)N * N + N) / 2;
  for (int x = 0; x < N; ++x) for (int y = 0; y <= x; ++y) {
    for (int part = 0; part <= cplx; ++part) {
      i128 s0 = 0, s1 = 0, s2 = 0;
      for (int term = 0; term <= cplx; ++term) {
        /* real part: re_y re_x + im_y im_x ; imaginary part: re_y im_x - im_y re_x */
        const i128 *qy, *qx; int neg = 0;
        if (part == 0) { qy = q + ((int64_t)term * N + y) * M; qx = q + ((int64_t)term * N + x) * M; }
        else if (term == 0) { qy = q + (int64_t)y * M; qx = q + ((int64_t)N + x) * M; }
        else { qy = q + ((int64_t)N + y) * M; qx = q + (int64_t)x * M; neg = 1; }
        i128 t0 = 0, t1 = 0, t2 = 0;
        for (int k = 0; k < M; ++k) {
          i128 yh, yl, xh, xl; split40(qy[k], &yh, &yl); split40(qx[k], &xh, &xl);
          t0 += yl * xl; t1 += yh * xl + yl * xh; t2 += yh * xh;
        }
        if (neg) { s0 -= t0; s1 -= t1; s2 -= t2; } else { s0 += t0; s1 += t1; s2 += t2; }
      }
      uint64_t* dst = C + (int64_t)part * order * tri + y + ((int64_t)x * (x + 1)) / 2;
      big_t acc; memset(&acc, 0, sizeof acc);
      if (beta) acc = limbs_to_big(order, dst, tri);
      big_add_i128_shifted(&acc, s0, 0); big_add_i128_shifted(&acc, s1, 40); big_add_i128_shifted(&acc, s2, 80);
      big_to_limbs(acc, order, dst, tri);
    }
  }
}

/* Cross-rank reduction: plain integer sum of `count` packed values held by `ranks` arrays laid out one
 * after another in `in` (each panels * order * count words).  The reference re-slices the limbs so that an
 * unsigned 64-bit sum cannot overflow and re-assembles them afterwards (src/allreduce_1drow.cu:81-131,
 * 145-169); the result is the exact sum whatever the slicing. */
void orc_allreduce_sum(int32_t ranks, int32_t panels, int32_t order, int64_t count, const uint64_t* in, uint64_t* out) {
  int64_t per_rank = (int64_t)panels * order * count;
  for (int p = 0; p < panels; ++p) for (int64_t i = 0; i < count; ++i) {
    big_t acc; memset(&acc, 0, sizeof acc);
    for (int r = 0; r < ranks; ++r) {
      const uint64_t* src = in + r * per_rank + (int64_t)p * order * count + i;
      for (int l = 0; l < order; ++l) big_add_i128_shifted(&acc, (i128)(int64_t)src[l * count], 63 * l);
    }
    big_to_limbs(acc, order, out + (int64_t)p * order * count + i, count);
  }
}

/* ---------------------------------------------------------------------------------------------------
 * Choice of the floating-point format of the dequantised Gram.  Follows
 * src/fp_i63tp_dequantize.cu:6-26 (bit length of the diagonal entry with the largest true-scale
 * magnitude; ties resolved towards the longer integer) and :41-53 (thresholds 23 / 52 / 71 / 95 bits after
 * removing 2*corr guard bits; triple- and quad-float only on GPUs without fast FP64).
 * Returns the hyacinPrecision_t value of G; *elem_bytes receives its element size.
 * ------------------------------------------------------------------------------------------------- */
static int bitlen64(uint64_t a) { int n = 0; while (a) { n++; a >>= 1; } return n; }

int32_t orc_dequantize_init(int32_t N, int32_t order, const uint64_t* C, const int32_t* vexp, int32_t atype,
                            int32_t corr, int32_t f64_capable, int32_t* elem_bytes, int32_t* bits_out) {
  static const int bytes[12] = {8, 16, 4, 8, 2, 4, 16, 32, 12, 24, 16, 32};
  int64_t tri = ((int64_t)N * N + N) / 2;
  int best_key = INT_MIN, best_e = 0;
  for (int i = 0; i < N; ++i) {
    if (vexp[i] == INT_MAX) continue;
    const uint64_t* d = C + ((int64_t)i * (i + 3)) / 2;
    int e = bitlen64(d[0]);
    if (order > 1) { int en = 63 + bitlen64(d[tri]); if (en > 63) e = en; }
    if (order > 2) { int en = 126 + bitlen64(d[2 * tri]); if (en > 126) e = en; }
    int key = e - 2 * vexp[i];
    if (key > best_key || (key == best_key && e > best_e)) { best_key = key; best_e = e; }
  }
  int bits = best_e - 2 * corr;
  if (bits_out) *bits_out = bits;
  int g;   /* complex flavour first, as in the reference */
  if (bits <= 23) g = 3; else if (bits <= 52) g = 1;
  else if (bits <= 71 && !f64_capable) g = 9; else if (bits <= 95 && !f64_capable) g = 11; else g = 7;
  if (!(atype & 1)) g -= 1;
  if (elem_bytes) *elem_bytes = bytes[g];
  return g;
}

/* ---------------------------------------------------------------------------------------------------
 * Dequantisation.  Follows src/fp_i63tp_dequantize.cu:56-69 (conversion order), :100-102 (complex panel
 * order), :121-129 (scale 2^-(vexp[x]+vexp[y]), zero rows/columns, Hermitian mirror) and the double-double
 * helpers of include/internal.hpp:181-214.  gtype: 0 F64, 1 F64 complex, 2 F32, 3 F32 complex, 6 DD,
 * 7 DD complex.  G is column-major with leading dimension ldg (in elements of the Gram type).
 * ------------------------------------------------------------------------------------------------- */
typedef struct { double x, y; } dd_t;

static dd_t i64_split(uint64_t i) {   /* (high 32 bits as signed) * 2^32, low 32 bits as unsigned */
  dd_t r; r.x = scalbn((double)(int32_t)(i >> 32), 32); r.y = (double)(uint32_t)i; return r;
}
static dd_t dd_renorm(dd_t a) { double s = a.x + a.y, d = a.x - s; dd_t r = {s, a.y + d}; return r; }
static dd_t dd_add(dd_t a, dd_t b) {
  double s = a.x + b.x, d = a.x - s, sd = s + d, e = (b.x + d) + (a.x - sd);
  dd_t t = {s, (a.y + b.y) + e}; return dd_renorm(t);
}

static double limbs_to_f64(int order, const uint64_t* a, int64_t stride, int e) {
  double res = (double)(int64_t)a[(order - 1) * stride];
  for (int l = order - 2; l >= 0; --l) { dd_t i = i64_split(a[l * stride]); res = (scalbn(res, 63) + i.x) + i.y; }
  return scalbn(res, e);
}

static dd_t limbs_to_dd(int order, const uint64_t* a, int64_t stride, int e) {
  dd_t res = dd_renorm(i64_split(a[(order - 1) * stride]));
  for (int l = order - 2; l >= 0; --l) {
    dd_t sh = {scalbn(res.x, 63), scalbn(res.y, 63)};
    res = dd_add(sh, dd_renorm(i64_split(a[l * stride])));
  }
  dd_t out = {scalbn(res.x, e), scalbn(res.y, e)}; return out;
}

void orc_dequantize(int32_t N, int32_t order, const uint64_t* C, const int32_t* vexp, int32_t gtype, void* G, int64_t ldg) {
  int64_t tri = ((int64_t)N * N + N) / 2;
  int cplx = gtype & 1, base = gtype & ~1;
  for (int x = 0; x < N; ++x) for (int y = 0; y <= x; ++y) {
    int zero = vexp[x] == INT_MAX || vexp[y] == INT_MAX;
    int e = zero ? 0 : -(vexp[x] + vexp[y]);
    const uint64_t* re = C + y + ((int64_t)x * (x + 1)) / 2;
    const uint64_t* im = re + (int64_t)order * tri;
    int64_t up = y + x * ldg, lo = x + y * ldg;
    if (base == 0) {
      double* g = (double*)G; double r = zero ? 0.0 : limbs_to_f64(order, re, tri, e);
      if (cplx) { double i = zero ? 0.0 : limbs_to_f64(order, im, tri, e);
        g[2 * up] = r; g[2 * up + 1] = i; g[2 * lo] = r; g[2 * lo + 1] = -i; }
      else { g[up] = r; g[lo] = r; }
    } else if (base == 2) {
      float* g = (float*)G; float r = zero ? 0.f : (float)limbs_to_f64(order, re, tri, e);
      if (cplx) { float i = zero ? 0.f : (float)limbs_to_f64(order, im, tri, e);
        g[2 * up] = r; g[2 * up + 1] = i; g[2 * lo] = r; g[2 * lo + 1] = -i; }
      else { g[up] = r; g[lo] = r; }
    } else if (base == 6) {
      dd_t* g = (dd_t*)G; dd_t z = {0.0, 0.0}; dd_t r = zero ? z : limbs_to_dd(order, re, tri, e);
      if (cplx) { dd_t i = zero ? z : limbs_to_dd(order, im, tri, e); dd_t ni = {-i.x, -i.y};
        g[2 * up] = r; g[2 * up + 1] = i; g[2 * lo] = r; g[2 * lo + 1] = ni; }
      else { g[up] = r; g[lo] = r; }
    }
  }
}

/* ---- truncated pivoted Cholesky of a Gram matrix, FP64 real or complex -----------------------------------------
 * Restates what fixes the BITS of the reference's factor (src/hyacin_potrfp.cu:214-272), sequentially:
 *   - the new row of a column is  w = G[l, j] - sum_m conj(R[m, l]) R[m, j]  summed as 128 chains (chain t takes the
 *     previous rows t, t + 128, ... in order with fused multiply-adds, chain 0 starts from the Gram entry; :226-230),
 *     combined per 32 chains by the tree (x_i + x_{i+1}) + (x_{i+2} + x_{i+3}) ... and then left to right over the four
 *     groups (the block reduction of :231); the first step has no sum (:223);
 *   - entry r = w / sqrt(d) as a product with 1 / sqrt(d), diagonal d -= |r|^2 by fused multiply-adds (:172-176);
 *   - pivot = largest remaining diagonal entry, ties to the candidate the reference's reduction meets first (:243-261);
 *   - stop when the remaining trace <= eps^2 * initial trace, or N - K columns are left; a single remaining column is
 *     always counted (:262-269); both traces are summed in the order of the reference's reduction, so the comparison
 *     has the reference's bits even when it is taken on rounding noise (exactly rank-deficient matrices).
 * Only the double formats are restated: their arithmetic is explicit fused multiply-adds.  The double-double formats
 * depend on which products the device compiler contracts and are checked against the reference library on the GPU.
 * G: n x n column-major (2 doubles per entry if cplx).  R: rows x n column-major BY POSITION, R[k + x ldr] for k <= x,
 * zero elsewhere (what the reference leaves in the upper triangle of its Gram matrix).  jpiv: one-based.  Returns rank. */
static int chol_key(int th, int second) {
  int b = th >> 7, t = th & 127, walker = 0, turn = 0;
  if (b > 0) { walker = (b - 1) & 127; turn = ((b - 1) >> 7) + (walker == 0 ? 1 : 0); }
  return (((walker * 32 + turn) * 128 + t) << 1) | second;
}
static double tree128(const double* x) {
  double g[4];
  for (int w = 0; w < 4; ++w) {
    double v[32];
    for (int i = 0; i < 32; ++i) v[i] = x[32 * w + i];
    for (int o = 1; o < 32; o <<= 1) for (int i = 0; i + o < 32; i += 2 * o) v[i] = v[i] + v[i + o];
    g[w] = v[0];
  }
  return ((g[0] + g[1]) + g[2]) + g[3];
}

/* Remaining trace in the order of the reference's reduction (src/hyacin_potrfp.cu:243-261, 128-132): candidate number th sits
 * in thread th % 128 of block th / 128; thread 0 of block 0 first takes the one extra value `special` (the column swapped
 * into the pivot's old place), then its own; a block sums its 128 threads by the shuffle tree and its four warps left to
 * right; thread t of block 0 then adds the sums of blocks t + 1, t + 129, ... to its own (thread 0: its block's sum, the
 * others: zero) and the 128 threads are summed by the same tree.  Valid while every thread holds at most one candidate
 * (n <= 148 * 128 on a B200 whatever the occupancy of the reference's kernel). */
static double trace_in_reference_order(const double* d, int count, int have_special, double special) {
  const int nb = count > 0 ? (count + 127) / 128 : 1;
  double* agg = (double*)malloc((size_t)nb * sizeof(double));
  for (int b = 0; b < nb; ++b) {
    double x[128];
    for (int t = 0; t < 128; ++t) { const int th = 128 * b + t; x[t] = th < count ? d[th] : 0.0; }
    if (b == 0 && have_special) x[0] = (0.0 + special) + x[0];
    agg[b] = tree128(x);
  }
  double u[128];
  for (int t = 0; t < 128; ++t) { u[t] = t == 0 ? agg[0] : 0.0; for (int i = t + 1; i < nb; i += 128) u[t] += agg[i]; }
  const double out = tree128(u);
  free(agg);
  return out;
}

/* exported for the tests of the summation order itself */
double orc_trace_in_reference_order(const double* d, int32_t count, int32_t have_special, double special) {
  return trace_in_reference_order(d, count, have_special, special);
}

int32_t orc_potrfp_f64(int32_t n, int32_t cap, double eps, int32_t cplx, const double* G, int64_t ldg, int32_t* jpiv, double* R, int64_t ldr) {
  const int w = cplx ? 2 : 1;
  if (n <= 0 || cap <= 0) return 0;
  if (cap > n) cap = n;
  const int rows = cap + 1 < n ? cap + 1 : n;            /* a counted last column may add one row */
  double* F = (double*)calloc((size_t)n * rows * w, sizeof(double));      /* F[(col * rows + k) * w]: factor by original column */
  double* D = (double*)malloc((size_t)n * sizeof(double));
  int* perm = (int*)malloc((size_t)n * sizeof(int));
  double re[128], im[128];
  const double eps_sq = eps * eps;
  const int iter_n = cap >= n ? 1 : n - cap;
  /* first candidates: position i is the reference's candidate number i */
  double trace = 0.0, best = 0.0; int best_pos = -1, best_key = INT_MAX;
  double* cand = (double*)malloc((size_t)n * sizeof(double));      /* remaining diagonal entries by candidate number */
  for (int i = 0; i < n; ++i) {
    perm[i] = i; D[i] = G[((int64_t)i + (int64_t)i * ldg) * w]; cand[i] = D[i];
    int key = chol_key(i, 0);
    if (D[i] > 0.0 && (best_pos < 0 || best < D[i] || (best == D[i] && key < best_key))) { best = D[i]; best_pos = i; best_key = key; }
  }
  trace = trace_in_reference_order(cand, n, 0, 0.0);
  double threshold = 0.0; int rank = 0, k = 0;
  for (;; ++k) {
    const int have = best_pos >= 0;
    if (k == 0) { if (!have) { rank = 0; break; } threshold = eps_sq * trace; }
    else {
      const int remaining = n - k;
      if (!(have && threshold < trace) || remaining <= iter_n) {
        rank = k + (remaining == 1 ? 1 : 0);
        if (remaining == 1) F[((size_t)perm[k] * rows + k) * w] = sqrt(have ? best : 0.0);
        break;
      }
    }
    const int q = best_pos, j = q - k, pc = perm[q], front = perm[k];
    const double root = sqrt(best), rinv = 1.0 / root;
    F[((size_t)pc * rows + k) * w] = root;
    best = 0.0; best_pos = -1; best_key = INT_MAX;
    double special = 0.0; int count = 0;
    for (int p = k + 1; p < n; ++p) {
      const int col = p == q ? front : perm[p];
      const double* fc = F + (size_t)col * rows * w; const double* fp = F + (size_t)pc * rows * w;
      const double* g = G + ((int64_t)col + (int64_t)pc * ldg) * w;          /* row = this column, column = pivot column */
      for (int t = 0; t < 128; ++t) {
        double ar = t == 0 ? g[0] : 0.0, ai = (t == 0 && cplx) ? g[1] : 0.0;
        for (int m = t; m < k; m += 128) {
          if (cplx) {
            const double ax = fc[2 * m], ay = fc[2 * m + 1], bx = fp[2 * m], by = fp[2 * m + 1];
            const double nr = fma(-ax, bx, fma(-ay, by, ar)), ni = fma(-ax, by, fma(ay, bx, ai));
            ar = nr; ai = ni;
          } else ar = fma(-fc[m], fp[m], ar);
        }
        re[t] = ar; im[t] = ai;
      }
      double wr = k > 0 ? tree128(re) : re[0], wi = cplx ? (k > 0 ? tree128(im) : im[0]) : 0.0;
      double d = D[col];
      if (cplx) { const double rr = rinv * wr, ri = -rinv * wi; d = fma(-rr, rr, fma(-ri, ri, d)); F[((size_t)col * rows + k) * 2] = rr; F[((size_t)col * rows + k) * 2 + 1] = ri; }
      else { const double rc = rinv * wr; d = fma(-rc, rc, d); F[(size_t)col * rows + k] = rc; }
      D[col] = d;
      const int l = p - k;
      if (j > 0 && l == j) special = d; else { cand[j > 0 ? l - (l > j ? 1 : 0) - 1 : l - 1] = d; ++count; }
      const int key = (j > 0 && l == j) ? chol_key(0, 0) : (j > 0 ? chol_key(l - (l > j ? 1 : 0) - 1, 1) : chol_key(l - 1, 1));
      if (d > 0.0 && (best_pos < 0 || best < d || (best == d && key < best_key))) { best = d; best_pos = p; best_key = key; }
    }
    trace = trace_in_reference_order(cand, count, j > 0, special);
    perm[q] = front; perm[k] = pc;
  }
  free(cand);
  for (int x = 0; x < n; ++x) {
    jpiv[x] = perm[x] + 1;
    for (int kk = 0; kk < rank && kk < rows; ++kk)
      for (int c = 0; c < w; ++c) R[((int64_t)kk + (int64_t)x * ldr) * w + c] = kk <= x ? F[((size_t)perm[x] * rows + kk) * w + c] : 0.0;
  }
  free(F); free(D); free(perm);
  return rank;
}
