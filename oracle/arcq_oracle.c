/*
 * CPU oracle for the ARC-NVFP4 quantized-linear path.  TEST INFRASTRUCTURE ONLY:
 * nothing in the shipped package may call into this file; it exists so the
 * CUDA kernels can be checked bit for bit (codes, scale bytes) and within a
 * tolerance (GEMM) on small inputs.
 *
 * It restates, in plain scalar C, the arithmetic of the reference CUDA kernels
 * (paths are relative to the ARCQuant source tree):
 *
 *   kernels/src/reorder.cu:17-19     constants FP4_MAX=6, FP8_MAX=448, SCALE_EPS=2^-9
 *   kernels/src/reorder.cu:115-118   gather xr[j] = x[reorder_index[j]]
 *   kernels/src/reorder.cu:124-146   group amax, block scale, reciprocal
 *   kernels/src/reorder.cu:151-202   e2m1 codes, residual, packed row layout
 *   kernels/src/reorder.cu:139-143   scale-factor column of a group
 *   kernels/src/reorder.cu:292-329   weights: residual slot is a copy
 *   kernels/src/reorder.cu:381-555   32-channels-per-thread variant (pairs of groups)
 *   kernels/src/down.cu:71-236       same arithmetic on a pre-gathered row
 *   kernels/src/rmsnorm.cu:113-171   sum-of-squares order, normalisation
 *   kernels/src/bindings.cpp:83-95   scale-factor buffer size
 *   kernels/src/nvfp4.cu:35-132      D = alpha * (A.SFA)(B.SFB)^T, fp32 accumulate
 *
 * Number formats follow the converters those kernels use
 * (cutlass::NumericConverter<..., round_to_nearest>): float -> e2m1 and
 * float -> ue4m3 are round-to-nearest-even, saturating, and keep the sign of a
 * zero result.
 *
 * PARITY UNPINNED: the reference ships no golden vector, known-answer test or
 * fixture for this path and its kernels (sm_120a, CUTLASS not vendored) can
 * neither be built nor run here.  The pins that do exist are the known-answer
 * tables under tests/golden/ (derived from the format definitions) and the
 * cross-check of the shared structure against the reference's torch fake-quant
 * path (see oracle/fake_port.py).
 *
 * One deliberate definition: the reference computes the RMSNorm reciprocal
 * root with the device's approximate rsqrt, which no CPU can reproduce.  Here
 * (and in the CUDA kernel under test) it is the correctly rounded fp32 value
 * of 1/sqrt(v), v = fp32(fp32(ss/KQ) + eps).
 *
 * Build: gcc -O2 -ffp-contract=off -fPIC -shared (see oracle/Makefile).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ bf16 */

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* fp32 -> bf16, round to nearest even (NaN kept quiet). */
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}

uint16_t arcq_f32_to_bf16(float f) { return f32_to_bf16(f); }
float arcq_bf16_to_f32(uint16_t h) { return bf16_to_f32(h); }

/* ------------------------------------------------------------------ e2m1 */

static const float E2M1_VAL[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};

float arcq_e2m1_decode(uint8_t code) {
  float v = E2M1_VAL[code & 7];
  return (code & 8) ? -v : v;
}

/* float -> e2m1 code (4 bits), RNE, saturating at 6, sign kept on zero.
 * Midpoints go to the code with an even mantissa bit:
 * 0.25->0, 0.75->1, 1.25->1, 1.75->2, 2.5->2, 3.5->4, 5->4. */
uint8_t arcq_e2m1_encode(float x) {
  uint32_t u;
  memcpy(&u, &x, 4);
  uint8_t sign = (uint8_t)((u >> 31) << 3);
  float a = fabsf(x);
  uint8_t c;
  if (!(a == a)) c = 7;              /* NaN: the format has none; saturate */
  else if (a <= 0.25f) c = 0;
  else if (a < 0.75f) c = 1;
  else if (a <= 1.25f) c = 2;
  else if (a < 1.75f) c = 3;
  else if (a <= 2.5f) c = 4;
  else if (a < 3.5f) c = 5;
  else if (a <= 5.0f) c = 6;
  else c = 7;
  return (uint8_t)(sign | c);
}

/* ----------------------------------------------------------------- ue4m3 */

/* e4m3 (bias 7, 3 mantissa bits, subnormal step 2^-9, max 448, no inf). */
float arcq_ue4m3_decode(uint8_t code) {
  int e = (code >> 3) & 15, m = code & 7;
  float v;
  if (e == 15 && m == 7) return NAN;
  if (e == 0) v = ldexpf((float)m, -9);
  else v = ldexpf(1.0f + (float)m / 8.0f, e - 7);
  return (code & 0x80) ? -v : v;
}

/* non-negative float -> ue4m3 byte, RNE, saturating at 448 (0x7e). */
uint8_t arcq_ue4m3_encode(float x) {
  if (!(x == x)) return 0x7f;
  if (x <= 0.f) return 0;
  if (x >= 448.f) return 0x7e;
  int ex;
  (void)frexpf(x, &ex);        /* x = f * 2^ex, f in [0.5,1) */
  int e = ex - 1;              /* x = (1.xxx) * 2^e */
  if (e < -6) e = -6;          /* subnormal range shares the step of e=-6 */
  /* quantum = 2^(e-3); q = RNE(x / quantum) computed exactly */
  float q = ldexpf(x, 3 - e);  /* exact scaling */
  float r = nearbyintf(q);     /* default rounding mode: nearest even */
  int qi = (int)r;             /* in [0,16] */
  if (e == -6 && qi < 8) return (uint8_t)qi;         /* subnormal (or zero) */
  if (qi == 16) { qi = 8; e += 1; }
  if (e > 8) return 0x7e;
  uint8_t code = (uint8_t)(((e + 7) << 3) | (qi - 8));
  if (code > 0x7e) code = 0x7e;
  return code;
}

/* ------------------------------------------------------- scale-factor map */

/* Byte offset of the scale of (row r, scale column c) in the swizzled layout
 * the block-scaled GEMM consumes: 512-byte atoms of 128 rows x 4 columns,
 * column atoms fastest (kernels/include/reorder.cuh:118-123 through
 * kernels/src/reorder.cu:140-143). ncols = K_eff/16. */
int64_t arcq_sf_offset(int64_t r, int64_t c, int64_t ncols) {
  int64_t natoms = (ncols + 3) / 4;
  return ((r / 128) * natoms + c / 4) * 512 + (r % 32) * 16 + ((r / 32) % 4) * 4 + (c % 4);
}

/* Size the reference allocates (kernels/src/bindings.cpp:87,94). */
int64_t arcq_sf_bytes_reference(int64_t rows, int64_t k_eff) {
  return (rows / 128 + 1) * 128 * k_eff / 16;
}

/* Bytes the layout really spans for `rows` rows. */
int64_t arcq_sf_bytes_span(int64_t rows, int64_t k_eff) {
  int64_t ncols = k_eff / 16;
  return ((rows + 127) / 128) * ((ncols + 3) / 4) * 512;
}

/* ------------------------------------------------------------ quantizer */

static inline float clampf(float x, float lo, float hi) {
  float t = hi < x ? hi : x;       /* fpmin(b, x) then fpmax(a, .) as reorder.cu:33-37 */
  return lo > t ? lo : t;
}

#define ARCQ_FLAG_UNROUNDED_RESIDUAL 1  /* 32-wide kernels' quirk */
#define ARCQ_FLAG_TIE_LOW            2  /* fake path: ties to the more negative value */
#define ARCQ_FLAG_DIVIDE             4  /* fake path: x / s instead of x * fp32(1/s) */

/* e2m1 with the fake path's tie rule (model/quantize.py:14-22: argmin over the
 * ascending value list returns the first, i.e. more negative, of two equally
 * near candidates). */
static uint8_t e2m1_encode_tie_low(float x) {
  static const float mid[7] = {0.25f, 0.75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.0f};
  float a = fabsf(x);
  int neg = x < 0.f;
  uint8_t c = 0;
  for (int i = 0; i < 7; ++i) {
    /* positive: move up only when strictly above the midpoint;
     * negative: a tie moves to the larger magnitude (more negative value). */
    if (neg ? (a >= mid[i]) : (a > mid[i])) c = (uint8_t)(i + 1);
  }
  return (uint8_t)((neg && c) ? (8 | c) : c);
}

/* One 16-element group: codes[16] (4-bit each), *sf = ue4m3 byte.
 * If res != NULL it receives the fp32 residuals x - q*s (callers round them to
 * bf16 as reorder.cu:157-160 does).  ARCQ_FLAG_UNROUNDED_RESIDUAL selects the
 * 32-wide kernels' quirk (reorder.cu:474-477, down.cu:152-155): the residual is
 * formed with the fp32 scale before its ue4m3 rounding, in one fused
 * multiply-add (nvcc contracts a - b*c by default). */
static void quantize_group(const float* xr, uint8_t* codes, uint8_t* sf, float* res, int flags) {
  float maxv = 0.f;
  for (int i = 0; i < 16; ++i) {
    float a = fabsf(xr[i]);
    maxv = maxv > a ? maxv : a;     /* mymax keeps maxv on NaN, as reorder.cu:53,60 */
  }
  float scale = clampf(maxv / 6.0f, 0.001953125f, 448.0f);
  uint8_t s8 = arcq_ue4m3_encode(scale);
  float sdec = arcq_ue4m3_decode(s8);
  float r_scale = (float)(1.0 / (double)sdec);          /* reorder.cu:146 */
  *sf = s8;
  for (int i = 0; i < 16; ++i) {
    float x = xr[i];
    float t = (flags & ARCQ_FLAG_DIVIDE) ? (x / sdec) : (x * r_scale);
    float v = clampf(t, -6.0f, 6.0f);
    uint8_t c = (flags & ARCQ_FLAG_TIE_LOW) ? e2m1_encode_tie_low(v) : arcq_e2m1_encode(v);
    codes[i] = c;
    if (res) {
      float q = arcq_e2m1_decode(c);
      res[i] = (flags & ARCQ_FLAG_UNROUNDED_RESIDUAL) ? fmaf(-q, scale, x) : (x - q * sdec);
    }
  }
}

static inline void pack8(const uint8_t* codes, uint8_t* out) {
  for (int i = 0; i < 8; ++i) out[i] = (uint8_t)((codes[2 * i] & 15) | (codes[2 * i + 1] << 4));
}

/* Quantize one already gathered (and, for the fused op, normalised) row.
 * mode 16: one group per reference thread; critical group j (>= G0) lands at
 *          scale columns G0+2j', G0+2j'+1 and code bytes [8 main][8 residual].
 * mode 32: two groups per reference thread; a critical pair lands at columns
 *          p, p+1 (mains) p+2, p+3 (residuals) and bytes [8 m1][8 m2][8 r1][8 r2].
 * is_weight: the residual slots are byte copies of the main codes and scale. */
static void quantize_row(const uint16_t* xr, int64_t row, int KQ, int KE, int mode, int is_weight,
                         uint8_t* q_row, uint8_t* sf_base) {
  const int G = KQ / 16, GE = KE / 16, G0 = G - GE;
  const int64_t ncols = (KQ + KE) / 16;
  uint8_t codes[16], rcodes[16], sf, rsf = 0;
  float xf[16], res[16];
  for (int g = 0; g < G; ++g) {
    int critical = g >= G0;
    for (int i = 0; i < 16; ++i) xf[i] = bf16_to_f32(xr[16 * g + i]);
    quantize_group(xf, codes, &sf, (critical && !is_weight) ? res : NULL,
                   mode == 32 ? ARCQ_FLAG_UNROUNDED_RESIDUAL : 0);
    if (critical) {
      if (is_weight) { memcpy(rcodes, codes, 16); rsf = sf; }
      else {
        for (int i = 0; i < 16; ++i) res[i] = bf16_to_f32(f32_to_bf16(res[i]));   /* reorder.cu:157 */
        quantize_group(res, rcodes, &rsf, NULL, 0);
      }
    }
    int64_t col_m, col_r = 0, byte_m, byte_r = 0;
    if (!critical) { col_m = g; byte_m = 8 * (int64_t)g; }
    else if (mode == 16) {
      int j = g - G0;
      col_m = G0 + 2 * j; col_r = col_m + 1;
      byte_m = 8 * (int64_t)G0 + 16 * j; byte_r = byte_m + 8;
    } else {
      int j = g - G0, pair = j / 2, h = j & 1;
      col_m = G0 + 4 * pair + h; col_r = col_m + 2;
      byte_m = 8 * (int64_t)G0 + 32 * pair + 8 * h; byte_r = byte_m + 16;
    }
    pack8(codes, q_row + byte_m);
    sf_base[arcq_sf_offset(row, col_m, ncols)] = sf;
    if (critical) {
      pack8(rcodes, q_row + byte_r);
      sf_base[arcq_sf_offset(row, col_r, ncols)] = rsf;
    }
  }
}

/* Correctly rounded fp32 1/sqrt(v) for finite v > 0.  Candidate from double
 * arithmetic, then fixed up with exact integer comparisons of m^2*v against 1
 * at the two neighbouring rounding boundaries. */
static int boundary_below_target(double m, float v) {
  /* returns 1 if m < 1/sqrt(v)  <=>  m*m*v < 1, evaluated exactly */
  int em, ev;
  double fm = frexp(m, &em);             /* m = fm * 2^em, fm in [0.5,1) */
  float fv = frexpf(v, &ev);
  uint64_t Mm = (uint64_t)ldexp(fm, 26); /* m has <= 25 significant bits */
  uint64_t Mv = (uint64_t)ldexpf(fv, 24);
  /* m^2 v = Mm^2 * Mv * 2^(2*(em-26) + ev - 24) */
  unsigned __int128 p = (unsigned __int128)Mm * Mm * Mv;
  int sh = -(2 * (em - 26) + ev - 24);   /* compare p with 2^sh */
  if (sh < 0) return 0;
  if (sh >= 127) return 1;
  unsigned __int128 one = (unsigned __int128)1 << sh;
  return p < one;
}

float arcq_rsqrt_rn(float v) {
  float r = (float)(1.0 / sqrt((double)v));
  for (int it = 0; it < 4; ++it) {
    float up = nextafterf(r, INFINITY), dn = nextafterf(r, 0.f);
    double mid_up = ((double)r + (double)up) * 0.5;
    double mid_dn = ((double)r + (double)dn) * 0.5;
    if (boundary_below_target(mid_up, v)) { r = up; continue; }   /* target above upper boundary */
    if (!boundary_below_target(mid_dn, v)) {                      /* target at or below lower boundary */
      /* exactly on the boundary cannot happen for a non-square-free tie; move down */
      r = dn; continue;
    }
    break;
  }
  return r;
}

/* Sum of squares of one row in the reference's order (rmsnorm.cu:113-154):
 * bdx = KQ/16 threads, thread t adds elements 8t..8t+7 then 8(bdx+t)..+7
 * sequentially; shared-memory tree +256,+128 (guarded), +64,+32; then a
 * shuffle-down tree 16..1 whose lane 0 holds the total. */
static float rms_sum_squares(const uint16_t* x, int KQ) {
  int bdx = KQ / 16;
  int n = bdx < 512 ? 512 : bdx;
  float* s = (float*)calloc((size_t)n + 512, sizeof(float));
  for (int t = 0; t < bdx; ++t) {
    float acc = 0.f;
    for (int i = 0; i < 8; ++i) { float v = bf16_to_f32(x[8 * t + i]); acc = fmaf(v, v, acc); }
    for (int i = 0; i < 8; ++i) { float v = bf16_to_f32(x[8 * (bdx + t) + i]); acc = fmaf(v, v, acc); }
    s[t] = acc;
  }
  /* levels above 256 only exist for rows wider than the reference supports;
   * they extend the same pattern (guarded adds) upwards. */
  for (int lvl = 4096; lvl >= 512; lvl >>= 1)
    for (int t = 0; t < lvl && t < bdx; ++t) if (t + lvl < bdx) s[t] = s[t] + s[t + lvl];
  for (int t = 0; t < 256 && t < bdx; ++t) s[t] = s[t] + ((t + 256) < bdx ? s[t + 256] : 0.f);
  for (int t = 0; t < 128 && t < bdx; ++t) s[t] = s[t] + ((t + 128) < bdx ? s[t + 128] : 0.f);
  for (int t = 0; t < 64; ++t) s[t] = s[t] + s[t + 64];
  for (int t = 0; t < 32; ++t) s[t] = s[t] + s[t + 32];
  for (int sh = 16; sh > 0; sh >>= 1)
    for (int t = 0; t < sh; ++t) s[t] = s[t] + s[t + sh];
  float total = s[0];
  free(s);
  return total;
}

/* Activation path.  X: bf16 [M,KQ] row-major.  idx: int16 [KQ] or NULL
 * (identity / pre-gathered input, as down.cu).  gamma: bf16 [KQ] or NULL;
 * non-NULL selects the fused RMSNorm op (rmsnorm.cu).  QX: [M,(KQ+KE)/2],
 * SFX: swizzled scale bytes (only valid positions are written).
 * Returns 0, or -1 on a shape the layout cannot express. */
int arcq_oracle_quantize_x(const uint16_t* X, int64_t M, int KQ, const int16_t* idx, int KE, int mode,
                           const uint16_t* gamma, float eps, uint8_t* QX, uint8_t* SFX) {
  if (KQ % 16 || KE % 16 || KE > KQ || KE < 0 || (mode != 16 && mode != 32)) return -1;
  if (mode == 32 && (KQ % 32 || KE % 32)) return -1;
  if (gamma && KQ % 16) return -1;
  uint16_t* xr = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)KQ);
  const int64_t row_bytes = (KQ + KE) / 2;
  for (int64_t m = 0; m < M; ++m) {
    const uint16_t* x = X + m * (int64_t)KQ;
    if (gamma) {
      float ss = rms_sum_squares(x, KQ);
      float v = ss / (float)KQ + eps;
      float rstd = arcq_rsqrt_rn(v);
      for (int j = 0; j < KQ; ++j) {
        int c = idx ? (int)idx[j] : j;
        float t = bf16_to_f32(x[c]) * bf16_to_f32(gamma[c]);   /* exact in fp32 */
        xr[j] = f32_to_bf16(t * rstd);
      }
    } else {
      for (int j = 0; j < KQ; ++j) xr[j] = x[idx ? (int)idx[j] : j];
    }
    quantize_row(xr, m, KQ, KE, mode, 0, QX + m * row_bytes, SFX);
  }
  free(xr);
  return 0;
}

/* Weight path (reorder.cu:210-330, 563-696; down.cu:240-361). */
int arcq_oracle_quantize_w(const uint16_t* W, int64_t N, int KQ, const int16_t* idx, int KE, int mode,
                           uint8_t* QW, uint8_t* SFW) {
  if (KQ % 16 || KE % 16 || KE > KQ || KE < 0 || (mode != 16 && mode != 32)) return -1;
  if (mode == 32 && (KQ % 32 || KE % 32)) return -1;
  uint16_t* xr = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)KQ);
  const int64_t row_bytes = (KQ + KE) / 2;
  for (int64_t n = 0; n < N; ++n) {
    const uint16_t* w = W + n * (int64_t)KQ;
    for (int j = 0; j < KQ; ++j) xr[j] = w[idx ? (int)idx[j] : j];
    quantize_row(xr, n, KQ, KE, mode, 1, QW + n * row_bytes, SFW);
  }
  free(xr);
  return 0;
}

/* Dequantise packed codes + swizzled scales to fp32 [rows, K_eff]. */
void arcq_oracle_dequant(const uint8_t* Q, const uint8_t* SF, int64_t rows, int k_eff, float* out) {
  const int64_t ncols = k_eff / 16;
  for (int64_t r = 0; r < rows; ++r)
    for (int k = 0; k < k_eff; ++k) {
      uint8_t b = Q[r * (k_eff / 2) + k / 2];
      uint8_t c = (k & 1) ? (b >> 4) : (b & 15);
      float s = arcq_ue4m3_decode(SF[arcq_sf_offset(r, k / 16, ncols)]);
      out[r * (int64_t)k_eff + k] = arcq_e2m1_decode(c) * s;
    }
}

/* C[m,n] = alpha * sum_k deq(A)[m,k] * deq(B)[n,k]  (nvfp4.cu:35-132), with the
 * sum carried in double so that the oracle itself adds no fp32 ordering noise.
 * Small shapes only. */
void arcq_oracle_gemm(const uint8_t* A, const uint8_t* SFA, const uint8_t* B, const uint8_t* SFB,
                      int64_t M, int64_t N, int k_eff, float alpha, float* C) {
  float* a = (float*)malloc(sizeof(float) * (size_t)M * k_eff);
  float* b = (float*)malloc(sizeof(float) * (size_t)N * k_eff);
  arcq_oracle_dequant(A, SFA, M, k_eff, a);
  arcq_oracle_dequant(B, SFB, N, k_eff, b);
  for (int64_t m = 0; m < M; ++m)
    for (int64_t n = 0; n < N; ++n) {
      double acc = 0.0;
      const float* pa = a + m * (int64_t)k_eff;
      const float* pb = b + n * (int64_t)k_eff;
      for (int k = 0; k < k_eff; ++k) acc += (double)pa[k] * (double)pb[k];
      C[m * N + n] = (float)((double)alpha * acc);
    }
  free(a);
  free(b);
}

/* Bridge to the reference's torch fake-quant path (model/quantize.py:145-172,
 * 314-343): same gather, grouping, block scales and residual structure as
 * above, but with that path's arithmetic knobs (division by the block scale,
 * ties towards the more negative value, fp32 residuals that are not rounded to
 * bf16) and its output form: dequantised values [M, KQ+KE], main block first,
 * the KE residual columns appended.  Equal to the fake path wherever block
 * scales stay in the normal ue4m3 range (>= 2^-6). */
int arcq_oracle_fake_values(const uint16_t* X, int64_t M, int KQ, const int16_t* idx, int KE, float* out) {
  if (KQ % 16 || KE % 16 || KE > KQ || KE < 0) return -1;
  const int G = KQ / 16, G0 = (KQ - KE) / 16;
  const int flags = ARCQ_FLAG_TIE_LOW | ARCQ_FLAG_DIVIDE;
  uint8_t codes[16], sf;
  float xf[16], res[16];
  for (int64_t m = 0; m < M; ++m) {
    const uint16_t* x = X + m * (int64_t)KQ;
    float* o = out + m * (int64_t)(KQ + KE);
    for (int g = 0; g < G; ++g) {
      for (int i = 0; i < 16; ++i) xf[i] = bf16_to_f32(x[idx ? (int)idx[16 * g + i] : 16 * g + i]);
      quantize_group(xf, codes, &sf, res, flags);
      float s = arcq_ue4m3_decode(sf);
      for (int i = 0; i < 16; ++i) o[16 * g + i] = arcq_e2m1_decode(codes[i]) * s;
      if (g >= G0) {
        quantize_group(res, codes, &sf, NULL, flags);
        s = arcq_ue4m3_decode(sf);
        for (int i = 0; i < 16; ++i) o[KQ + 16 * (g - G0) + i] = arcq_e2m1_decode(codes[i]) * s;
      }
    }
  }
  return 0;
}
