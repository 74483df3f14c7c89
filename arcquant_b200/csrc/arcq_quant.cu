// ARC-NVFP4 quantizer for sm_100a: (RMSNorm ->) channel gather -> NVFP4 block quantization ->
// re-quantized residuals of the critical channels, written as packed e2m1 codes plus ue4m3 block
// scales in the 128x4 atom layout of block-scaled tensor-core GEMMs.
//
// One kernel serves the reference's reorder_x / reorder32_x / down32_x / rmsnorm_x and the three
// weight kernels (kernels/src/reorder.cu, down.cu, rmsnorm.cu of ARCQuant); the arithmetic is theirs,
// the organisation is not:
//
//  * persistent CTAs walk over PAIRS of rows.  A pair is staged in shared memory interleaved at
//    2-byte granularity - word c = (row0[c], row1[c]) - so the random channel gather costs one
//    32-bit shared load per TWO elements, and everything downstream works on both rows at once:
//    packed 16-bit max for the block amax, packed fp32x2 multiplies (FMUL2) for the scaling,
//    cvt.rn.bf16x2 for the RMSNorm rounding;
//  * the next pair is in flight in registers (128-bit coalesced streaming loads) while the current
//    one is quantized (double buffer); 16-byte chunks are stored XOR-swizzled so the 128-bit shared
//    stores are conflict free;
//  * the channel order becomes, once per CTA, a shared table of (swizzled) byte offsets read back
//    with 128-bit loads - no per-row index traffic;
//  * block scale: ue4m3(clamp(amax/6)) and its fp32 reciprocal come from two tiny tables indexed by
//    the bf16 bits of the amax (built in the prologue with the IEEE slow path, so both paths agree
//    by construction); the slow path still serves subnormal / saturated scales and critical groups;
//  * conversions use the hardware cvt.rn.satfinite.{e2m1x2,e4m3x2}.f32 (round to nearest even,
//    saturating), eight codes are packed per 32-bit word and stored 8 bytes per group;
//  * RMSNorm partial sums are taken from the registers of the streaming load, in the reference's
//    accumulation order, and the reciprocal root is the correctly rounded one.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>


#include "arcq_internal.h"

namespace arcq {
namespace {

struct QuantParams {
  const uint16_t* x;      // bf16 bits [rows, KQ]
  const uint16_t* gamma;  // bf16 bits [KQ] (RMSNorm gain) or nullptr
  const int16_t* idx;     // [KQ] or nullptr (identity)
  uint8_t* q;             // [rows, (KQ+KE)/2]
  uint8_t* sf;            // swizzled ue4m3 scales
  long long rows;
  long long npairs;
  int KQ, KE;
  int G, G0;      // groups per row, groups without residual
  int natoms;     // ceil(((KQ+KE)/16)/4): 512-byte scale atoms per 128-row tile
  int nchunks;    // KQ/8: 16-byte chunks per row
  int mode;       // 16 or 32 (placement of critical groups, residual flavour)
  int is_weight;  // residual slot = copy of the main codes
  float eps;
  const float* scale;   // warp-specialised plain kernel only: x is divided by *scale (device) first, or nullptr
  // Grouped rows (warp-specialised kernel only): the rows form `ngroups` runs, run e starting at output
  // row groups[e] with groups[ngroups + e] rows (device memory, so the host never learns the sizes);
  // run e uses the channel order idx + e*KQ and the scale scale[e].  row_map (or nullptr): input row of
  // every output row.
  const int* groups;
  int ngroups;
  const int* row_map;
};

__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// (lo, hi) fp32 -> packed bf16x2, round to nearest even.
__device__ __forceinline__ uint32_t pack_bf16x2_rn(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// a * b + c with a, b bf16 and c, result fp32 (one rounding): the mixed-precision FMA of sm_100.
// With c = -0.0f it is the exact product a * b, signed zeros included.
__device__ __forceinline__ float fma_bf16(uint16_t a, uint16_t b, float c) {
  float d;
  asm("fma.rn.f32.bf16 %0, %1, %2, %3;" : "=f"(d) : "h"(a), "h"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint16_t half_lo(uint32_t w) { return (uint16_t)(w & 0xffffu); }
__device__ __forceinline__ uint16_t half_hi(uint32_t w) { return (uint16_t)(w >> 16); }
// per-halfword unsigned max
__device__ __forceinline__ uint32_t max_u16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("max.u16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// float -> ue4m3 byte: round to nearest even, saturating at 448 (input is in [2^-9, 448]).
__device__ __forceinline__ uint32_t ue4m3_encode(float s) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.0f), "f"(s));
  return (uint32_t)r & 0xffu;
}
__device__ __forceinline__ float ue4m3_decode(uint32_t c) {
  uint32_t e = (c >> 3) & 15u, m = c & 7u;
  return e ? __uint_as_float(((e + 120u) << 23) | (m << 20)) : (float)m * 0.001953125f;
}

// Eight floats -> eight e2m1 codes in one word, element 0 in the lowest nibble
// (cvt.e2m1x2 puts its first source in the high nibble).
__device__ __forceinline__ uint32_t e2m1x8(float a0, float a1, float a2, float a3, float a4, float a5,
                                           float a6, float a7) {
  uint32_t out;
  asm("{\n"
      ".reg .b8 b0, b1, b2, b3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n"
      "mov.b32 %0, {b0, b1, b2, b3};\n"
      "}"
      : "=r"(out)
      : "f"(a0), "f"(a1), "f"(a2), "f"(a3), "f"(a4), "f"(a5), "f"(a6), "f"(a7));
  return out;
}

// One byte of two e2m1 codes -> their values (exact): x = low nibble, y = high nibble.
__device__ __forceinline__ float2 e2m1x2_decode(uint32_t byte) {
  uint32_t h2;
  const uint16_t b16 = (uint16_t)(byte & 0xffu);
  asm("{\n.reg .b8 t;\nmov.b16 {t, _}, %1;\ncvt.rn.f16x2.e2m1x2 %0, t;\n}" : "=r"(h2) : "h"(b16));
  return __half22float2(*reinterpret_cast<__half2*>(&h2));
}

struct GroupScale {
  uint32_t byte;  // ue4m3 code
  float dec;      // its value
  float raw;      // clamp(amax/6, 2^-9, 448) before rounding
  float rcp;      // fp32(1/dec)
};

// IEEE path: every case, including subnormal and saturated scales.
__device__ __noinline__ GroupScale make_scale_slow(float amax) {
  GroupScale s;
  float t = __fdiv_rn(amax, 6.0f);
  t = fminf(t, 448.0f);
  s.raw = fmaxf(t, 0.001953125f);
  s.byte = ue4m3_encode(s.raw);
  s.dec = ue4m3_decode(s.byte);
  s.rcp = __frcp_rn(s.dec);
  return s;
}

// Table path.  ab = bf16 bits of the amax (15 bits).  For a normal result the scale code is
// T[mantissa] shifted by the exponent, and 1/scale is RB[code mantissa] shifted likewise (powers
// of two do not change any rounding).  Anything outside the normal, unsaturated range takes the
// IEEE path.
struct ScaleLut {
  const uint8_t* T;     // [128] code of amax = 1.m7 (exponent field 127)
  const uint32_t* RB;   // [8]   fp32 bits of 1/(1+m3/8), exponent pre-biased by 7
};
// Both rows of a pair: one (rarely taken) branch covers the IEEE fallback of either row.
__device__ __forceinline__ void scale_of_pair(uint32_t m, const ScaleLut& lut, uint32_t& c0, uint32_t& c1, float& r0,
                                              float& r1) {
  const uint32_t a0 = m & 0xffffu, a1 = m >> 16;
  const int s0 = (int)lut.T[a0 & 127u] + (int)((a0 >> 7) << 3) - 1016;
  const int s1 = (int)lut.T[a1 & 127u] + (int)((a1 >> 7) << 3) - 1016;
  c0 = (uint32_t)s0;
  c1 = (uint32_t)s1;
  r0 = __uint_as_float(lut.RB[s0 & 7] - ((uint32_t)(s0 >> 3) << 23));
  r1 = __uint_as_float(lut.RB[s1 & 7] - ((uint32_t)(s1 >> 3) << 23));
  // (unsigned)(s - 8) > 118  <=>  s < 8 or s > 126
  if (__builtin_expect(((uint32_t)(s0 - 8) > 118u) | ((uint32_t)(s1 - 8) > 118u), 0)) {
    const GroupScale g0 = make_scale_slow(__uint_as_float(a0 << 16));
    const GroupScale g1 = make_scale_slow(__uint_as_float(a1 << 16));
    c0 = g0.byte; r0 = g0.rcp;
    c1 = g1.byte; r1 = g1.rcp;
  }
}

__device__ __forceinline__ size_t sf_row_base(long long r, int natoms) {
  return ((size_t)(r >> 7) * (size_t)natoms) * 512 + (size_t)(r & 31) * 16 + (size_t)((r >> 5) & 3) * 4;
}
__device__ __forceinline__ size_t sf_col(int c) { return (size_t)(c >> 2) * 512 + (size_t)(c & 3); }

// Where a critical group's main / residual codes and scales go.
struct Slot {
  int byte_main, col_main, byte_res, col_res;
};
__device__ __forceinline__ Slot slot_of(int g, int G0, int mode) {
  Slot s;
  if (mode == 32) {
    int j = g - G0, pair = j >> 1, h = j & 1;
    s.col_main = G0 + 4 * pair + h; s.col_res = s.col_main + 2;
    s.byte_main = 8 * G0 + 32 * pair + 8 * h; s.byte_res = s.byte_main + 16;
  } else {
    int j = g - G0;
    s.col_main = G0 + 2 * j; s.col_res = s.col_main + 1;
    s.byte_main = 8 * G0 + 16 * j; s.byte_res = s.byte_main + 8;
  }
  return s;
}

// Both rows of a pair at once: w[i] = (row0 value, row1 value) as bf16x2.  Multiplies every value by
// its row's reciprocal scale (one FMUL2 per word) and converts to e2m1, eight codes per word.
__device__ __forceinline__ void encode_pair(const uint32_t (&w)[16], float rcp0, float rcp1, uint2& c0, uint2& c1) {
  const float2 r = make_float2(rcp0, rcp1);
  uint32_t o0[2], o1[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {   // eight words (one output word per row) at a time: fewer values live
    float2 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __fmul2_rn(make_float2(bf16lo(w[8 * h + i]), bf16hi(w[8 * h + i])), r);
    o0[h] = e2m1x8(v[0].x, v[1].x, v[2].x, v[3].x, v[4].x, v[5].x, v[6].x, v[7].x);
    o1[h] = e2m1x8(v[0].y, v[1].y, v[2].y, v[3].y, v[4].y, v[5].y, v[6].y, v[7].y);
  }
  c0 = make_uint2(o0[0], o0[1]);
  c1 = make_uint2(o1[0], o1[1]);
}

// Packed |.| maximum of the sixteen words: low half = row0 amax bits, high half = row1.
__device__ __forceinline__ uint32_t amax_pair(const uint32_t (&w)[16]) {
  uint32_t m = 0;
#pragma unroll
  for (int i = 0; i < 16; ++i) m = max_u16x2(m, w[i] & 0x7fff7fffu);
  return m;
}

// The same with the packed bf16 maximum of magnitudes (one instruction per word).  A NaN input gives
// the canonical NaN 0x7fff, which the caller clamps like the integer maximum of a NaN pattern.
__device__ __forceinline__ uint32_t amax_pair_h(const uint32_t (&w)[16]) {
  uint32_t m[4] = {w[0], w[1], w[2], w[3]};
#pragma unroll
  for (int i = 4; i < 16; ++i)
    asm("max.NaN.xorsign.abs.bf16x2 %0, %0, %1;" : "+r"(m[i & 3]) : "r"(w[i]));
  asm("max.NaN.xorsign.abs.bf16x2 %0, %0, %1;" : "+r"(m[0]) : "r"(m[1]));
  asm("max.NaN.xorsign.abs.bf16x2 %0, %0, %1;" : "+r"(m[2]) : "r"(m[3]));
  asm("max.NaN.xorsign.abs.bf16x2 %0, %0, %1;" : "+r"(m[0]) : "r"(m[2]));
  return m[0] & 0x7fff7fffu;
}

// Residuals of a critical group, both rows: w[i] <- bf16(x - q*s) per half.
// mode 16 subtracts against the rounded scale (q*s is exact in fp32, so the fused form is the same
// number); mode 32 against the un-rounded one, fused, as the 32-wide reference kernels compile.
__device__ __forceinline__ void residual_pair(uint32_t (&w)[16], uint2 c0, uint2 c1, float s0, float s1) {
#pragma unroll
  for (int i = 0; i < 16; i += 2) {
    const uint32_t b0 = ((i < 8 ? c0.x : c0.y) >> (4 * (i & 7))) & 0xffu;
    const uint32_t b1 = ((i < 8 ? c1.x : c1.y) >> (4 * (i & 7))) & 0xffu;
    const float2 q0 = e2m1x2_decode(b0), q1 = e2m1x2_decode(b1);
    float d00 = __fmaf_rn(-q0.x, s0, bf16lo(w[i])), d01 = __fmaf_rn(-q0.y, s0, bf16lo(w[i + 1]));
    float d10 = __fmaf_rn(-q1.x, s1, bf16hi(w[i])), d11 = __fmaf_rn(-q1.y, s1, bf16hi(w[i + 1]));
    w[i] = pack_bf16x2_rn(d00, d10);
    w[i + 1] = pack_bf16x2_rn(d01, d11);
  }
}

// Quantize one group of both rows and store codes + scales.  Every lane runs the same main path
// (table scale, FMUL2 + cvt); only the residual of a critical group is a divergent extra.
// Row 1 is stored before row 0: for the odd last row of the input the caller aliases row 1's
// output pointers to row 0's, and the later store wins.
__device__ __forceinline__ void quantize_group_pair(uint32_t (&w)[16], int g, const QuantParams& p,
                                                    const ScaleLut& lut, uint8_t* q0, uint8_t* q1, uint8_t* sf0,
                                                    uint8_t* sf1) {
  const uint32_t m = amax_pair(w);
  uint32_t s0, s1;
  float r0, r1;
  scale_of_pair(m, lut, s0, s1, r0, r1);
  uint2 c0, c1;
  encode_pair(w, r0, r1, c0, c1);
  const bool critical = g >= p.G0;
  int byte_main = 8 * g, col_main = g;
  Slot sl;
  if (critical) {
    sl = slot_of(g, p.G0, p.mode);
    byte_main = sl.byte_main;
    col_main = sl.col_main;
  }
  const size_t cm = sf_col(col_main);
  *reinterpret_cast<uint2*>(q1 + byte_main) = c1;
  sf1[cm] = (uint8_t)s1;
  *reinterpret_cast<uint2*>(q0 + byte_main) = c0;
  sf0[cm] = (uint8_t)s0;
  if (!critical) return;

  // critical group: the re-quantized residual (or, for weights, a copy of the main codes)
  uint2 e0 = c0, e1 = c1;
  uint32_t t0 = s0, t1 = s1;
  if (!p.is_weight) {
    float d0 = ue4m3_decode(s0), d1 = ue4m3_decode(s1);
    if (p.mode == 32) {   // against the un-rounded fp32 scale
      d0 = make_scale_slow(__uint_as_float((m & 0xffffu) << 16)).raw;
      d1 = make_scale_slow(__uint_as_float((m >> 16) << 16)).raw;
    }
    residual_pair(w, c0, c1, d0, d1);
    const uint32_t rm = amax_pair(w);
    float h0, h1;
    scale_of_pair(rm, lut, t0, t1, h0, h1);
    encode_pair(w, h0, h1, e0, e1);
  }
  const size_t cr = sf_col(sl.col_res);
  *reinterpret_cast<uint2*>(q1 + sl.byte_res) = e1;
  sf1[cr] = (uint8_t)t1;
  *reinterpret_cast<uint2*>(q0 + sl.byte_res) = e0;
  sf0[cr] = (uint8_t)t0;
}

// Sum-of-squares tree of one row in the reference's order (rmsnorm.cu:131-154 of ARCQuant), done by
// one warp: lane l owns the partials of reference threads l, l+32, ... (zero where none exists).
__device__ __forceinline__ float rms_tree(const float* ps, int nt, int lane) {
  // slot t = lane + 32k, k < 16; the tree adds slots 256, 128, 64 and 32 apart, in that order
  auto slot = [&](int k) { const int t = lane + 32 * k; return t < nt ? ps[t] : 0.f; };
  auto b = [&](int k) { return __fadd_rn(slot(k), slot(k + 8)); };       // +256
  auto c = [&](int k) { return __fadd_rn(b(k), b(k + 4)); };             // +128
  const float d0 = __fadd_rn(c(0), c(2)), d1 = __fadd_rn(c(1), c(3));    // +64
  float s = __fadd_rn(d0, d1);                                           // +32
#pragma unroll
  for (int d2 = 16; d2 > 0; d2 >>= 1) s = __fadd_rn(s, __shfl_down_sync(0xffffffffu, s, d2));
  return s;  // valid in lane 0
}

// Physical position (in 16-byte units) of logical 16-byte unit j of an interleaved row pair.
__device__ __forceinline__ uint32_t swz16(uint32_t j) { return j ^ ((j >> 3) & 1u); }
// Byte offset of channel ch's (row0,row1) word.
__device__ __forceinline__ uint32_t word_offset(uint32_t ch) { return (swz16(ch >> 2) << 4) | ((ch & 3u) << 2); }

// CPT: 16-byte chunks per thread per row; NBUF: shared buffers (2 = the next unit streams in while
// the current one is quantized); PAIRS: row pairs per loop iteration ("unit") - two pairs halve the
// per-row cost of the table reads, the barrier and the loop bookkeeping and double the independent
// shared loads in flight; RMS: fused RMSNorm; RAWIDX: the offset table holds 16-bit channel numbers
// (rows wider than 16384 channels) instead of 32-bit byte offsets.  MAXT / MINB: launch bounds.
template <int CPT, int NBUF, int PAIRS, bool RMS, bool RAWIDX, int MAXT, int MINB>
__global__ void __launch_bounds__(MAXT, MINB) arcq_quantize_kernel(const QuantParams p) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int tid = threadIdx.x, nt = blockDim.x;
  const int KQ = p.KQ, G = p.G, nchunks = p.nchunks;
  const long long rows = p.rows, npairs = p.npairs;

  // shared layout: [scale tables 160 B][offsets][gain (RMS)][partial sums, rstd (RMS)][row-pair buffers]
  uint8_t* lutT = smem;
  uint32_t* lutRB = reinterpret_cast<uint32_t*>(smem + 128);
  size_t cursor = 160;
  uint32_t* offs32 = reinterpret_cast<uint32_t*>(smem + cursor);
  uint16_t* offs16 = reinterpret_cast<uint16_t*>(smem + cursor);
  cursor += ((size_t)KQ * (RAWIDX ? 2 : 4) + 15) & ~(size_t)15;
  float* gperm = reinterpret_cast<float*>(smem + cursor);
  float* psum = nullptr;
  float* rstd_s = nullptr;
  if (RMS) {
    cursor += (size_t)KQ * 4;
    psum = reinterpret_cast<float*>(smem + cursor);
    cursor += (size_t)2 * PAIRS * nt * sizeof(float);
    rstd_s = reinterpret_cast<float*>(smem + cursor);
    cursor += 16;
  }
  uint32_t* bufs = reinterpret_cast<uint32_t*>(smem + cursor);   // [NBUF][PAIRS][KQ] words

  for (int j = tid; j < 128; j += nt)
    lutT[j] = (uint8_t)make_scale_slow(__uint_as_float(((127u << 7) | (uint32_t)j) << 16)).byte;
  if (tid < 8)
    lutRB[tid] = tid ? (__float_as_uint(__frcp_rn(1.0f + 0.125f * (float)tid)) + (7u << 23)) : (134u << 23);
  // Tables are laid out [vector v][group g][4]: consecutive lanes (groups) read consecutive 16 bytes,
  // so every 128-bit table load is conflict free.
  for (int j = tid; j < KQ; j += nt) {
    int c = p.idx ? (int)p.idx[j] : j;
    const int g = j >> 4, i = j & 15;
    const int slot = (((i >> 2) * G + g) << 2) | (i & 3);
    if (RAWIDX) offs16[j] = (uint16_t)c; else offs32[slot] = word_offset((uint32_t)c);
    if (RMS) gperm[slot] = __uint_as_float((uint32_t)p.gamma[c] << 16);
  }
  const ScaleLut lut{lutT, lutRB};

  uint4 ra[PAIRS][CPT], rb[PAIRS][CPT];

  auto load_unit = [&](long long unit) {
#pragma unroll
    for (int u = 0; u < PAIRS; ++u) {
      const long long r0 = 2 * (unit * PAIRS + u);
      const bool has0 = r0 < rows, has1 = (r0 + 1) < rows;
      const uint4* x0 = reinterpret_cast<const uint4*>(p.x + r0 * (long long)KQ);
      const uint4* x1 = reinterpret_cast<const uint4*>(p.x + (r0 + 1) * (long long)KQ);
#pragma unroll
      for (int j = 0; j < CPT; ++j) {
        int c = tid + j * nt;
        if (c < nchunks) {
          ra[u][j] = has0 ? ldg_stream(x0 + c) : make_uint4(0, 0, 0, 0);
          rb[u][j] = has1 ? ldg_stream(x1 + c) : make_uint4(0, 0, 0, 0);
        }
      }
    }
  };

  auto store_unit = [&](uint32_t* buf) {
#pragma unroll
    for (int u = 0; u < PAIRS; ++u) {
      float2 ss = make_float2(0.f, 0.f);
      uint4* b4 = reinterpret_cast<uint4*>(buf + (size_t)u * KQ);
#pragma unroll
      for (int j = 0; j < CPT; ++j) {
        int c = tid + j * nt;
        if (c < nchunks) {
          const uint4 a = ra[u][j], b = rb[u][j];
          uint4 lo, hi;  // words of channels 8c..8c+3 and 8c+4..8c+7: (row0[ch], row1[ch]) per word
          lo.x = __byte_perm(a.x, b.x, 0x5410); lo.y = __byte_perm(a.x, b.x, 0x7632);
          lo.z = __byte_perm(a.y, b.y, 0x5410); lo.w = __byte_perm(a.y, b.y, 0x7632);
          hi.x = __byte_perm(a.z, b.z, 0x5410); hi.y = __byte_perm(a.z, b.z, 0x7632);
          hi.z = __byte_perm(a.w, b.w, 0x5410); hi.w = __byte_perm(a.w, b.w, 0x7632);
          // XOR-swizzled 16-byte units: the eight lanes of a 128-bit store wavefront hit distinct banks
          b4[swz16(2u * c)] = lo;
          b4[swz16(2u * c + 1u)] = hi;
          if (RMS) {
            // reference thread t adds chunk t then chunk t+KQ/16, eight elements each, in order;
            // the two rows ride in the two lanes of a packed FMA
            const uint32_t ws[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float2 v = make_float2(bf16lo(ws[i]), bf16hi(ws[i]));
              ss = __ffma2_rn(v, v, ss);
            }
          }
        }
      }
      if (RMS) {
        psum[(2 * u) * nt + tid] = ss.x;
        psum[(2 * u + 1) * nt + tid] = ss.y;
      }
    }
  };

  // The register prefetch above is scheduled late by the assembler (it holds 16+ registers), so its
  // latency is partly exposed; pulling the rows of the unit after next into L2 ahead of time turns
  // that exposed latency from an HBM access into an L2 hit.
  auto prefetch_unit_l2 = [&](long long unit) {
    if (tid < 2 * PAIRS) {
      const long long r = 2 * unit * PAIRS + tid;
      if (r < rows)
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.x + r * (long long)KQ), "r"(KQ * 2)
                     : "memory");
    }
  };

  const long long nunits = (npairs + PAIRS - 1) / PAIRS;
  long long unit = blockIdx.x;
  if (unit < nunits) { load_unit(unit); store_unit(bufs); }
  if (unit + gridDim.x < nunits) prefetch_unit_l2(unit + gridDim.x);
  __syncthreads();

  int cur = 0;
  const size_t row_bytes = (size_t)(KQ + p.KE) / 2;
  const size_t buf_words = (size_t)PAIRS * KQ;
  for (; unit < nunits; unit += gridDim.x) {
    const long long nxt = unit + gridDim.x;
    const bool more = nxt < nunits;
    if (NBUF == 2 && more) load_unit(nxt);
    if (nxt + gridDim.x < nunits) prefetch_unit_l2(nxt + gridDim.x);

    float2 rstd[PAIRS];
    if (RMS) {
      const int warp = tid >> 5, lane = tid & 31;
      if (warp < 2 * PAIRS) {
        float ss = rms_tree(psum + warp * nt, nt, lane);
        if (lane == 0) rstd_s[warp] = __frsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)KQ), p.eps));
      }
      __syncthreads();
#pragma unroll
      for (int u = 0; u < PAIRS; ++u) rstd[u] = make_float2(rstd_s[2 * u], rstd_s[2 * u + 1]);
    }

    const uint8_t* buf = reinterpret_cast<const uint8_t*>(bufs + (size_t)cur * buf_words);
    uint8_t *q0[PAIRS], *q1[PAIRS], *sf0[PAIRS], *sf1[PAIRS];
    bool live[PAIRS];
#pragma unroll
    for (int u = 0; u < PAIRS; ++u) {
      const long long r0 = 2 * (unit * PAIRS + u), r1 = r0 + 1;
      live[u] = r0 < rows;
      const bool has1 = r1 < rows;
      q0[u] = p.q + (size_t)r0 * row_bytes;
      q1[u] = has1 ? q0[u] + row_bytes : q0[u];          // odd last row: alias, row 0 is stored last
      sf0[u] = p.sf + sf_row_base(r0, p.natoms);
      sf1[u] = has1 ? p.sf + sf_row_base(r1, p.natoms) : sf0[u];
    }

    for (int g = tid; g < G; g += nt) {
      uint32_t w[PAIRS][16];
      if (RAWIDX) {
        const uint4* op = reinterpret_cast<const uint4*>(offs16 + 16 * g);
        const uint4 o0 = op[0], o1 = op[1];
        const uint32_t ow[8] = {o0.x, o0.y, o0.z, o0.w, o1.x, o1.y, o1.z, o1.w};
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const uint32_t ch = (i & 1) ? (ow[i >> 1] >> 16) : (ow[i >> 1] & 0xffffu);
          const uint32_t o = word_offset(ch);
#pragma unroll
          for (int u = 0; u < PAIRS; ++u)
            w[u][i] = *reinterpret_cast<const uint32_t*>(buf + (size_t)u * KQ * 4 + o);
        }
      } else {
        const uint4* op = reinterpret_cast<const uint4*>(offs32) + g;
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const uint4 o = op[v * G];
#pragma unroll
          for (int u = 0; u < PAIRS; ++u) {
            const uint8_t* bu = buf + (size_t)u * KQ * 4;
            w[u][4 * v + 0] = *reinterpret_cast<const uint32_t*>(bu + o.x);
            w[u][4 * v + 1] = *reinterpret_cast<const uint32_t*>(bu + o.y);
            w[u][4 * v + 2] = *reinterpret_cast<const uint32_t*>(bu + o.z);
            w[u][4 * v + 3] = *reinterpret_cast<const uint32_t*>(bu + o.w);
          }
        }
      }
      if (RMS) {
        const float4* gp = reinterpret_cast<const float4*>(gperm) + g;
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const float4 gm = gp[v * G];
          const float gs[4] = {gm.x, gm.y, gm.z, gm.w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int i = 4 * v + k;
#pragma unroll
            for (int u = 0; u < PAIRS; ++u) {
              // bf16 x bf16 is exact in fp32; then one rounding by rstd (both rows in one FMUL2), one to bf16
              const float2 t = make_float2(__fmul_rn(bf16lo(w[u][i]), gs[k]), __fmul_rn(bf16hi(w[u][i]), gs[k]));
              const float2 n = __fmul2_rn(t, rstd[u]);
              w[u][i] = pack_bf16x2_rn(n.x, n.y);
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < PAIRS; ++u)
        if (live[u]) quantize_group_pair(w[u], g, p, lut, q0[u], q1[u], sf0[u], sf1[u]);
    }

    if (NBUF == 2) {
      if (more) store_unit(bufs + (size_t)(cur ^ 1) * buf_words);
      __syncthreads();
      cur ^= 1;
    } else {
      __syncthreads();
      if (more) { load_unit(nxt); store_unit(bufs); }
      __syncthreads();
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Warp-specialised variant (rows of 1024..8192 channels, the hidden sizes of decoder layers).
//
// Producer warps stream row pairs from global memory, (RMSNorm them,) interleave them and fill a ring
// of shared stages; consumer warps gather their groups from a full stage, release it as soon as the
// gather has landed in registers, and quantize.  Stages are handed over with mbarriers, so there is
// no CTA-wide barrier in the loop and the warp that carries the critical (residual) groups - a
// different warp for every row pair - does not hold the others back.  Producers keep the next pair in
// flight in registers while they fill the current one.
//
// Block scales are computed without tables or branches: amax/6 by a multiply and one FMA correction
// (exact for every bf16 amax), the ue4m3 code of both rows by one packed conversion, and 1/scale by
// the approximate reciprocal plus one Newton step (exact here: a scale is k*2^e with k <= 15, so its
// reciprocal lies far from every fp32 rounding boundary).

__device__ int g_quant_error = 0;   // sticky until polled
constexpr unsigned long long QUANT_WAIT_LIMIT_NS = 2000000000ull;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false if this wait (or another warp's) gave up; the CTA then winds down.  The clock is
// first read after 64 failed polls, so a wait of ordinary length never touches it.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long t0 = 0;
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 63u) == 0) {
      if (*abort_flag) return false;
      unsigned long long t1;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
      if (t0 == 0) t0 = t1;
      if (t1 - t0 > QUANT_WAIT_LIMIT_NS) {
        *abort_flag = 1;
        atomicExch(&g_quant_error, ARCQ_ERR_TIMEOUT);
        return false;
      }
    }
  }
}
// Named barrier over `nthreads` threads that also ORs a flag across them.
__device__ __forceinline__ bool named_barrier_or(int id, int nthreads, bool flag) {
  uint32_t out;
  asm volatile(
      "{\n.reg .pred p, q;\n"
      "setp.ne.u32 q, %3, 0;\n"
      "bar.red.or.pred p, %1, %2, q;\n"
      "selp.u32 %0, 1, 0, p;\n}"
      : "=r"(out)
      : "r"(id), "r"(nthreads), "r"((uint32_t)flag)
      : "memory");
  return out != 0;
}

__device__ __forceinline__ uint32_t min_u16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("min.u16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// Scales of both rows from the packed amax bits (low half row 0, high half row 1).
// codes = ue4m3(row0) | ue4m3(row1) << 8; dec = their values; rcp = fp32(1/dec).
__device__ __forceinline__ void scale_of_pair_fma(uint32_t m, uint32_t& codes, float2& dec, float2& rcp) {
  m = min_u16x2(m, 0x7f7f7f7fu);                       // inf/NaN amax -> largest finite (saturates to 448)
  const float2 a = make_float2(bf16lo(m), bf16hi(m));
  const float sixth = 0.16666667163372039794921875f;   // fp32(1/6)
  const float2 c = make_float2(sixth, sixth);
  const float2 q = __fmul2_rn(a, c);
  const float2 r = __ffma2_rn(make_float2(-6.0f, -6.0f), q, a);
  float2 t = __ffma2_rn(r, c, q);                      // = fp32(amax / 6), correctly rounded
  t.x = fmaxf(t.x, 0.001953125f);
  t.y = fmaxf(t.y, 0.001953125f);                      // values above 448 saturate in the conversion
  uint16_t c2;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(c2) : "f"(t.y), "f"(t.x));
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(c2));
  dec = __half22float2(*reinterpret_cast<__half2*>(&h2));
  float2 r0;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r0.x) : "f"(dec.x));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r0.y) : "f"(dec.y));
  const float2 e = __ffma2_rn(make_float2(-dec.x, -dec.y), r0, make_float2(1.0f, 1.0f));
  rcp = __ffma2_rn(r0, e, r0);
  codes = c2;
}

// As quantize_group_pair, with the branch-free scales; q1 / sf1 are row 1's outputs (equal to row 0's
// for the odd last row: row 1 is stored first and row 0 overwrites it).  In every layout the codes of
// scale column c start at byte 8 c of the row, and a critical group's residual sits 1 (mode 16) or 2
// (mode 32) columns after its main part.
__device__ __forceinline__ void quantize_group_pair_ws(uint32_t (&w)[16], int g, int G0, bool mode32, bool is_weight,
                                                       uint8_t* q0, uint8_t* q1, uint8_t* sf0, uint8_t* sf1) {
  const uint32_t m = amax_pair_h(w);
  uint32_t codes;
  float2 dec, rcp;
  scale_of_pair_fma(m, codes, dec, rcp);
  uint2 c0, c1;
  encode_pair(w, rcp.x, rcp.y, c0, c1);
  const int j = g - G0;
  const bool critical = j >= 0;
  uint32_t col = (uint32_t)g;
  if (critical) col = mode32 ? (uint32_t)(G0 + ((j >> 1) << 2) + (j & 1)) : (uint32_t)(g + j);
  const uint32_t cm = ((col >> 2) << 9) | (col & 3u);
  *reinterpret_cast<uint2*>(q1 + 8u * col) = c1;
  sf1[cm] = (uint8_t)(codes >> 8);
  *reinterpret_cast<uint2*>(q0 + 8u * col) = c0;
  sf0[cm] = (uint8_t)codes;
  if (!critical) return;

  uint2 e0 = c0, e1 = c1;
  uint32_t rcodes = codes;
  if (!is_weight) {
    float d0 = dec.x, d1 = dec.y;
    if (mode32) {   // against the un-rounded fp32 scale
      d0 = make_scale_slow(__uint_as_float((m & 0xffffu) << 16)).raw;
      d1 = make_scale_slow(__uint_as_float((m >> 16) << 16)).raw;
    }
    residual_pair(w, c0, c1, d0, d1);
    const uint32_t rm = amax_pair_h(w);
    float2 rdec, rrcp;
    scale_of_pair_fma(rm, rcodes, rdec, rrcp);
    encode_pair(w, rrcp.x, rrcp.y, e0, e1);
  }
  const uint32_t rcol = col + (mode32 ? 2u : 1u);
  const uint32_t cr = ((rcol >> 2) << 9) | (rcol & 3u);
  *reinterpret_cast<uint2*>(q1 + 8u * rcol) = e1;
  sf1[cr] = (uint8_t)(rcodes >> 8);
  *reinterpret_cast<uint2*>(q0 + 8u * rcol) = e0;
  sf0[cr] = (uint8_t)rcodes;
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), completing on `bar`.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// bf16(x / s) for bf16 x and a bf16 divisor s shared by the whole tensor, as one multiplication by
// r = fp32(1/s): the caller rounds the product to bf16, and that rounding cannot differ from the
// rounding of the exact quotient.  With 8-bit significands mx, ms the quotient mx/ms is never within
// 2^-18 (relative) of the midpoint of two bf16 values unless it is a bf16 value itself (a dyadic
// mx/ms has at most 8 significant bits), while x*r is within 2^-23 of it; the same holds for the
// fp32 quotient an IEEE division would round first.  That argument needs a product that is a normal
// number with room to spare.  Products below 2^-60 in magnitude may round differently from the quotient,
// but never visibly: with the smallest block scale 2^-9 and the coarsest step of the e2m1 grid such an
// element (and its residual) quantizes to a zero of its own sign either way, and a group in which every
// element is that small gets the smallest scale either way - the codes and scale bytes, the only outputs,
// are the same.  So there is no per-element guard (it cost more than the multiplication: a third of the
// time of the wide operator); what is checked once is the divisor: when it is zero, not finite, or so
// large or small that 1/s is not a well-scaled normal number, every element takes the IEEE division.
// A large product is as accurate as any other, and where it overflows the quotient is beyond the largest
// bf16 number as well; NaN and infinite elements give the same NaN / infinity either way.
__device__ __forceinline__ bool div_by_reciprocal_ok(float s) {
  const float m = fabsf(s);
  return m >= 7.8886091e-31f && m <= 1.2676506e30f;   // 2^-100 .. 2^100
}
// Words wa, wb: two channels of row 0 and of row 1.  o0 / o1: (row 0, row 1) of the first / second channel.
__device__ __forceinline__ void div_pair_words(uint32_t wa, uint32_t wb, float s, float r, bool fast, uint32_t& o0,
                                               uint32_t& o1) {
  if (fast) {
    const float2 r2 = make_float2(r, r);
    const float2 q0 = __fmul2_rn(make_float2(bf16lo(wa), bf16lo(wb)), r2);
    const float2 q1 = __fmul2_rn(make_float2(bf16hi(wa), bf16hi(wb)), r2);
    o0 = pack_bf16x2_rn(q0.x, q0.y);
    o1 = pack_bf16x2_rn(q1.x, q1.y);
  } else {
    o0 = pack_bf16x2_rn(__fdiv_rn(bf16lo(wa), s), __fdiv_rn(bf16lo(wb), s));
    o1 = pack_bf16x2_rn(__fdiv_rn(bf16hi(wa), s), __fdiv_rn(bf16hi(wb), s));
  }
}

// S: stages of the gather ring (interleaved row pairs).  R: stages of the raw ring (row pairs as they
// lie in global memory, filled by bulk copies - this is what keeps enough bytes in flight to cover
// the HBM latency).  RMS: fused RMSNorm.  WIDE (plain only): rows of more than 8192 channels - the offset
// table holds 16-bit entries so that table, two gather stages and one raw stage fit in shared memory.
// Threads [0, nteams*nct) are consumers in teams of nct threads - team k takes the row pairs
// k, k + nteams, ... of this CTA, so several pairs are being quantized at once.  After them come
// npteams producer teams of npt = KQ/16 threads (more than one only with RMSNorm, whose producers carry
// real arithmetic), sharing the pairs the same way; producer t of a team owns the 16-byte chunks t and
// t + KQ/16 of each row, the reference's assignment and summation order for RMSNorm.
// XR: the CTA is launched with 1024 threads at 64 registers each and re-divides them: every warp that is
// not a consumer gives registers back (56 left; padding warps then leave), the consumer warps take 88.
// Measured on the fused operator at 4096 channels: 0.0988 -> 0.0953 ms per 32 768 tokens.  Other splits were
// slower: 48 / 104 (0.105 ms) and 40 / 128 (0.152 ms) starve the producers; helper warps cut to 32 or 48
// registers in warpgroups of their own double the time (the reducers sit on the critical path); quantizing a
// thread's two groups side by side instead of one after the other costs time with 88 and with 104 registers.
template <bool RMS, bool WIDE, bool SCALED, int S, int R, bool XR = false>
__global__ void __launch_bounds__(1024, 1) arcq_quantize_ws_kernel(const QuantParams p, const int nct, const int npt, const int nteams,
                                                                        const int npteams) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int tid = threadIdx.x;
  const int KQ = p.KQ, G = p.G;
  uint32_t rows = (uint32_t)p.rows, npairs = (uint32_t)p.npairs;
  // This CTA is number `cta` of the `stride` CTAs that share a run of rows: the whole input, or - with
  // grouped rows - run e = blockIdx.x % ngroups, whose rows start at output row `row_base`.
  uint32_t cta = blockIdx.x, stride = gridDim.x, row_base = 0;
  const int16_t* idx_g = p.idx;
  const float* scale_g = p.scale;
  if (p.groups != nullptr) {
    // (the table may have been written by the previous kernel of the stream)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t ng = (uint32_t)p.ngroups, e = blockIdx.x % ng;
    cta = blockIdx.x / ng;
    stride = (gridDim.x - e + ng - 1) / ng;
    row_base = (uint32_t)__ldg(p.groups + e);
    rows = (uint32_t)__ldg(p.groups + ng + e);
    npairs = (rows + 1) >> 1;
    if (idx_g) idx_g += (size_t)e * (size_t)KQ;
    if (scale_g) scale_g += e;
  }
  if (cta >= npairs) return;   // (whole CTA: nothing was set up yet)
  const int* row_map = p.row_map;
  // input row of output row r of this run
  auto in_row = [&](uint32_t r) -> const uint16_t* {
    const uint32_t gr = row_base + r;
    return p.x + (size_t)(row_map ? (uint32_t)__ldg(row_map + gr) : gr) * (size_t)KQ;
  };

  // shared layout: [barriers, abort flag: 384 B][offsets][partial sums, rstd][gather ring][raw ring]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 376);
  size_t cursor = 384;
  uint32_t* offs32 = reinterpret_cast<uint32_t*>(smem + cursor);
  uint16_t* offs16 = reinterpret_cast<uint16_t*>(smem + cursor);
  cursor += (size_t)KQ * (WIDE ? 2 : 4);
  float* psum = nullptr;
  float* rstd_s = nullptr;
  if (RMS) {
    psum = reinterpret_cast<float*>(smem + cursor);
    cursor += (size_t)4 * npt * npteams * sizeof(float);   // per producer team: two buffers of two rows
    rstd_s = reinterpret_cast<float*>(smem + cursor);
    cursor += (size_t)16 * npteams;
  }
  uint8_t* stages = smem + cursor;
  const uint32_t stage_bytes = (uint32_t)KQ * 4;
  uint8_t* raw = stages + (size_t)S * stage_bytes;
  const uint32_t row_in_bytes = (uint32_t)KQ * 2;
  const uint32_t full0 = smem_addr(bars), empty0 = smem_addr(bars + S), raw0 = smem_addr(bars + 2 * S);
  // RMSNorm only: raw stage handed back to the loader; per producer team, partial sums ready (x2
  // buffers) and reciprocal roots ready (x2)
  const uint32_t rawe0 = raw0 + 8 * R, psr0 = rawe0 + 8 * R, rsr0 = psr0 + 8 * 4;

  asm volatile("griddepcontrol.launch_dependents;");   // the next kernel of the stream may be set up now
  // Bulk copies of the rows of `unit` into raw stage `rs` (one thread).
  auto issue = [&](uint32_t unit, uint32_t rs) {
    if (unit >= npairs) return;
    const uint32_t r0 = 2 * unit;
    const bool has1 = (r0 + 1) < rows;
    const uint32_t bar = raw0 + 8 * rs;
    const uint32_t dst = smem_addr(raw + (size_t)rs * stage_bytes);
    mbar_expect_tx(bar, has1 ? 2 * row_in_bytes : row_in_bytes);
    bulk_load(dst, in_row(r0), row_in_bytes, bar);
    if (has1) bulk_load(dst + row_in_bytes, in_row(r0 + 1), row_in_bytes, bar);
  };
  // WIDE: the raw ring holds half pairs (the same half of the channels of both rows), so that the
  // copies of the next half overlap the work on this one although only ~1.5 pairs of raw rows fit.
  // Half u of this CTA is half u & 1 of its pair u >> 1.
  auto issue_half = [&](uint32_t u, uint32_t rs) {
    const uint32_t unit = cta + (u >> 1) * stride;
    if (unit >= npairs) return;
    const uint32_t r0 = 2 * unit, hbytes = row_in_bytes >> 1;
    const bool has1 = (r0 + 1) < rows;
    const uint32_t bar = raw0 + 8 * rs;
    const uint32_t dst = smem_addr(raw + (size_t)rs * row_in_bytes);
    const size_t hoff = (size_t)(u & 1u) * (size_t)(KQ >> 1);
    mbar_expect_tx(bar, has1 ? 2 * hbytes : hbytes);
    bulk_load(dst, in_row(r0) + hoff, hbytes, bar);
    if (has1) bulk_load(dst + hbytes, in_row(r0 + 1) + hoff, hbytes, bar);
  };
  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full0 + 8 * s, (uint32_t)(npt >> 5));    // one arrival per producer warp
      mbar_init(empty0 + 8 * s, (uint32_t)(nct >> 5));   // one arrival per warp of the consuming team
    }
    for (int r = 0; r < R; ++r) mbar_init(raw0 + 8 * r, 1);   // the thread that issues the copies
    if (RMS) {
      for (int r = 0; r < R; ++r) mbar_init(rawe0 + 8 * r, (uint32_t)(npt >> 5));   // one arrival per producer warp
      for (int k = 0; k < 4; ++k) {
        mbar_init(psr0 + 8 * k, (uint32_t)(npt >> 5));
        mbar_init(rsr0 + 8 * k, 2);                                                 // the two reducer warps
      }
    }
    abort_flag[0] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the bulk copies see the barriers
    // The first R row pairs start streaming in while the CTA builds its tables (global memory may
    // still be written by the previous kernel of the stream until this wait returns).
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (uint32_t r = 0; r < (uint32_t)R; ++r) {
      if (WIDE) issue_half(r, r);
      else issue(cta + r * stride, r);
    }
  }
  // Everything before this line touched shared memory only; global memory may still be written by
  // the previous kernel of the stream (no-op unless launched as a programmatic dependent).
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // Offsets are laid out [vector v][group g][entries of one 128-bit load]: consecutive lanes (groups)
  // read consecutive 16 bytes, so every table load is conflict free.
  auto put = [&](int j, int c) {
    const int g = j >> 4, i = j & 15;
    if (WIDE) offs16[(((i >> 3) * G + g) << 3) | (i & 7)] = (uint16_t)word_offset((uint32_t)c);
    else offs32[(((i >> 2) * G + g) << 2) | (i & 3)] = word_offset((uint32_t)c);
  };
  if (idx_g && (reinterpret_cast<uintptr_t>(idx_g) & 15u) == 0) {
    // eight indices per 128-bit load: one round trip to global memory for rows of up to 8192 channels
    const uint4* idx4 = reinterpret_cast<const uint4*>(idx_g);
    for (int v = tid; v < (KQ >> 3); v += blockDim.x) {
      const uint4 w = __ldg(idx4 + v);
      const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        put(8 * v + 2 * k, (int)(int16_t)(ww[k] & 0xffffu));
        put(8 * v + 2 * k + 1, (int)(int16_t)(ww[k] >> 16));
      }
    }
  } else {
    for (int j = tid; j < KQ; j += blockDim.x) put(j, idx_g ? (int)idx_g[j] : j);
  }
  __syncthreads();

  const int ncons = nteams * nct;
  if (tid >= ncons) {
    if (XR) {   // (whole warpgroups: the consumers are a multiple of 128 threads)
      asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
      if (tid >= ncons + npteams * (npt + (RMS ? 96 : 0))) return;   // padding warps
    }
    // ------------------------------------------------------------------ producers
    // A producer team is npt producers and, with RMSNorm, three helper warps behind them: two reducers
    // (one per row of the pair: they finish the sum of squares of pair m while the producers normalise
    // pair m-1) and a loader (one thread that starts the bulk copies).
    const int team_threads = npt + (RMS ? 96 : 0);
    const int pteam = (tid - ncons) / team_threads, ptid = (tid - ncons) - pteam * team_threads;
    const int lane = tid & 31, bar_id = 1 + pteam;
    const uint32_t NP = (uint32_t)npteams;
    const int c0 = ptid, c1 = ptid + npt;   // this thread's 16-byte chunks
    if (RMS) { psum += (size_t)pteam * 4 * npt; rstd_s += 4 * pteam; }
    const uint32_t n = (npairs - cta + stride - 1) / stride;   // row pairs of this CTA
    const uint32_t nt = n > (uint32_t)pteam ? (n - pteam + NP - 1) / NP : 0;   // pairs of this team
    const uint32_t psr = psr0 + 16 * pteam, rsr = rsr0 + 16 * pteam;           // this team's barrier pairs
    if (RMS && ptid >= npt) {
      const int helper = (ptid - npt) >> 5;
      if (helper < 2) {
        // -------------------------------------------------------------- reducers (row = helper)
        for (uint32_t m = 0; m < nt; ++m) {
          if (!mbar_wait(psr + 8 * (m & 1u), (m >> 1) & 1u, abort_flag)) break;
          const float t = rms_tree(psum + (size_t)(m & 1u) * 2 * npt + helper * npt, npt, lane);
          if (lane == 0) {
            rstd_s[(m & 1u) * 2 + helper] = __frsqrt_rn(__fadd_rn(__fdiv_rn(t, (float)KQ), p.eps));
            mbar_arrive(rsr + 8 * (m & 1u));
          }
        }
      } else if (lane == 0) {
        // -------------------------------------------------------------- loader
        uint32_t next = (uint32_t)pteam;    // first pair of this team whose copies are not started yet
        while (next < n && next < (uint32_t)R) next += NP;   // (the first R pairs were started in the prologue)
        // Stay until the producers have taken the team's last pair (or the CTA aborts): every stage that
        // comes back is refilled with the pair R further on, while there is one.
        uint32_t freed = (uint32_t)pteam;   // first pair of this team whose stage is not handed back yet
        bool ok = true;
        for (; freed < n; freed += NP) {
          const uint32_t bar = rawe0 + 8 * (freed % R), par = (freed / R) & 1u;
          if (!mbar_try_wait(bar, par)) {
            unsigned long long t0, t1;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
            for (uint32_t spin = 1; !mbar_try_wait(bar, par); ++spin) {
              if ((spin & 255u) == 0) {
                asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
                if (*abort_flag) { ok = false; break; }
                if (t1 - t0 > QUANT_WAIT_LIMIT_NS) {
                  *abort_flag = 1;
                  atomicExch(&g_quant_error, ARCQ_ERR_TIMEOUT);
                  ok = false;
                  break;
                }
              }
            }
            if (!ok) break;
          }
          if (next < n) { issue(cta + next * stride, freed % R); next += NP; }
        }
        if (!ok) {
          // Giving up with bulk copies possibly in flight: wait (bounded) for those started here, so
          // that none lands in shared memory after the CTA has gone.
          for (uint32_t j = freed; j < next && j < n; j += NP) {
            unsigned long long t0, t1;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
            while (!mbar_try_wait(raw0 + 8 * (j % R), (j / R) & 1u)) {
              __nanosleep(256);
              asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
              if (t1 - t0 > QUANT_WAIT_LIMIT_NS) break;
            }
          }
        }
      }
      return;
    }
    // RMSNorm gains of this thread's sixteen channels, kept packed (two bf16 per register)
    uint4 gn0 = make_uint4(0, 0, 0, 0), gn1 = gn0;
    if (RMS) {
      gn0 = reinterpret_cast<const uint4*>(p.gamma)[c0];
      gn1 = reinterpret_cast<const uint4*>(p.gamma)[c1];
    }

    const uint4 zero = make_uint4(0, 0, 0, 0);
    auto read_raw = [&](uint32_t j, bool has1, uint4& a0, uint4& a1, uint4& b0, uint4& b1) {
      const uint4* rw = reinterpret_cast<const uint4*>(raw + (size_t)(j % R) * stage_bytes);
      a0 = rw[c0]; a1 = rw[c1];
      b0 = has1 ? rw[2 * npt + c0] : zero;
      b1 = has1 ? rw[2 * npt + c1] : zero;
    };
    // Interleaves (and, with RMSNorm, normalises) this thread's chunks of pair j into its gather stage.
    auto fill_stage = [&](uint32_t j, const uint4& a0, const uint4& a1, const uint4& b0, const uint4& b1,
                          const float2 rstd) {
      const uint32_t s = j % S;
      uint4* b4 = reinterpret_cast<uint4*>(stages + (size_t)s * stage_bytes);
      auto fill = [&](int c, const uint4& a, const uint4& b, const uint4& g8) {
        uint4 lo, hi;  // words of channels 8c..8c+3 and 8c+4..8c+7: (row0[ch], row1[ch]) per word
        if (RMS) {
          // bf16 x bf16 is exact in fp32; then one rounding by rstd (both rows in one FMUL2), one to bf16
          auto norm = [&](uint32_t wa, uint32_t wb, uint32_t gw, uint32_t& o0, uint32_t& o1) {
            const uint16_t ga = half_lo(gw), gb = half_hi(gw);
            const float2 t0 = make_float2(fma_bf16(half_lo(wa), ga, -0.0f), fma_bf16(half_lo(wb), ga, -0.0f));
            const float2 t1 = make_float2(fma_bf16(half_hi(wa), gb, -0.0f), fma_bf16(half_hi(wb), gb, -0.0f));
            const float2 n0 = __fmul2_rn(t0, rstd), n1 = __fmul2_rn(t1, rstd);
            o0 = pack_bf16x2_rn(n0.x, n0.y);
            o1 = pack_bf16x2_rn(n1.x, n1.y);
          };
          norm(a.x, b.x, g8.x, lo.x, lo.y);
          norm(a.y, b.y, g8.y, lo.z, lo.w);
          norm(a.z, b.z, g8.z, hi.x, hi.y);
          norm(a.w, b.w, g8.w, hi.z, hi.w);
        } else {
          lo.x = __byte_perm(a.x, b.x, 0x5410); lo.y = __byte_perm(a.x, b.x, 0x7632);
          lo.z = __byte_perm(a.y, b.y, 0x5410); lo.w = __byte_perm(a.y, b.y, 0x7632);
          hi.x = __byte_perm(a.z, b.z, 0x5410); hi.y = __byte_perm(a.z, b.z, 0x7632);
          hi.z = __byte_perm(a.w, b.w, 0x5410); hi.w = __byte_perm(a.w, b.w, 0x7632);
        }
        // XOR-swizzled 16-byte units: the eight lanes of a 128-bit store wavefront hit distinct banks
        b4[swz16(2u * c)] = lo;
        b4[swz16(2u * c + 1u)] = hi;
      };
      fill(c0, a0, b0, gn0);
      fill(c1, a1, b1, gn1);
      __syncwarp();
      if (lane == 0) mbar_arrive(full0 + 8 * s);
    };

    // Copies in flight are tracked by pair number (this team's pairs: pteam, pteam + NP, ...):
    uint32_t issued = (uint32_t)pteam;   // first pair of this team whose copies were NOT started yet
    while (issued < n && issued < (uint32_t)R) issued += NP;
    uint32_t landed = (uint32_t)pteam;   // first pair of this team whose copies were not waited for yet
    bool failed = false;
    if (!RMS && WIDE) {
      const int hc = KQ >> 4;   // 16-byte chunks of half a row
      float sc = 1.0f, rsc = 1.0f;
      bool fast = true;
      if (SCALED) {
        sc = __uint_as_float(pack_bf16x2_rn(__ldg(scale_g), 0.f) << 16);   // (the divisor as bf16, see below)
        rsc = __frcp_rn(sc);
        fast = div_by_reciprocal_ok(sc);
      }
      const uint32_t nu = 2 * n;
      issued = nu < (uint32_t)R ? nu : (uint32_t)R;
      landed = 0;
      for (uint32_t u = 0; u < nu; ++u) {
        const uint32_t it = u >> 1, h = u & 1u;
        const uint32_t unit = cta + it * stride;
        const bool has1 = (2 * unit + 1) < rows;
        if (!failed && !mbar_wait(raw0 + 8 * (u % R), (u / R) & 1u, abort_flag)) failed = true;
        if (!failed) landed = u + 1;
        if (h == 0 && !failed && !mbar_wait(empty0 + 8 * (it % S), ((it / S) & 1u) ^ 1u, abort_flag)) failed = true;
        if (!failed) {
          const uint4* rw = reinterpret_cast<const uint4*>(raw + (size_t)(u % R) * row_in_bytes);
          uint4* b4 = reinterpret_cast<uint4*>(stages + (size_t)(it % S) * stage_bytes);
          const uint32_t cbase = h * (uint32_t)hc;
          for (int c = ptid; c < hc; c += npt) {
            const uint4 a = rw[c], b = has1 ? rw[hc + c] : zero;
            uint4 lo, hi;
            if (SCALED) {
              auto dv = [&](uint32_t wa, uint32_t wb, uint32_t& o0, uint32_t& o1) {
                div_pair_words(wa, wb, sc, rsc, fast, o0, o1);
              };
              dv(a.x, b.x, lo.x, lo.y); dv(a.y, b.y, lo.z, lo.w);
              dv(a.z, b.z, hi.x, hi.y); dv(a.w, b.w, hi.z, hi.w);
            } else {
              lo.x = __byte_perm(a.x, b.x, 0x5410); lo.y = __byte_perm(a.x, b.x, 0x7632);
              lo.z = __byte_perm(a.y, b.y, 0x5410); lo.w = __byte_perm(a.y, b.y, 0x7632);
              hi.x = __byte_perm(a.z, b.z, 0x5410); hi.y = __byte_perm(a.z, b.z, 0x7632);
              hi.z = __byte_perm(a.w, b.w, 0x5410); hi.w = __byte_perm(a.w, b.w, 0x7632);
            }
            const uint32_t cc = cbase + (uint32_t)c;
            b4[swz16(2u * cc)] = lo;
            b4[swz16(2u * cc + 1u)] = hi;
          }
          if (h == 1u) {
            __syncwarp();
            if (lane == 0) mbar_arrive(full0 + 8 * (it % S));
          }
        }
        // every producer is done with this half stage: refill it, or leave together
        if (named_barrier_or(bar_id, team_threads, failed)) break;
        if (ptid == 0 && u + R < nu) { issue_half(u + R, u % R); issued = u + R + 1; }
      }
    } else if (!RMS) {
      const int nchunks = KQ >> 3;
      float sc = 1.0f, rsc = 1.0f;
      bool fast = true;
      if (SCALED) {
        // torch's CUDA kernel for (bf16 tensor) / (fp32 scalar tensor) loads the divisor as bf16
        sc = __uint_as_float(pack_bf16x2_rn(__ldg(scale_g), 0.f) << 16);
        rsc = __frcp_rn(sc);
        fast = div_by_reciprocal_ok(sc);
      }
      for (uint32_t it = 0; it < n; ++it) {
        const uint32_t unit = cta + it * stride;
        const bool has1 = (2 * unit + 1) < rows;
        if (!failed && !mbar_wait(raw0 + 8 * (it % R), (it / R) & 1u, abort_flag)) failed = true;
        if (!failed) landed = it + 1;
        if (!failed && !mbar_wait(empty0 + 8 * (it % S), ((it / S) & 1u) ^ 1u, abort_flag)) failed = true;
        if (!failed) {
          // this thread's chunks c = ptid, ptid + npt, ...: interleave the two rows (dividing by the
          // tensor's scale first, if asked) straight from the raw stage into the gather stage
          const uint4* rw = reinterpret_cast<const uint4*>(raw + (size_t)(it % R) * stage_bytes);
          uint4* b4 = reinterpret_cast<uint4*>(stages + (size_t)(it % S) * stage_bytes);
          auto do_chunk = [&](int c) {
            const uint4 a = rw[c], b = has1 ? rw[nchunks + c] : zero;
            uint4 lo, hi;  // words of channels 8c..8c+3 and 8c+4..8c+7: (row0[ch], row1[ch]) per word
            if (SCALED) {
              auto dv = [&](uint32_t wa, uint32_t wb, uint32_t& o0, uint32_t& o1) {
                div_pair_words(wa, wb, sc, rsc, fast, o0, o1);
              };
              dv(a.x, b.x, lo.x, lo.y); dv(a.y, b.y, lo.z, lo.w);
              dv(a.z, b.z, hi.x, hi.y); dv(a.w, b.w, hi.z, hi.w);
            } else {
              lo.x = __byte_perm(a.x, b.x, 0x5410); lo.y = __byte_perm(a.x, b.x, 0x7632);
              lo.z = __byte_perm(a.y, b.y, 0x5410); lo.w = __byte_perm(a.y, b.y, 0x7632);
              hi.x = __byte_perm(a.z, b.z, 0x5410); hi.y = __byte_perm(a.z, b.z, 0x7632);
              hi.z = __byte_perm(a.w, b.w, 0x5410); hi.w = __byte_perm(a.w, b.w, 0x7632);
            }
            // XOR-swizzled 16-byte units: the eight lanes of a 128-bit store wavefront hit distinct banks
            b4[swz16(2u * c)] = lo;
            b4[swz16(2u * c + 1u)] = hi;
          };
          if (nchunks == 2 * npt) {   // the decoder-layer widths: exactly two chunks per thread
            do_chunk(ptid);
            do_chunk(ptid + npt);
          } else {
            for (int c = ptid; c < nchunks; c += npt) do_chunk(c);
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(full0 + 8 * (it % S));
        }
        // Producers meet once per pair: every one of them is done with the raw stage, so it is
        // refilled; and all leave together if any wait gave up.
        if (named_barrier_or(bar_id, team_threads, failed)) break;
        if (ptid == 0 && it + R < n) { issue(unit + R * stride, it % R); issued = it + R + 1; }
      }
    } else {
      // Software pipeline, synchronised by mbarriers only: normalise and hand over this team's pair
      // m-1 (pass 2, its chunks still in registers; the reducers had a whole iteration for its sum),
      // then take pair m out of its raw stage, give the stage back to the loader, and accumulate its
      // sum of squares (pass 1).
      uint4 a0 = zero, a1 = zero, b0 = zero, b1 = zero;
      for (uint32_t m = 0; m <= nt; ++m) {
        const uint32_t it = pteam + m * NP;               // pair number within the CTA
        if (m >= 1) {
          const uint32_t j = it - NP, q = m - 1;
          if (!mbar_wait(rsr + 8 * (q & 1u), (q >> 1) & 1u, abort_flag)) break;
          const float2 rstd = make_float2(rstd_s[(q & 1u) * 2], rstd_s[(q & 1u) * 2 + 1]);
          if (!mbar_wait(empty0 + 8 * (j % S), ((j / S) & 1u) ^ 1u, abort_flag)) break;
          fill_stage(j, a0, a1, b0, b1, rstd);
        }
        if (m < nt) {
          const uint32_t unit = cta + it * stride;
          const bool has1 = (2 * unit + 1) < rows;
          if (!mbar_wait(raw0 + 8 * (it % R), (it / R) & 1u, abort_flag)) break;
          read_raw(it, has1, a0, a1, b0, b1);
          // reference thread t adds chunk t, then chunk t + KQ/16, eight elements each, in order
          float ss0 = 0.f, ss1 = 0.f;   // x*x is exact in fp32, so each step rounds once, like the fp32 FMA
          const uint32_t wa[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
          const uint32_t wb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            ss0 = fma_bf16(half_lo(wa[i]), half_lo(wa[i]), ss0);
            ss1 = fma_bf16(half_lo(wb[i]), half_lo(wb[i]), ss1);
            ss0 = fma_bf16(half_hi(wa[i]), half_hi(wa[i]), ss0);
            ss1 = fma_bf16(half_hi(wb[i]), half_hi(wb[i]), ss1);
          }
          float* ps = psum + (size_t)(m & 1u) * 2 * npt;
          ps[ptid] = ss0;
          ps[npt + ptid] = ss1;
          __syncwarp();   // every lane has its chunks in registers and its partial sums in place
          if (lane == 0) {
            mbar_arrive(rawe0 + 8 * (it % R));
            mbar_arrive(psr + 8 * (m & 1u));
          }
        }
      }
    }
    // Giving up with bulk copies possibly in flight: wait (bounded) for those this CTA started, so that
    // none lands in shared memory after the CTA has gone.
    if (!RMS && failed && ptid == 0) {
      for (uint32_t j = landed; j < issued; j += NP) {
        unsigned long long t0, t1;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
        while (!mbar_try_wait(raw0 + 8 * (j % R), (j / R) & 1u)) {
          __nanosleep(256);
          asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
          if (t1 - t0 > QUANT_WAIT_LIMIT_NS) break;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ consumers
    if (XR) asm volatile("setmaxnreg.inc.sync.aligned.u32 88;");
    const int team = tid / nct, ctid = tid - team * nct;
    const int warp = ctid >> 5, lane = tid & 31, ncw = nct >> 5;
    const size_t row_bytes = (size_t)(KQ + p.KE) / 2, tile_bytes = (size_t)p.natoms * 512;
    const int G0 = p.G0;
    const bool mode32 = p.mode == 32, is_weight = p.is_weight != 0;
    int slot = warp;   // which 32 groups this warp takes; rotates so the critical groups move around
    // (npairs < 2^29 and at most a few grid strides beyond it: 32-bit unit numbers do not wrap)
    uint32_t it = (uint32_t)team;
    for (uint32_t unit = cta + it * stride; unit < npairs; unit += (uint32_t)nteams * stride, it += (uint32_t)nteams) {
      const uint32_t s = it % S, ph = (it / S) & 1u;
      const bool has1 = (2 * unit + 1) < rows;
      const uint32_t r0 = row_base + 2 * unit;     // output row (runs start on even rows)
      uint8_t* q0 = p.q + (size_t)r0 * row_bytes;
      // 128-row tile, then 16 bytes per row % 32 and 4 per (row / 32) % 4; row 1 of the pair is the
      // next row of the same 32-row run
      uint8_t* sf0 = p.sf + (size_t)(r0 >> 7) * tile_bytes + (((r0 & 31u) << 4) | (((r0 >> 5) & 3u) << 2));
      uint8_t* q1 = has1 ? q0 + row_bytes : q0;
      uint8_t* sf1 = has1 ? sf0 + 16 : sf0;
      const uint8_t* buf = stages + (size_t)s * stage_bytes;
      if (!mbar_wait(full0 + 8 * s, ph, abort_flag)) break;
      // Whole warps walk the groups: a lane beyond the last group (rows whose group count is not a
      // multiple of 32) gathers the last group again and stores nothing; a warp without any group for
      // this pair still hands the stage back.
      bool released = false;
      for (int gb = slot * 32; gb < G; gb += nct) {
        const bool live = gb + lane < G;
        const int g = live ? gb + lane : G - 1;
        uint32_t w[16];
        if (WIDE) {
          const uint4* op = reinterpret_cast<const uint4*>(offs16) + g;
#pragma unroll
          for (int v = 0; v < 2; ++v) {
            const uint4 o = op[v * G];
            const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              w[8 * v + 2 * k] = *reinterpret_cast<const uint32_t*>(buf + (ow[k] & 0xffffu));
              w[8 * v + 2 * k + 1] = *reinterpret_cast<const uint32_t*>(buf + (ow[k] >> 16));
            }
          }
        } else {
          const uint4* op = reinterpret_cast<const uint4*>(offs32) + g;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const uint4 o = op[v * G];
            w[4 * v + 0] = *reinterpret_cast<const uint32_t*>(buf + o.x);
            w[4 * v + 1] = *reinterpret_cast<const uint32_t*>(buf + o.y);
            w[4 * v + 2] = *reinterpret_cast<const uint32_t*>(buf + o.z);
            w[4 * v + 3] = *reinterpret_cast<const uint32_t*>(buf + o.w);
          }
        }
        if (gb + nct >= G) {   // last group of this warp: the stage can be refilled
          __syncwarp();
          if (lane == 0) mbar_arrive(empty0 + 8 * s);
          released = true;
        }
        if (live) quantize_group_pair_ws(w, g, G0, mode32, is_weight, q0, q1, sf0, sf1);
      }
      if (!released && lane == 0) mbar_arrive(empty0 + 8 * s);
      slot = slot + 1 == ncw ? 0 : slot + 1;
    }
  }
}

// `nvec` 16-byte words from src to each of n destinations: the codes and scale tiles a rank has just made of
// its token rows, to the same place in its peers' gathered buffers (peer memory over NVLink).  Storing them from
// inside the quantizer as they are made was measured no faster (the transfer is bound by NVLink either way) and
// needs single-byte stores for the scales, a packet each.
struct BroadcastDests {
  uint4* p[7];
};
__global__ void arcq_broadcast_kernel(const uint4* __restrict__ src, const BroadcastDests dst, int n, long long nvec) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const uint4 v = src[i];
    for (int d = 0; d < n; ++d) dst.p[d][i] = v;
  }
}

__global__ void arcq_absmax_kernel(const uint4* __restrict__ x, long long nvec, const uint16_t* tail,
                                   int ntail, unsigned int* out) {
  uint32_t m = 0;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    uint4 v = ldg_stream(x + i);
    m = max_u16x2(m, v.x & 0x7fff7fffu);
    m = max_u16x2(m, v.y & 0x7fff7fffu);
    m = max_u16x2(m, v.z & 0x7fff7fffu);
    m = max_u16x2(m, v.w & 0x7fff7fffu);
  }
  uint32_t r = max(m & 0xffffu, m >> 16);
  if (blockIdx.x == 0 && (int)threadIdx.x < ntail) r = max(r, (uint32_t)tail[threadIdx.x] & 0x7fffu);
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) r = max(r, __shfl_xor_sync(0xffffffffu, r, d));
  // non-negative floats order like their bit patterns
  if ((threadIdx.x & 31) == 0) atomicMax(out, r << 16);
}

template <bool RMS, bool WIDE, bool SCALED, int S, int R, bool XR = false>
int launch_ws(const QuantParams& p, int nct, int npt, int nteams, int npteams, size_t smem, const DeviceInfo& di,
              cudaStream_t stream) {
  auto kern = arcq_quantize_ws_kernel<RMS, WIDE, SCALED, S, R, XR>;
  const int threads = XR ? 1024 : nteams * nct + npteams * (npt + (RMS ? 96 : 0));
  // the attribute and the occupancy query cost host time: once per (device, block size, shared memory)
  static thread_local int c_dev = -1, c_threads = 0, c_occ = 0;
  static thread_local size_t c_smem = 0;
  int occ = 0;
  if (c_dev == di.device && c_threads == threads && c_smem == smem) {
    occ = c_occ;
  } else {
    ARCQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    ARCQ_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, threads, smem));
    c_dev = di.device; c_threads = threads; c_smem = smem; c_occ = occ;
  }
  if (occ < 1) return ARCQ_ERR_UNSUPPORTED_K;
  long long grid = (long long)di.num_sms * occ;
  if (p.groups == nullptr && grid > p.npairs) grid = p.npairs;
  if (p.groups != nullptr && grid < p.ngroups) return ARCQ_ERR_BAD_SHAPE;   // every run needs a CTA
  // Programmatic dependent launch: the grid may be set up while the previous kernel of the stream is
  // still draining; the kernel itself waits (griddepcontrol.wait) before it touches global memory.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3((unsigned)threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  ARCQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, p, nct, npt, nteams, npteams));
  ARCQ_CUDA_TRY(cudaGetLastError());
  return ARCQ_OK;
}

template <int CPT, int NBUF, int PAIRS, bool RMS, bool RAWIDX, int MAXT, int MINB>
int launch_variant(const QuantParams& p, int nt, size_t smem, const DeviceInfo& di, cudaStream_t stream) {
  auto kern = arcq_quantize_kernel<CPT, NBUF, PAIRS, RMS, RAWIDX, MAXT, MINB>;
  ARCQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int occ = 0;
  ARCQ_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, nt, smem));
  if (occ < 1) return ARCQ_ERR_UNSUPPORTED_K;
  const long long nunits = (p.npairs + PAIRS - 1) / PAIRS;
  long long grid = (long long)di.num_sms * occ;
  if (grid > nunits) grid = nunits;
  kern<<<(unsigned)grid, nt, smem, stream>>>(p);
  ARCQ_CUDA_TRY(cudaGetLastError());
  return ARCQ_OK;
}

}  // namespace

static int launch_quantize_one(const void* x, const void* gamma, float eps, const int16_t* idx, int64_t rows, int KQ,
                               int KE, int mode, int is_weight, uint8_t* q, uint8_t* sf, cudaStream_t stream,
                               const float* scale, const int* groups, int ngroups, const int* row_map);

int launch_quantize(const void* x, const void* gamma, float eps, const int16_t* idx, int64_t rows, int KQ,
                    int KE, int mode, int is_weight, uint8_t* q, uint8_t* sf, cudaStream_t stream, const float* scale,
                    const int* groups, int ngroups, const int* row_map, uint8_t* const* q_extra,
                    uint8_t* const* sf_extra, int nextra) {
  if (rows == 0) return ARCQ_OK;
  if (nextra > 0 && (rows % 128 || nextra > 7)) return ARCQ_ERR_BAD_SHAPE;   // whole scale tiles travel
  int rc = launch_quantize_one(x, gamma, eps, idx, rows, KQ, KE, mode, is_weight, q, sf, stream, scale, groups,
                               ngroups, row_map);
  if (rc != ARCQ_OK || nextra == 0) return rc;
  DeviceInfo di;
  rc = get_device_info(&di);
  if (rc != ARCQ_OK) return rc;
  BroadcastDests bq = {}, bs = {};
  for (int d = 0; d < nextra; ++d) {
    bq.p[d] = reinterpret_cast<uint4*>(q_extra[d]);
    bs.p[d] = reinterpret_cast<uint4*>(sf_extra[d]);
  }
  const long long nq = rows * (long long)((KQ + KE) / 2) / 16;
  const long long ns = (rows / 128) * (long long)(((KQ + KE) / 16 + 3) / 4) * 32;
  const long long cap = (long long)di.num_sms * 8;
  long long bl = (nq + 255) / 256;
  arcq_broadcast_kernel<<<(unsigned)(bl < cap ? bl : cap), 256, 0, stream>>>(reinterpret_cast<const uint4*>(q), bq,
                                                                            nextra, nq);
  bl = (ns + 255) / 256;
  arcq_broadcast_kernel<<<(unsigned)(bl < cap ? bl : cap), 256, 0, stream>>>(reinterpret_cast<const uint4*>(sf), bs,
                                                                            nextra, ns);
  ARCQ_CUDA_TRY(cudaGetLastError());
  return ARCQ_OK;
}

static int launch_quantize_one(const void* x, const void* gamma, float eps, const int16_t* idx, int64_t rows, int KQ,
                               int KE, int mode, int is_weight, uint8_t* q, uint8_t* sf, cudaStream_t stream,
                               const float* scale, const int* groups, int ngroups, const int* row_map) {
  DeviceInfo di;
  int rc = get_device_info(&di);
  if (rc != ARCQ_OK) return rc;

  QuantParams p;
  p.x = static_cast<const uint16_t*>(x);
  p.gamma = static_cast<const uint16_t*>(gamma);
  p.idx = idx;
  p.q = q;
  p.sf = sf;
  p.rows = rows;
  p.npairs = (rows + 1) / 2;
  p.KQ = KQ;
  p.KE = KE;
  p.G = KQ / 16;
  p.G0 = (KQ - KE) / 16;
  p.natoms = ((KQ + KE) / 16 + 3) / 4;
  p.nchunks = KQ / 8;
  p.mode = mode;
  p.is_weight = is_weight;
  p.eps = eps;
  p.scale = scale;
  p.groups = groups;
  p.ngroups = ngroups;
  p.row_map = row_map;

  const bool rms = gamma != nullptr;
  int nt, cpt;
  if (rms) {
    nt = p.G;  // one reference thread per CUDA thread: keeps the accumulation order
    cpt = 2;
  } else {
    int gpt = (p.G + 511) / 512;
    nt = (((p.G + gpt - 1) / gpt) + 31) / 32 * 32;
    int need = (p.nchunks + nt - 1) / nt;
    if (need > 8) return ARCQ_ERR_UNSUPPORTED_K;
    cpt = need <= 2 ? 2 : (need <= 4 ? 4 : 8);
  }
  const bool rawidx = KQ > 16384;

  // Warp-specialised kernel: rows of 512..8192 channels
  // in full, rows of up to 16384 channels for the plain operator.
  const bool gamma_ok = !rms || (reinterpret_cast<uintptr_t>(gamma) & 15u) == 0;   // read with 128-bit loads
  const bool wide = p.G > 512;
  // (RMSNorm: one producer per 16-channel group, in whole warps - the reference's summation order)
  if (gamma_ok && p.G >= 32 && (!rms || (p.G % 32 == 0 && p.G >= 64)) && rows < (1LL << 30) &&
      (wide ? (!rms && p.G <= 1024) : true)) {
    const size_t stage = (size_t)KQ * 4;
    if (wide) {
      // 256 producers, two consumer teams of 256, two gather stages, 16-bit offset table; one raw
      // stage (two if they fit)
      // (twice the producers when they also divide by the tensor's scale)
      const int nct = 256, npt = p.scale ? 512 : 256, nteams = 2;
      // (raw stages here are half pairs, half a gather stage each: two to four of them)
      const size_t fixed = 384 + (size_t)KQ * 2;
      int R = 0;
      if (fixed + 2 * stage <= (size_t)di.max_smem_optin) R = (int)(((size_t)di.max_smem_optin - fixed - 2 * stage) / (stage / 2));
      if (R > 4) R = 4;
      const size_t smem = fixed + 2 * stage + (size_t)R * (stage / 2);
      if (R >= 2) {
        if (p.scale) {
          if (R == 4) return launch_ws<false, true, true, 2, 4>(p, nct, npt, nteams, 1, smem, di, stream);
          if (R == 3) return launch_ws<false, true, true, 2, 3>(p, nct, npt, nteams, 1, smem, di, stream);
          return launch_ws<false, true, true, 2, 2>(p, nct, npt, nteams, 1, smem, di, stream);
        }
        if (R == 4) return launch_ws<false, true, false, 2, 4>(p, nct, npt, nteams, 1, smem, di, stream);
        if (R == 3) return launch_ws<false, true, false, 2, 3>(p, nct, npt, nteams, 1, smem, di, stream);
        return launch_ws<false, true, false, 2, 2>(p, nct, npt, nteams, 1, smem, di, stream);
      }
    } else {
      // Consumer teams of 128 threads (two groups per thread at hidden 4096) were measured faster than
      // teams of 256: more row pairs in flight for the same number of warps.
      const int g32 = (p.G + 31) / 32 * 32;   // threads of a role are whole warps
      int nct = g32 < 128 ? g32 : 128;
      // producers: two 16-byte chunks of each row per thread (the RMSNorm summation order needs exactly
      // that); with the division by the tensor's scale, at least 512 of them share the arithmetic
      const int npt = (p.scale && p.G < 512) ? 512 : g32;
      // One CTA per SM, up to 1024 threads.  Plain: one producer team (it only moves data).  RMSNorm: two
      // producer teams, each with three helper warps.  The rest, up to three teams, are consumers.
      const int ptt = npt + (rms ? 96 : 0);   // threads of a producer team
      int npteams = (rms && 2 * ptt + nct <= 1024) ? 2 : 1;
      int nteams = (1024 - npteams * ptt) / nct;
      if (nteams > 3) nteams = 3;
      // gather stages: 2 for a single consumer team, else 4.  Raw stages: a multiple of the number of
      // producer teams (a stage always serves pairs of the same team), at least two per team.
      int S = nteams > 1 ? 4 : 2;
      size_t fixed = 384 + (size_t)KQ * 4 + (rms ? ((size_t)4 * npt * sizeof(float) + 16) * npteams : 0);
      if (fixed + (S + 2 * npteams) * stage > (size_t)di.max_smem_optin && S == 4) S = 2;
      if (rms && npteams == 2 && fixed + (S + 4) * stage > (size_t)di.max_smem_optin) {
        npteams = 1;   // not enough shared memory for two pipelines
        fixed = 384 + (size_t)KQ * 4 + (size_t)4 * npt * sizeof(float) + 16;
      }
      // A consumer team that is more than one lap of the gather ring ahead would pass its "full" wait
      // on the previous lap's phase: never more consumer teams than gather stages.
      if (nteams > S) nteams = S;
      // With two producer teams the pairs are not filled in order, and a consumer team that comes back to a
      // stage only every third lap would take the parity of an older lap for its own: the number of
      // consumer teams must divide the number of gather stages.
      if (npteams == 2 && nteams == 3) nteams = 2;
      const int r_floor = 2 * npteams;
      int R = 8;
      while (R > r_floor && fixed + (S + R) * stage > (size_t)di.max_smem_optin) R -= 2;
      const size_t smem = fixed + (S + R) * stage;
      if (nteams >= 1 && smem <= (size_t)di.max_smem_optin) {
        const int kind = rms ? 0 : (p.scale ? 2 : 1);   // RMSNorm / plain / plain with the division
        // Fused RMSNorm with one or two whole warpgroups of consumers: registers move from the other warps to them
        // (1024 - ncons warps' worth at 56 leave at least 88 for the consumers).
        // (Only where one CTA per SM is the rule anyway: narrow rows, whose CTAs are small enough for two per
        // SM, keep their own thread count.)
        const int ncons = nteams * nct;
        if (kind == 0 && (ncons == 128 || ncons == 256) && ncons + npteams * ptt > 512) {
#define ARCQ_WS_XR(S_, R_) \
  if (S == S_ && R == R_) return launch_ws<true, false, false, S_, R_, true>(p, nct, npt, nteams, npteams, smem, di, stream);
          ARCQ_WS_XR(2, 2) ARCQ_WS_XR(2, 4) ARCQ_WS_XR(2, 6) ARCQ_WS_XR(2, 8)
          ARCQ_WS_XR(4, 2) ARCQ_WS_XR(4, 4) ARCQ_WS_XR(4, 6) ARCQ_WS_XR(4, 8)
#undef ARCQ_WS_XR
        }
#define ARCQ_WS_CASE(KIND_, RMS_, SCALED_, S_, R_) \
  if (kind == KIND_ && S == S_ && R == R_) \
    return launch_ws<RMS_, false, SCALED_, S_, R_>(p, nct, npt, nteams, npteams, smem, di, stream);
#define ARCQ_WS_ROW(KIND_, RMS_, SCALED_, S_)                                                          \
  ARCQ_WS_CASE(KIND_, RMS_, SCALED_, S_, 2) ARCQ_WS_CASE(KIND_, RMS_, SCALED_, S_, 4)                  \
  ARCQ_WS_CASE(KIND_, RMS_, SCALED_, S_, 6) ARCQ_WS_CASE(KIND_, RMS_, SCALED_, S_, 8)
        ARCQ_WS_ROW(0, true, false, 2) ARCQ_WS_ROW(0, true, false, 4)
        ARCQ_WS_ROW(1, false, false, 2) ARCQ_WS_ROW(1, false, false, 4)
        ARCQ_WS_ROW(2, false, true, 2) ARCQ_WS_ROW(2, false, true, 4)
#undef ARCQ_WS_ROW
#undef ARCQ_WS_CASE
      }
    }
  }
  // only the warp-specialised kernel divides by the scale, walks grouped rows or follows a row map
  if (p.scale || p.groups || p.row_map) return ARCQ_ERR_UNSUPPORTED_K;

  const size_t table = 160 + (((size_t)KQ * (rawidx ? 2 : 4) + 15) & ~(size_t)15);
  auto smem_for = [&](int nbuf, int pairs) {
    return table + (rms ? (size_t)KQ * 4 + (size_t)2 * pairs * nt * sizeof(float) + 16 : 0) +
           (size_t)nbuf * pairs * KQ * 4;
  };
  size_t smem = smem_for(2, 1);
  if (cpt == 8 || rawidx || smem > (size_t)di.max_smem_optin) {
    // very wide rows: one buffer, loads not overlapped with the arithmetic
    smem = smem_for(1, 1);
    if (rms || smem > (size_t)di.max_smem_optin) return ARCQ_ERR_UNSUPPORTED_K;
    return rawidx ? launch_variant<8, 1, 1, false, true, 512, 1>(p, nt, smem, di, stream)
                  : launch_variant<8, 1, 1, false, false, 512, 1>(p, nt, smem, di, stream);
  }
  if (nt <= 256 && cpt == 2) {
    // Narrow rows: one row pair per iteration, three resident CTAs per SM (two pairs per iteration with
    // two resident CTAs were measured slower on B200: fewer warps to hide latency).
    if (rms) return launch_variant<2, 2, 1, true, false, 256, 3>(p, nt, smem, di, stream);
    return launch_variant<2, 2, 1, false, false, 256, 3>(p, nt, smem, di, stream);
  }
  if (rms) return launch_variant<2, 2, 1, true, false, 512, 1>(p, nt, smem, di, stream);
  if (cpt == 2) return launch_variant<2, 2, 1, false, false, 512, 1>(p, nt, smem, di, stream);
  return launch_variant<4, 2, 1, false, false, 512, 1>(p, nt, smem, di, stream);
}

int quant_poll_error() {
  int v = 0, zero = 0;
  ARCQ_CUDA_TRY(cudaDeviceSynchronize());
  ARCQ_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_quant_error, sizeof(int)));
  if (v) ARCQ_CUDA_TRY(cudaMemcpyToSymbol(g_quant_error, &zero, sizeof(int)));
  return v;
}

int launch_absmax(const void* x, int64_t n, float* out, int accumulate, cudaStream_t stream) {
  DeviceInfo di;
  int rc = get_device_info(&di);
  if (rc != ARCQ_OK) return rc;
  if (!accumulate) ARCQ_CUDA_TRY(cudaMemsetAsync(out, 0, sizeof(float), stream));
  if (n == 0) return ARCQ_OK;
  long long nvec = n / 8;
  int ntail = (int)(n - nvec * 8);
  const uint16_t* tail = static_cast<const uint16_t*>(x) + nvec * 8;
  long long blocks = (nvec + 255) / 256;
  long long cap = (long long)di.num_sms * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  arcq_absmax_kernel<<<(unsigned)blocks, 256, 0, stream>>>(static_cast<const uint4*>(x), nvec, tail, ntail,
                                                          reinterpret_cast<unsigned int*>(out));
  ARCQ_CUDA_TRY(cudaGetLastError());
  return ARCQ_OK;
}

}  // namespace arcq
