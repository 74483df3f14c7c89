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
//    32-bit shared load per TWO elements (half the bank-conflict wavefronts of a 16-bit gather);
//  * the next pair is in flight in registers (128-bit coalesced streaming loads) while the current
//    one is quantized (double buffer), so HBM latency is covered by arithmetic;
//  * the channel order is turned once per CTA into a shared table of byte offsets, read back with
//    128-bit loads (8 offsets each) instead of one global int16 load per element per row;
//  * conversions use the hardware cvt.rn.satfinite.{e2m1x2,e4m3x2}.f32 (round to nearest even,
//    saturating), eight codes are packed per 32-bit word and stored 8 bytes per group;
//  * RMSNorm partial sums are taken from the registers of the streaming load, in the reference's
//    accumulation order, and the reciprocal root is the correctly rounded one.
#include <cuda_bf16.h>
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
};

__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

__device__ __forceinline__ uint32_t f32_to_bf16_bits(float f) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f));
}

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
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

__device__ __forceinline__ float e2m1_decode(uint32_t c) {
  uint32_t e = (c >> 1) & 3u, m = c & 1u;
  float v = e ? __uint_as_float(((126u + e) << 23) | (m << 22)) : 0.5f * (float)m;
  return (c & 8u) ? -v : v;
}

// Eight floats -> eight e2m1 codes in one word, element 0 in the lowest nibble.
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

struct GroupScale {
  uint32_t byte;  // ue4m3 code
  float dec;      // its value
  float raw;      // clamp(amax/6, 2^-9, 448) before rounding
  float rcp;      // fp32(1/dec)
};

__device__ __forceinline__ GroupScale make_scale(float amax) {
  GroupScale s;
  float t = __fdiv_rn(amax, 6.0f);
  t = fminf(t, 448.0f);
  s.raw = fmaxf(t, 0.001953125f);
  s.byte = ue4m3_encode(s.raw);
  s.dec = ue4m3_decode(s.byte);
  s.rcp = __frcp_rn(s.dec);
  return s;
}

// Quantize the 16 values held in the low (HI=false) or high (HI=true) halves of w[0..15].
template <bool HI>
__device__ __forceinline__ uint2 encode16(const uint32_t (&w)[16], float rcp) {
  float v[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __fmul_rn(HI ? bf16hi(w[i]) : bf16lo(w[i]), rcp);
  uint2 c;
  c.x = e2m1x8(v[0], v[1], v[2], v[3], v[4], v[5], v[6], v[7]);
  c.y = e2m1x8(v[8], v[9], v[10], v[11], v[12], v[13], v[14], v[15]);
  return c;
}

template <bool HI>
__device__ __forceinline__ float amax16(const uint32_t (&w)[16]) {
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(HI ? bf16hi(w[i]) : bf16lo(w[i])));
  return m;
}

// Residuals of one row's critical group: r[i] = bf16(x - q*s), left in the same half of w.
template <bool HI>
__device__ __forceinline__ void residual16(uint32_t (&w)[16], uint2 codes, const GroupScale& s, int mode) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    uint32_t c = ((i < 8 ? codes.x : codes.y) >> (4 * (i & 7))) & 15u;
    float x = HI ? bf16hi(w[i]) : bf16lo(w[i]);
    float qv = e2m1_decode(c);
    // mode 16: against the rounded scale (the product is exact in fp32);
    // mode 32: against the un-rounded scale, fused, as the 32-wide reference kernels compile.
    float d = (mode == 32) ? __fmaf_rn(-qv, s.raw, x) : __fsub_rn(x, __fmul_rn(qv, s.dec));
    uint32_t b = f32_to_bf16_bits(d);
    w[i] = HI ? ((w[i] & 0x0000ffffu) | (b << 16)) : ((w[i] & 0xffff0000u) | b);
  }
}

__device__ __forceinline__ size_t sf_row_base(long long r, int natoms) {
  return ((size_t)(r >> 7) * (size_t)natoms) * 512 + (size_t)(r & 31) * 16 + (size_t)((r >> 5) & 3) * 4;
}
__device__ __forceinline__ size_t sf_col(int c) { return (size_t)(c >> 2) * 512 + (size_t)(c & 3); }

// Where a group's main / residual codes and scales go.
struct Slot {
  int byte_main, col_main, byte_res, col_res;
};
__device__ __forceinline__ Slot slot_of(int g, int G0, int mode) {
  Slot s;
  if (g < G0) {
    s.byte_main = 8 * g; s.col_main = g; s.byte_res = -1; s.col_res = -1;
  } else if (mode == 32) {
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

template <bool HI>
__device__ __forceinline__ void quantize_store(uint32_t (&w)[16], int g, const QuantParams& p,
                                               uint8_t* qrow, uint8_t* sfrow) {
  GroupScale s = make_scale(amax16<HI>(w));
  uint2 codes = encode16<HI>(w, s.rcp);
  Slot sl = slot_of(g, p.G0, p.mode);
  *reinterpret_cast<uint2*>(qrow + sl.byte_main) = codes;
  sfrow[sf_col(sl.col_main)] = (uint8_t)s.byte;
  if (g >= p.G0) {
    if (p.is_weight) {
      *reinterpret_cast<uint2*>(qrow + sl.byte_res) = codes;
      sfrow[sf_col(sl.col_res)] = (uint8_t)s.byte;
    } else {
      residual16<HI>(w, codes, s, p.mode);
      GroupScale rs = make_scale(amax16<HI>(w));
      uint2 rc = encode16<HI>(w, rs.rcp);
      *reinterpret_cast<uint2*>(qrow + sl.byte_res) = rc;
      sfrow[sf_col(sl.col_res)] = (uint8_t)rs.byte;
    }
  }
}

// Sum-of-squares tree of one row in the reference's order (rmsnorm.cu:131-154 of ARCQuant), done by
// one warp: lane l owns the partials of reference threads l, l+32, ... (zero where none exists).
__device__ __forceinline__ float rms_tree(const float* ps, int nt, int lane) {
  float v[16];
#pragma unroll
  for (int k = 0; k < 16; ++k) {
    int t = lane + 32 * k;
    v[k] = t < nt ? ps[t] : 0.f;
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) v[k] = __fadd_rn(v[k], v[k + 8]);   // +256
#pragma unroll
  for (int k = 0; k < 4; ++k) v[k] = __fadd_rn(v[k], v[k + 4]);   // +128
  v[0] = __fadd_rn(v[0], v[2]);                                   // +64
  v[1] = __fadd_rn(v[1], v[3]);
  float s = __fadd_rn(v[0], v[1]);                                // +32
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) s = __fadd_rn(s, __shfl_down_sync(0xffffffffu, s, d));
  return s;  // valid in lane 0
}

__device__ __forceinline__ float sumsq8(uint4 a, float acc) {
  const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float lo = bf16lo(w[i]), hi = bf16hi(w[i]);
    acc = __fmaf_rn(lo, lo, acc);
    acc = __fmaf_rn(hi, hi, acc);
  }
  return acc;
}

// CPT: 16-byte chunks per thread per row; NBUF: shared row-pair buffers; RMS: fused RMSNorm;
// RAWIDX: the offset table holds channel numbers (rows wider than 16384) instead of byte offsets.
// MAXT / MINB: launch bounds (threads per CTA, CTAs per SM the register budget must allow).
template <int CPT, int NBUF, bool RMS, bool RAWIDX, int MAXT, int MINB>
__global__ void __launch_bounds__(MAXT, MINB) arcq_quantize_kernel(const QuantParams p) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int tid = threadIdx.x, nt = blockDim.x;
  const int KQ = p.KQ;

  uint16_t* offs = reinterpret_cast<uint16_t*>(smem);
  size_t cursor = ((size_t)KQ * 2 + 15) & ~(size_t)15;
  uint16_t* gperm = reinterpret_cast<uint16_t*>(smem + cursor);
  float* psum = nullptr;
  float* rstd_s = nullptr;
  if (RMS) {
    cursor += ((size_t)KQ * 2 + 15) & ~(size_t)15;
    psum = reinterpret_cast<float*>(smem + cursor);
    cursor += (size_t)2 * nt * sizeof(float);
    rstd_s = reinterpret_cast<float*>(smem + cursor);
    cursor += 16;
  }
  uint32_t* bufs = reinterpret_cast<uint32_t*>(smem + cursor);

  for (int j = tid; j < KQ; j += nt) {
    int c = p.idx ? (int)p.idx[j] : j;
    offs[j] = (uint16_t)(RAWIDX ? c : c * 4);
    if (RMS) gperm[j] = p.gamma[c];
  }

  uint4 ra[CPT], rb[CPT];

  auto load_pair = [&](long long pair) {
    const long long r0 = 2 * pair;
    const bool has1 = (r0 + 1) < p.rows;
    const uint4* x0 = reinterpret_cast<const uint4*>(p.x + r0 * (long long)KQ);
    const uint4* x1 = reinterpret_cast<const uint4*>(p.x + (r0 + 1) * (long long)KQ);
#pragma unroll
    for (int j = 0; j < CPT; ++j) {
      int c = tid + j * nt;
      if (c < p.nchunks) {
        ra[j] = ldg_stream(x0 + c);
        rb[j] = has1 ? ldg_stream(x1 + c) : make_uint4(0, 0, 0, 0);
      }
    }
  };

  auto store_pair = [&](uint32_t* buf) {
#pragma unroll
    for (int j = 0; j < CPT; ++j) {
      int c = tid + j * nt;
      if (c < p.nchunks) {
        uint4 lo, hi;  // words 8c..8c+3 and 8c+4..8c+7: (row0[ch], row1[ch]) per word
        lo.x = __byte_perm(ra[j].x, rb[j].x, 0x5410); lo.y = __byte_perm(ra[j].x, rb[j].x, 0x7632);
        lo.z = __byte_perm(ra[j].y, rb[j].y, 0x5410); lo.w = __byte_perm(ra[j].y, rb[j].y, 0x7632);
        hi.x = __byte_perm(ra[j].z, rb[j].z, 0x5410); hi.y = __byte_perm(ra[j].z, rb[j].z, 0x7632);
        hi.z = __byte_perm(ra[j].w, rb[j].w, 0x5410); hi.w = __byte_perm(ra[j].w, rb[j].w, 0x7632);
        uint4* dst = reinterpret_cast<uint4*>(buf + 8 * (size_t)c);
        // Lanes 4..7 of each quarter warp write the upper half first, so that the eight lanes of
        // one 128-bit store wavefront land on distinct banks (byte stride 32 would fold them 2-way).
        const bool swap = (tid & 4) != 0;
        uint4 first, second;
        first.x = swap ? hi.x : lo.x; first.y = swap ? hi.y : lo.y;
        first.z = swap ? hi.z : lo.z; first.w = swap ? hi.w : lo.w;
        second.x = swap ? lo.x : hi.x; second.y = swap ? lo.y : hi.y;
        second.z = swap ? lo.z : hi.z; second.w = swap ? lo.w : hi.w;
        dst[swap ? 1 : 0] = first;
        dst[swap ? 0 : 1] = second;
      }
    }
    if (RMS) {
      // Reference thread t adds chunk t then chunk t+KQ/16, eight elements each, in order.
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int j = 0; j < CPT; ++j) { s0 = sumsq8(ra[j], s0); s1 = sumsq8(rb[j], s1); }
      psum[tid] = s0;
      psum[nt + tid] = s1;
    }
  };

  long long pair = blockIdx.x;
  if (pair < p.npairs) { load_pair(pair); store_pair(bufs); }
  __syncthreads();

  int cur = 0;
  const size_t row_bytes = (size_t)(KQ + p.KE) / 2;
  for (; pair < p.npairs; pair += gridDim.x) {
    const long long nxt = pair + gridDim.x;
    const bool more = nxt < p.npairs;
    if (NBUF == 2 && more) load_pair(nxt);

    float rstd0 = 1.f, rstd1 = 1.f;
    if (RMS) {
      const int warp = tid >> 5, lane = tid & 31;
      if (warp < 2) {
        float ss = rms_tree(psum + warp * nt, nt, lane);
        if (lane == 0) rstd_s[warp] = __frsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)KQ), p.eps));
      }
      __syncthreads();
      rstd0 = rstd_s[0];
      rstd1 = rstd_s[1];
    }

    const uint8_t* buf = reinterpret_cast<const uint8_t*>(bufs + (size_t)cur * KQ);
    const long long r0 = 2 * pair, r1 = r0 + 1;
    const bool has1 = r1 < p.rows;
    uint8_t* q0 = p.q + (size_t)r0 * row_bytes;
    uint8_t* q1 = q0 + row_bytes;
    uint8_t* sf0 = p.sf + sf_row_base(r0, p.natoms);
    uint8_t* sf1 = p.sf + sf_row_base(r1, p.natoms);

    for (int g = tid; g < p.G; g += nt) {
      const uint4* op = reinterpret_cast<const uint4*>(offs + 16 * g);
      const uint4 o0 = op[0], o1 = op[1];
      const uint32_t ow[8] = {o0.x, o0.y, o0.z, o0.w, o1.x, o1.y, o1.z, o1.w};
      uint32_t w[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        uint32_t o = (i & 1) ? (ow[i >> 1] >> 16) : (ow[i >> 1] & 0xffffu);
        w[i] = *reinterpret_cast<const uint32_t*>(buf + (RAWIDX ? o * 4u : o));
      }
      if (RMS) {
        const uint4* gp = reinterpret_cast<const uint4*>(gperm + 16 * g);
        const uint4 g0 = gp[0], g1 = gp[1];
        const uint32_t gw[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float gm = (i & 1) ? bf16hi(gw[i >> 1]) : bf16lo(gw[i >> 1]);
          // bf16 x bf16 is exact in fp32; then one rounding by rstd, one to bf16
          float n0 = __fmul_rn(__fmul_rn(bf16lo(w[i]), gm), rstd0);
          float n1 = __fmul_rn(__fmul_rn(bf16hi(w[i]), gm), rstd1);
          w[i] = f32_to_bf16_bits(n0) | (f32_to_bf16_bits(n1) << 16);
        }
      }
      quantize_store<false>(w, g, p, q0, sf0);
      if (has1) quantize_store<true>(w, g, p, q1, sf1);
    }

    if (NBUF == 2) {
      if (more) store_pair(bufs + (size_t)(cur ^ 1) * KQ);
      __syncthreads();
      cur ^= 1;
    } else {
      __syncthreads();
      if (more) { load_pair(nxt); store_pair(bufs); }
      __syncthreads();
    }
  }
}

__global__ void arcq_absmax_kernel(const uint4* __restrict__ x, long long nvec, const uint16_t* tail,
                                   int ntail, unsigned int* out) {
  float m = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    uint4 v = ldg_stream(x + i);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) m = fmaxf(m, fmaxf(fabsf(bf16lo(w[k])), fabsf(bf16hi(w[k]))));
  }
  if (blockIdx.x == 0 && (int)threadIdx.x < ntail)
    m = fmaxf(m, fabsf(__uint_as_float((uint32_t)tail[threadIdx.x] << 16)));
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
  // non-negative floats order like their bit patterns
  if ((threadIdx.x & 31) == 0) atomicMax(out, __float_as_uint(m));
}

template <int CPT, int NBUF, bool RMS, bool RAWIDX, int MAXT, int MINB>
int launch_variant(const QuantParams& p, int nt, size_t smem, const DeviceInfo& di, cudaStream_t stream) {
  auto kern = arcq_quantize_kernel<CPT, NBUF, RMS, RAWIDX, MAXT, MINB>;
  ARCQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int occ = 0;
  ARCQ_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, nt, smem));
  if (occ < 1) return ARCQ_ERR_UNSUPPORTED_K;
  long long grid = (long long)di.num_sms * occ;
  if (grid > p.npairs) grid = p.npairs;
  kern<<<(unsigned)grid, nt, smem, stream>>>(p);
  ARCQ_CUDA_TRY(cudaGetLastError());
  return ARCQ_OK;
}

}  // namespace

int launch_quantize(const void* x, const void* gamma, float eps, const int16_t* idx, int64_t rows, int KQ,
                    int KE, int mode, int is_weight, uint8_t* q, uint8_t* sf, cudaStream_t stream) {
  if (rows == 0) return ARCQ_OK;
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

  const bool rms = gamma != nullptr;
  const size_t table = ((size_t)KQ * 2 + 15) & ~(size_t)15;
  int nt, cpt, nbuf;
  if (rms) {
    nt = p.G;  // one reference thread per CUDA thread: keeps the accumulation order
    cpt = 2;
    nbuf = 2;
  } else {
    int gpt = (p.G + 511) / 512;
    nt = (((p.G + gpt - 1) / gpt) + 31) / 32 * 32;
    int need = (p.nchunks + nt - 1) / nt;
    cpt = need <= 2 ? 2 : (need <= 4 ? 4 : 8);
    nbuf = 2;
    if (need > 8) return ARCQ_ERR_UNSUPPORTED_K;
  }
  const bool rawidx = KQ > 16384;
  size_t smem = table + (rms ? table + (size_t)2 * nt * sizeof(float) + 16 : 0) + (size_t)nbuf * KQ * 4;
  if (cpt == 8 || rawidx || smem > (size_t)di.max_smem_optin) {
    nbuf = 1;
    cpt = 8;
    smem = table + (size_t)KQ * 4;
    if (rms || smem > (size_t)di.max_smem_optin) return ARCQ_ERR_UNSUPPORTED_K;
    return rawidx ? launch_variant<8, 1, false, true, 512, 1>(p, nt, smem, di, stream)
                  : launch_variant<8, 1, false, false, 512, 1>(p, nt, smem, di, stream);
  }
  if (nt <= 256) {
    // narrow rows: three resident CTAs per SM keep enough loads in flight
    if (rms) return launch_variant<2, 2, true, false, 256, 3>(p, nt, smem, di, stream);
    if (cpt == 2) return launch_variant<2, 2, false, false, 256, 3>(p, nt, smem, di, stream);
  }
  if (rms) return launch_variant<2, 2, true, false, 512, 1>(p, nt, smem, di, stream);
  if (cpt == 2) return launch_variant<2, 2, false, false, 512, 1>(p, nt, smem, di, stream);
  return launch_variant<4, 2, false, false, 512, 1>(p, nt, smem, di, stream);
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
