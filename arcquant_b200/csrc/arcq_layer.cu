// Element-wise pieces of a decoder layer that sit between the quantized linears: rotary position
// embedding applied in place to the q and k columns of the fused qkv output, and SiLU(gate) * up with
// the per-tensor max|.| of the result (which the next activation quantizer needs) taken in the same
// pass.  The reference's layers call torch for these (model/qLlamaLayer.py of ARCQuant uses the
// Hugging Face `apply_rotary_pos_emb` and `act_fn(gate) * up`); the arithmetic below reproduces the
// eager torch results bit for bit: every product and sum is rounded to fp32 separately, the same
// `expf` and IEEE division, bf16 rounding after SiLU and after the product.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <math.h>
#include <stdlib.h>

#include <atomic>
#include <mutex>

#include "arcq_internal.h"

namespace arcq {
namespace {

__device__ __forceinline__ float lo_f(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float hi_f(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// x: [tokens, row_elems] bf16; the first `heads` heads of `dim` elements of each row are rotated:
// out[d] = x[d] * cos[d] - x[d + dim/2] * sin[d],  out[d + dim/2] = x[d + dim/2] * cos[..] + x[d] * sin[..]
// (rotate-half convention), cos/sin: [seq, dim] fp32 indexed by token % seq.  One thread = 8 + 8 elements.
__global__ void arcq_rope_kernel(uint16_t* __restrict__ x, const float* __restrict__ cs, const float* __restrict__ sn,
                                 long long tokens, int row_elems, int heads, int dim, int seq) {
  const int half = dim >> 1, per_head = half >> 3;
  const long long total = tokens * heads * per_head;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int d8 = (int)(i % per_head);
    const long long th = i / per_head;
    const int h = (int)(th % heads);
    const long long t = th / heads;
    const int pos = (int)(t % seq);
    uint16_t* base = x + t * row_elems + (long long)h * dim + d8 * 8;
    const uint4 a = *reinterpret_cast<const uint4*>(base), b = *reinterpret_cast<const uint4*>(base + half);
    const float* c0 = cs + (long long)pos * dim + d8 * 8;
    const float* s0 = sn + (long long)pos * dim + d8 * 8;
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
    uint32_t oa[4], ob[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float ra[2], rb[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float xa = e ? hi_f(aw[k]) : lo_f(aw[k]), xb = e ? hi_f(bw[k]) : lo_f(bw[k]);
        const int d = 2 * k + e;
        // first half: x_a * cos + (-x_b) * sin;  second half: x_b * cos + x_a * sin
        ra[e] = __fadd_rn(__fmul_rn(xa, c0[d]), __fmul_rn(-xb, s0[d]));
        rb[e] = __fadd_rn(__fmul_rn(xb, c0[half + d]), __fmul_rn(xa, s0[half + d]));
      }
      oa[k] = pack2(ra[0], ra[1]);
      ob[k] = pack2(rb[0], rb[1]);
    }
    *reinterpret_cast<uint4*>(base) = make_uint4(oa[0], oa[1], oa[2], oa[3]);
    *reinterpret_cast<uint4*>(base + half) = make_uint4(ob[0], ob[1], ob[2], ob[3]);
  }
}

__device__ __forceinline__ float silu_bf16(float g) {
  const float s = __fdiv_rn(g, __fadd_rn(1.0f, expf(-g)));
  return __uint_as_float(pack2(s, 0.f) << 16);   // rounded to bf16, as torch's bf16 SiLU returns it
}

// gu: [tokens, 2F] bf16 = [gate | up]; out: [tokens, F] bf16 = bf16(bf16(silu(gate)) * up); amax: max |out|.
__global__ void arcq_silu_mul_kernel(const uint16_t* __restrict__ gu, uint16_t* __restrict__ out, long long tokens, int F,
                                     unsigned int* amax) {
  const int vec_per_row = F >> 3;
  const long long total = tokens * vec_per_row;
  uint32_t m = 0;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vec_per_row;
    const int v = (int)(i - t * vec_per_row);
    const uint16_t* row = gu + t * 2LL * F;
    const uint4 g = *reinterpret_cast<const uint4*>(row + v * 8), u = *reinterpret_cast<const uint4*>(row + F + v * 8);
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float a = __fmul_rn(silu_bf16(lo_f(gw[k])), lo_f(uw[k]));
      const float b = __fmul_rn(silu_bf16(hi_f(gw[k])), hi_f(uw[k]));
      o[k] = pack2(a, b);
      uint32_t ab;
      asm("max.u16x2 %0, %1, %2;" : "=r"(ab) : "r"(m), "r"(o[k] & 0x7fff7fffu));
      m = ab;
    }
    *reinterpret_cast<uint4*>(out + t * (long long)F + v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
  }
  if (amax) {
    uint32_t r = max(m & 0xffffu, m >> 16);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) r = max(r, __shfl_xor_sync(0xffffffffu, r, d));
    if ((threadIdx.x & 31) == 0) atomicMax(amax, r << 16);   // non-negative floats order like their bit patterns
  }
}

// Large calls: bf16 SiLU is a function of 65 536 bit patterns, and its exact evaluation (expf, IEEE
// division: ~25 instructions per element) makes the pass above instruction bound at ~0.75 of the HBM
// rate.  g_silu_table holds bf16(silu(g)) for every g, written by arcq_silu_table_kernel with the very
// function above (so the results cannot differ); each CTA of the main kernel copies the 128 KB into
// shared memory and looks SiLU up.
__device__ uint16_t g_silu_table[65536];

__global__ void arcq_silu_table_kernel() {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  g_silu_table[i] = (uint16_t)(__float_as_uint(silu_bf16(__uint_as_float(i << 16))) >> 16);
}

// The table is written once per device: the first call launches the kernel on its own stream and records
// an event, later calls make their stream wait for that event until it has completed (after which the
// table is never touched again, so calls on any number of streams only ever read it).
int ensure_silu_table(int device, cudaStream_t stream) {
  struct State { bool started = false, done = false; cudaEvent_t ev = nullptr; };
  static std::mutex mu;
  static State st[64];
  if (device < 0 || device >= 64) return ARCQ_ERR_CUDA;
  std::lock_guard<std::mutex> lock(mu);
  State& s = st[device];
  if (s.done) return ARCQ_OK;
  if (!s.started) {
    ARCQ_CUDA_TRY(cudaEventCreateWithFlags(&s.ev, cudaEventDisableTiming));
    arcq_silu_table_kernel<<<65536 / 256, 256, 0, stream>>>();
    ARCQ_CUDA_TRY(cudaGetLastError());
    ARCQ_CUDA_TRY(cudaEventRecord(s.ev, stream));
    s.started = true;
    return ARCQ_OK;
  }
  if (cudaEventQuery(s.ev) == cudaSuccess) {
    s.done = true;
    return ARCQ_OK;
  }
  (void)cudaGetLastError();   // (cudaErrorNotReady is not an error)
  ARCQ_CUDA_TRY(cudaStreamWaitEvent(stream, s.ev, 0));
  return ARCQ_OK;
}

__global__ void __launch_bounds__(1024, 1) arcq_silu_mul_table_kernel(const uint16_t* __restrict__ gu, uint16_t* __restrict__ out,
                                                                      long long tokens, int F, unsigned int* amax) {
  extern __shared__ __align__(16) uint16_t tab[];
  {
    const uint4* src = reinterpret_cast<const uint4*>(g_silu_table);
    uint4* dst = reinterpret_cast<uint4*>(tab);
    for (int i = threadIdx.x; i < 65536 / 8; i += blockDim.x) dst[i] = src[i];
  }
  __syncthreads();
  const int vec_per_row = F >> 3;
  const long long total = tokens * vec_per_row;
  const long long step = (long long)gridDim.x * blockDim.x;
  uint32_t m = 0;
  // two vectors per thread and iteration: four 16-byte loads in flight before any is used
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += 2 * step) {
    const long long i1 = i + step;
    const bool two = i1 < total;
    const long long t0 = i / vec_per_row, t1 = two ? i1 / vec_per_row : t0;
    const int v0 = (int)(i - t0 * vec_per_row), v1 = two ? (int)(i1 - t1 * vec_per_row) : v0;
    const uint16_t* r0 = gu + t0 * 2LL * F + v0 * 8;
    const uint16_t* r1 = gu + t1 * 2LL * F + v1 * 8;
    const uint4 g0 = *reinterpret_cast<const uint4*>(r0), u0 = *reinterpret_cast<const uint4*>(r0 + F);
    const uint4 g1 = *reinterpret_cast<const uint4*>(r1), u1 = *reinterpret_cast<const uint4*>(r1 + F);
    auto one = [&](const uint4& g, const uint4& u, long long t, int v) {
      const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
      uint32_t o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float sa = __uint_as_float((uint32_t)tab[gw[k] & 0xffffu] << 16);
        const float sb = __uint_as_float((uint32_t)tab[gw[k] >> 16] << 16);
        o[k] = pack2(__fmul_rn(sa, lo_f(uw[k])), __fmul_rn(sb, hi_f(uw[k])));
        uint32_t ab;
        asm("max.u16x2 %0, %1, %2;" : "=r"(ab) : "r"(m), "r"(o[k] & 0x7fff7fffu));
        m = ab;
      }
      *reinterpret_cast<uint4*>(out + t * (long long)F + v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    };
    one(g0, u0, t0, v0);
    if (two) one(g1, u1, t1, v1);
  }
  if (amax) {
    uint32_t r = max(m & 0xffffu, m >> 16);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) r = max(r, __shfl_xor_sync(0xffffffffu, r, d));
    if ((threadIdx.x & 31) == 0) atomicMax(amax, r << 16);   // non-negative floats order like their bit patterns
  }
}

// SiLU(gate) * up over grouped rows (see arcq_silu_mul_grouped_bf16): tiles of 256 rows without rows are
// skipped, padding rows inside a tile are computed but kept out of the maxima, and amax[e] receives max|out|
// over the rows of run e.  F/8 is a multiple of 32, so the 32 vectors a warp takes per step lie in one row
// and the warp's run is uniform: its running maximum is flushed (one atomic per warp) when the run changes.
template <bool TABLE>
__global__ void __launch_bounds__(1024, 1)
arcq_silu_mul_grouped_kernel(const uint16_t* __restrict__ gu, uint16_t* __restrict__ out, long long rows, int F,
                             const int* __restrict__ tile_group, const int* __restrict__ groups, int ngroups,
                             unsigned int* amax) {
  extern __shared__ __align__(16) uint16_t tab[];
  if (TABLE) {
    const uint4* src = reinterpret_cast<const uint4*>(g_silu_table);
    uint4* dst = reinterpret_cast<uint4*>(tab);
    for (int i = threadIdx.x; i < 65536 / 8; i += blockDim.x) dst[i] = src[i];
    __syncthreads();
  }
  const int vec_per_row = F >> 3;
  const long long total = rows * vec_per_row;
  const long long step = (long long)gridDim.x * blockDim.x;
  uint32_t m = 0;
  int cur = -1;
  auto flush = [&]() {
    if (cur >= 0 && amax != nullptr) {
      uint32_t r = max(m & 0xffffu, m >> 16);
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) r = max(r, __shfl_xor_sync(0xffffffffu, r, d));
      if ((threadIdx.x & 31) == 0 && r) atomicMax(amax + cur, r << 16);
    }
    m = 0;
  };
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += step) {
    const long long t = i / vec_per_row;
    const int v = (int)(i - t * vec_per_row);
    const int e = __ldg(tile_group + (t >> 8));
    if (e < 0) continue;                                   // (warp-uniform)
    if (e != cur) { flush(); cur = e; }
    const bool valid = t < (long long)__ldg(groups + e) + __ldg(groups + ngroups + e);
    const uint16_t* row = gu + t * 2LL * F + v * 8;
    const uint4 g = *reinterpret_cast<const uint4*>(row), u = *reinterpret_cast<const uint4*>(row + F);
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float sa, sb;
      if (TABLE) {
        sa = __uint_as_float((uint32_t)tab[gw[k] & 0xffffu] << 16);
        sb = __uint_as_float((uint32_t)tab[gw[k] >> 16] << 16);
      } else {
        sa = silu_bf16(lo_f(gw[k]));
        sb = silu_bf16(hi_f(gw[k]));
      }
      o[k] = pack2(__fmul_rn(sa, lo_f(uw[k])), __fmul_rn(sb, hi_f(uw[k])));
      if (valid) asm("max.u16x2 %0, %0, %1;" : "+r"(m) : "r"(o[k] & 0x7fff7fffu));
    }
    *reinterpret_cast<uint4*>(out + t * (long long)F + v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
  }
  flush();
}

// out[t] = sum over the k routed copies of token t of bf16(y[pos[t][j]] * w[t][j]), accumulated in the
// output type in the order j = 0..k-1 (a bf16 index_add over the copies adds them in bf16 as well; with
// k = 2 the order does not matter).  One thread = 8 channels of one token.
__global__ void arcq_moe_combine_kernel(const uint16_t* __restrict__ y, const int* __restrict__ pos,
                                        const uint16_t* __restrict__ w, uint16_t* __restrict__ out, long long tokens,
                                        int hidden, int k) {
  const int vec_per_row = hidden >> 3;
  const long long total = tokens * vec_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vec_per_row;
    const int v = (int)(i - t * vec_per_row);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < k; ++j) {
      const long long r = pos[t * k + j];
      const float wj = __uint_as_float((uint32_t)w[t * k + j] << 16);
      const uint4 a = *reinterpret_cast<const uint4*>(y + r * hidden + v * 8);
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        // product rounded to bf16, then a bf16 addition: what `out.index_add_(0, idx, y * w)` computes
        const uint32_t pr = pack2(__fmul_rn(lo_f(aw[q]), wj), __fmul_rn(hi_f(aw[q]), wj));
        const uint32_t sm = pack2(__fadd_rn(acc[2 * q], lo_f(pr)), __fadd_rn(acc[2 * q + 1], hi_f(pr)));
        acc[2 * q] = lo_f(sm);
        acc[2 * q + 1] = hi_f(sm);
      }
    }
    uint4 o;
    o.x = pack2(acc[0], acc[1]); o.y = pack2(acc[2], acc[3]); o.z = pack2(acc[4], acc[5]); o.w = pack2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + t * (long long)hidden + v * 8) = o;
  }
}

// out = residual + bf16(src[0] + src[1] + ... + src[n-1]): the partial results of a row-parallel projection
// added in fp32 in the order of the sources (the same on every rank), rounded to the output type once, then
// the bf16 addition of the residual stream.  The sources are this rank's receive slots (local memory that the
// peers' GEMMs wrote) or, for a caller that pulls, addresses in the peers' memory.  One thread = 8 elements.
struct SumSources {
  const uint4* p[8];
};
__global__ void arcq_sum_partials_kernel(const SumSources src, int n, long long nvec, const uint4* __restrict__ residual,
                                         uint4* __restrict__ out) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
    for (int s = 0; s < n; ++s) {
      const uint4 a = __ldcs(src.p[s] + i);
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        acc[2 * q] = __fadd_rn(acc[2 * q], lo_f(aw[q]));
        acc[2 * q + 1] = __fadd_rn(acc[2 * q + 1], hi_f(aw[q]));
      }
    }
    uint32_t y[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) y[q] = pack2(acc[2 * q], acc[2 * q + 1]);
    if (residual != nullptr) {
      const uint4 r = __ldcs(residual + i);
      const uint32_t rw[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) y[q] = pack2(__fadd_rn(lo_f(rw[q]), lo_f(y[q])), __fadd_rn(hi_f(rw[q]), hi_f(y[q])));
    }
    out[i] = make_uint4(y[0], y[1], y[2], y[3]);
  }
}

// Barrier over the ranks of a tensor-parallel group through flags in peer memory.  Rank r owns a block of
// `world` 32-bit flags; arriving at barrier number e, it writes e into flag [r] of every rank's block and
// waits until all flags of its own block have reached e.  One CTA, thread d talks to rank d.  Everything this
// rank's earlier kernels of the stream wrote (into its own or a peer's memory) is visible to a peer's kernels
// that follow the peer's barrier: the kernel boundary orders those writes before this thread's system-scope
// fence and flag store, the peer's flag load and fence order its later reads after them.
// The wait is bounded: after `limit_ns` the kernel records ARCQ_ERR_TIMEOUT and returns.
struct PeerFlags {
  unsigned int* p[8];
};
__device__ int g_peer_error = 0;   // sticky until polled

__global__ void arcq_peer_barrier_kernel(const PeerFlags f, int rank, int world, unsigned int* counter,
                                         unsigned long long limit_ns) {
  __shared__ unsigned int epoch_s;
  if (threadIdx.x == 0) {
    epoch_s = *counter + 1u;
    *counter = epoch_s;
  }
  __syncthreads();
  const unsigned int epoch = epoch_s;
  const int d = threadIdx.x;
  if (d < world) {
    __threadfence_system();
    *reinterpret_cast<volatile unsigned int*>(f.p[d] + rank) = epoch;
    const volatile unsigned int* in = f.p[rank] + d;
    unsigned long long t0 = 0;
    for (unsigned int it = 0; (int)(*in - epoch) < 0; ++it) {
      if ((it & 255u) == 255u) {
        unsigned long long t1;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
        if (t0 == 0) t0 = t1;
        if (t1 - t0 > limit_ns) {
          atomicExch(&g_peer_error, ARCQ_ERR_TIMEOUT);
          break;
        }
      }
    }
    __threadfence_system();
  }
}

// Per-run max|x| of grouped rows: run e holds rows [groups[e], groups[e] + groups[ngroups + e]) of the
// (padded) row numbering; row r of that numbering is input row row_map[r] (or r).  One warp per row.
__global__ void arcq_absmax_grouped_kernel(const uint16_t* __restrict__ x, const int* __restrict__ row_map,
                                           const int* __restrict__ groups, int ngroups, int K, unsigned int* out) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int last = __ldg(groups + ngroups - 1) + __ldg(groups + 2 * ngroups - 1);   // end of the last run
  int e = 0;
  for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < last; r += warps) {
    while (e + 1 < ngroups && r >= __ldg(groups + e + 1)) ++e;
    if (r >= __ldg(groups + e) + __ldg(groups + ngroups + e)) continue;        // padding between runs
    const uint4* row = reinterpret_cast<const uint4*>(x + (size_t)(row_map ? __ldg(row_map + r) : r) * (size_t)K);
    uint32_t m = 0;
    for (int v = lane; v < (K >> 3); v += 32) {
      const uint4 a = __ldg(row + v);
      asm("max.u16x2 %0, %0, %1;" : "+r"(m) : "r"(a.x & 0x7fff7fffu));
      asm("max.u16x2 %0, %0, %1;" : "+r"(m) : "r"(a.y & 0x7fff7fffu));
      asm("max.u16x2 %0, %0, %1;" : "+r"(m) : "r"(a.z & 0x7fff7fffu));
      asm("max.u16x2 %0, %0, %1;" : "+r"(m) : "r"(a.w & 0x7fff7fffu));
    }
    uint32_t v = max(m & 0xffffu, m >> 16);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, d));
    if (lane == 0) atomicMax(out + e, v << 16);   // non-negative floats order like their bit patterns
  }
}

// Padded layout of routed rows, one CTA: slot i belongs to run slot_group[i] (or to nobody if that is >=
// ngroups); the runs follow one another, each starting at a multiple of `tile` rows, slots of one run in
// their original order.  dest[i] = padded row of slot i (rows_bound for nobody), row_map[r] = i / div for
// the padded row r that holds slot i (0 for padding), groups = [first row of every run | rows of every
// run], tile_group[m] = run of tile m or -1.
__global__ void __launch_bounds__(1024, 1)
arcq_moe_layout_kernel(const long long* __restrict__ slot_group, int n, int ngroups, int tile, int rows_bound, int div,
                       int* __restrict__ dest, int* __restrict__ row_map, int* __restrict__ groups,
                       int* __restrict__ tile_group) {
  __shared__ int s_cnt[64], s_off[64], s_warp[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int per = (n + 1023) >> 10;
  const int lo = min(n, tid * per), hi = min(n, lo + per);
  for (int r = tid; r < rows_bound; r += 1024) row_map[r] = 0;
  // this thread's matches of run e, and the number of matches in all earlier threads (exclusive scan)
  auto scan = [&](int e, int& mine, int& before, int& total) {
    mine = 0;
    for (int i = lo; i < hi; ++i) mine += (slot_group[i] == (long long)e) ? 1 : 0;
    int inc = mine;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, inc, d);
      if (lane >= d) inc += v;
    }
    if (lane == 31) s_warp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
      int w = s_warp[lane], winc = w;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, winc, d);
        if (lane >= d) winc += v;
      }
      s_warp[lane] = winc - w;                         // matches in earlier warps
      if (lane == 31) s_cnt[e] = winc;
    }
    __syncthreads();
    before = s_warp[warp] + inc - mine;
    total = s_cnt[e];
    __syncthreads();                                   // s_warp is reused by the next scan
  };
  int mine, before, total;
  for (int e = 0; e < ngroups; ++e) scan(e, mine, before, total);   // fills s_cnt
  if (tid == 0) {
    int off = 0;
    for (int e = 0; e < ngroups; ++e) {
      s_off[e] = off;
      groups[e] = off;
      groups[ngroups + e] = s_cnt[e];
      off += (s_cnt[e] + tile - 1) / tile * tile;
    }
  }
  __syncthreads();
  for (int e = 0; e < ngroups; ++e) {
    const int off = s_off[e];
    scan(e, mine, before, total);
    int r = off + before;
    for (int i = lo; i < hi; ++i) {
      if (slot_group[i] == (long long)e) {
        dest[i] = r;
        row_map[r] = i / div;
        ++r;
      }
    }
  }
  for (int i = lo; i < hi; ++i)
    if (slot_group[i] < 0 || slot_group[i] >= (long long)ngroups) dest[i] = rows_bound;
  for (int m = tid; m < rows_bound / tile; m += 1024) {
    const int start = m * tile;
    int g = -1;
    for (int e = 0; e < ngroups; ++e)
      if (start >= s_off[e] && start < s_off[e] + s_cnt[e]) g = e;
    tile_group[m] = g;
  }
}

// Expert-parallel dispatch through peer memory, send side, one CTA: copy i of this rank goes to local expert
// ids[i] % e_local of rank d = ids[i] / e_local and takes the next free place j of this rank's block in rank
// d's receive buffer (places in copy order): slot[i] = d * cap + j, and the place's local expert is written
// into rank d's slot table (meta.p[d][rank * cap + j]); places of the block that stay free are marked with
// e_local ("nobody").  Copies beyond a block's capacity are dropped: slot[i] = ep * cap, *overflow set.
struct PeerPtrs {
  void* p[8];
};
__global__ void __launch_bounds__(1024, 1)
arcq_ep_send_layout_kernel(const long long* __restrict__ ids, int n, int e_local, int ep, int cap, int rank,
                           int* __restrict__ slot, const PeerPtrs meta, int* __restrict__ overflow) {
  __shared__ int s_warp[32], s_total;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int per = (n + 1023) >> 10;
  const int lo = min(n, tid * per), hi = min(n, lo + per);
  for (int d = 0; d < ep; ++d) {
    long long* table = static_cast<long long*>(meta.p[d]) + (size_t)rank * cap;
    int mine = 0;
    for (int i = lo; i < hi; ++i) {
      const long long e = ids[i];
      mine += (e >= 0 && e / e_local == d) ? 1 : 0;
    }
    int inc = mine;
#pragma unroll
    for (int k = 1; k < 32; k <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, inc, k);
      if (lane >= k) inc += v;
    }
    if (lane == 31) s_warp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
      int w = s_warp[lane], winc = w;
#pragma unroll
      for (int k = 1; k < 32; k <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, winc, k);
        if (lane >= k) winc += v;
      }
      s_warp[lane] = winc - w;
      if (lane == 31) s_total = winc;
    }
    __syncthreads();
    int r = s_warp[warp] + inc - mine;
    const int total = s_total;
    for (int i = lo; i < hi; ++i) {
      const long long e = ids[i];
      if (e >= 0 && e / e_local == d) {
        if (r < cap) {
          slot[i] = d * cap + r;
          table[r] = e - (long long)d * e_local;
        } else {
          slot[i] = ep * cap;
          *overflow = 1;
        }
        ++r;
      }
    }
    for (int j = min(total, cap) + tid; j < cap; j += 1024) table[j] = e_local;
    __syncthreads();                                   // s_warp / s_total are reused by the next rank
  }
  for (int i = lo; i < hi; ++i)
    if (ids[i] < 0 || ids[i] >= (long long)ep * e_local) slot[i] = ep * cap;
}

// Rows into the peers' buffers, one warp per item: item i reads row (item_src ? item_src[i] : i / div) of src
// (skipped if that is >= src_limit) and writes place rank * cap + s % cap of the buffer of rank s / cap, where
// s = item_slot ? item_slot[i] : i (skipped if s >= ep * cap).  Dispatch: items = routed copies, s = their slot;
// return trip: items = the places of this rank's receive buffer, read through the experts' padded layout.
__global__ void arcq_ep_rows_kernel(const uint4* __restrict__ src, const int* __restrict__ item_src, int div, int src_limit,
                                    const int* __restrict__ item_slot, int n, int row_vec, int cap, int ep, int rank,
                                    const PeerPtrs dst) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < n; i += warps) {
    const int s = item_slot ? __ldg(item_slot + i) : i;
    if (s < 0 || s >= ep * cap) continue;
    const int r = item_src ? __ldg(item_src + i) : i / div;
    if (r < 0 || r >= src_limit) continue;
    const int d = s / cap;
    const uint4* from = src + (size_t)r * row_vec;
    uint4* to = static_cast<uint4*>(dst.p[d]) + ((size_t)rank * cap + (s - d * cap)) * row_vec;
    for (int v = lane; v < row_vec; v += 32) to[v] = __ldg(from + v);
  }
}

// Calibration statistics in one pass over the activations (utilize.py:108 and :546-547 of ARCQuant):
// per-channel running max|x| and the number of elements larger than an eighth of their row's (signed)
// maximum.  A CTA of 256 threads walks rows b, b + grid, ...; thread t owns the 16-byte chunks t, t + 256,
// ... of every row, so its channels' maxima stay in registers and leave with one atomic each at the end.
template <int CPT>
__global__ void __launch_bounds__(256) arcq_calib_stats_kernel(const uint16_t* __restrict__ x, long long rows, int K,
                                                               unsigned int* chan_absmax, unsigned long long* above) {
  __shared__ float s_max[2][8];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nchunks = K >> 3;
  uint32_t cmax[CPT][4];
#pragma unroll
  for (int j = 0; j < CPT; ++j) cmax[j][0] = cmax[j][1] = cmax[j][2] = cmax[j][3] = 0;
  unsigned long long count = 0;
  int buf = 0;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x, buf ^= 1) {
    const uint4* row = reinterpret_cast<const uint4*>(x + r * (long long)K);
    uint4 v[CPT];
    float m = -INFINITY;
#pragma unroll
    for (int j = 0; j < CPT; ++j) {
      const int c = tid + j * 256;
      v[j] = c < nchunks ? __ldg(row + c) : make_uint4(0xff80ff80u, 0xff80ff80u, 0xff80ff80u, 0xff80ff80u);   // -inf
      const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        m = fmaxf(m, fmaxf(lo_f(w[k]), hi_f(w[k])));
        if (c < nchunks) asm("max.u16x2 %0, %0, %1;" : "+r"(cmax[j][k]) : "r"(w[k] & 0x7fff7fffu));
      }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
    if (lane == 0) s_max[buf][warp] = m;
    __syncthreads();
    float rm = s_max[buf][0];
#pragma unroll
    for (int k = 1; k < 8; ++k) rm = fmaxf(rm, s_max[buf][k]);
    // the threshold in the tensor's own type, as torch computes `max * 0.125` on a bf16 tensor
    const float thr = __uint_as_float(pack2(__fmul_rn(rm, 0.125f), 0.f) << 16);
#pragma unroll
    for (int j = 0; j < CPT; ++j) {
      if (tid + j * 256 < nchunks) {
        const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) count += (lo_f(w[k]) > thr ? 1 : 0) + (hi_f(w[k]) > thr ? 1 : 0);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < CPT; ++j) {
    const int c = tid + j * 256;
    if (c < nchunks) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        atomicMax(chan_absmax + 8 * c + 2 * k, (cmax[j][k] & 0xffffu) << 16);
        atomicMax(chan_absmax + 8 * c + 2 * k + 1, cmax[j][k] & 0xffff0000u);
      }
    }
  }
  if (above != nullptr) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) count += __shfl_xor_sync(0xffffffffu, count, d);
    if (lane == 0 && count) atomicAdd(above, count);
  }
}

}  // namespace

int launch_calib_stats(const void* x, int64_t rows, int K, float* chan_absmax, unsigned long long* above,
                       cudaStream_t stream) {
  if (rows == 0) return ARCQ_OK;
  DeviceInfo di;
  int rc = get_device_info(&di);
  if (rc != ARCQ_OK) return rc;
  long long grid = (long long)di.num_sms * 8;
  if (grid > rows) grid = rows;
  const int cpt = (K / 8 + 255) / 256;
  auto xs = static_cast<const uint16_t*>(x);
  auto cm = reinterpret_cast<unsigned int*>(chan_absmax);
#define ARCQ_CALIB(CPT_) arcq_calib_stats_kernel<CPT_><<<(unsigned)grid, 256, 0, stream>>>(xs, rows, K, cm, above)
  if (cpt <= 1) ARCQ_CALIB(1);
  else if (cpt <= 2) ARCQ_CALIB(2);
  else if (cpt <= 4) ARCQ_CALIB(4);
  else if (cpt <= 8) ARCQ_CALIB(8);
  else if (cpt <= 16) ARCQ_CALIB(16);
  else return ARCQ_ERR_UNSUPPORTED_K;
#undef ARCQ_CALIB
  ARCQ_CUDA_TRY(cudaGetLastError());
  return ARCQ_OK;
}

int launch_ep_send_layout(const long long* ids, int n, int e_local, int ep, int cap, int rank, int* slot,
                          void* const* meta, int* overflow, cudaStream_t stream) {
  PeerPtrs m = {};
  for (int d = 0; d < ep; ++d) m.p[d] = meta[d];
  arcq_ep_send_layout_kernel<<<1, 1024, 0, stream>>>(ids, n, e_local, ep, cap, rank, slot, m, overflow);
  ARCQ_CUDA_TRY(cudaGetLastError());
  return ARCQ_OK;
}

int launch_ep_rows(const void* src, const int* item_src, int div, int src_limit, const int* item_slot, int n, int row_bytes,
                   int cap, int ep, int rank, void* const* dst, cudaStream_t stream) {
  if (n == 0) return ARCQ_OK;
  DeviceInfo di;
  int rc = get_device_info(&di);
  if (rc != ARCQ_OK) return rc;
  PeerPtrs b = {};
  for (int d = 0; d < ep; ++d) b.p[d] = dst[d];
  long long blocks = ((long long)n + 7) / 8;              // eight warps (rows) per CTA
  const long long capb = (long long)di.num_sms * 8;
  if (blocks > capb) blocks = capb;
  arcq_ep_rows_kernel<<<(unsigned)blocks, 256, 0, stream>>>(static_cast<const uint4*>(src), item_src, div, src_limit,
                                                           item_slot, n, row_bytes / 16, cap, ep, rank, b);
  ARCQ_CUDA_TRY(cudaGetLastError());
  return ARCQ_OK;
}

int launch_moe_layout(const long long* slot_group, int n, int ngroups, int tile, int rows_bound, int div, int* dest,
                      int* row_map, int* groups, int* tile_group, cudaStream_t stream) {
  arcq_moe_layout_kernel<<<1, 1024, 0, stream>>>(slot_group, n, ngroups, tile, rows_bound, div, dest, row_map, groups,
                                                 tile_group);
  ARCQ_CUDA_TRY(cudaGetLastError());
  return ARCQ_OK;
}

int launch_absmax_grouped(const void* x, const int* row_map, const int* groups, int ngroups, int K, float* out,
                          cudaStream_t stream) {
  ARCQ_CUDA_TRY(cudaMemsetAsync(out, 0, sizeof(float) * ngroups, stream));
  DeviceInfo di;
  int rc = get_device_info(&di);
  if (rc != ARCQ_OK) return rc;
  arcq_absmax_grouped_kernel<<<(unsigned)di.num_sms * 8, 256, 0, stream>>>(
      static_cast<const uint16_t*>(x), row_map, groups, ngroups, K, reinterpret_cast<unsigned int*>(out));
  ARCQ_CUDA_TRY(cudaGetLastError());
  return ARCQ_OK;
}

int launch_moe_combine(const void* y, const int* pos, const void* w, void* out, int64_t tokens, int hidden, int k,
                       cudaStream_t stream) {
  if (tokens == 0) return ARCQ_OK;
  DeviceInfo di;
  int rc = get_device_info(&di);
  if (rc != ARCQ_OK) return rc;
  const long long total = (long long)tokens * (hidden / 8);
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)di.num_sms * 16;
  if (blocks > cap) blocks = cap;
  arcq_moe_combine_kernel<<<(unsigned)blocks, 256, 0, stream>>>(static_cast<const uint16_t*>(y), pos,
                                                                static_cast<const uint16_t*>(w),
                                                                static_cast<uint16_t*>(out), tokens, hidden, k);
  ARCQ_CUDA_TRY(cudaGetLastError());
  return ARCQ_OK;
}

static std::atomic<long long> g_peer_wait_limit_ms{10000};

int peer_set_wait_limit_ms(int ms) {
  return (int)g_peer_wait_limit_ms.exchange(ms < 1 ? 1 : ms);
}

int launch_peer_barrier(void* const* flags, int rank, int world, unsigned int* counter, cudaStream_t stream) {
  PeerFlags f = {};
  for (int d = 0; d < world; ++d) f.p[d] = static_cast<unsigned int*>(flags[d]);
  arcq_peer_barrier_kernel<<<1, 32, 0, stream>>>(f, rank, world, counter,
                                                 (unsigned long long)g_peer_wait_limit_ms.load() * 1000000ull);
  ARCQ_CUDA_TRY(cudaGetLastError());
  return ARCQ_OK;
}

int peer_poll_error() {
  int v = 0, zero = 0;
  ARCQ_CUDA_TRY(cudaDeviceSynchronize());
  ARCQ_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_peer_error, sizeof(int)));
  if (v) ARCQ_CUDA_TRY(cudaMemcpyToSymbol(g_peer_error, &zero, sizeof(int)));
  return v;
}

int launch_sum_partials(const void* const* srcs, int n, int64_t elems, const void* residual, void* out,
                        cudaStream_t stream) {
  if (elems == 0) return ARCQ_OK;
  DeviceInfo di;
  int rc = get_device_info(&di);
  if (rc != ARCQ_OK) return rc;
  SumSources src = {};
  for (int s = 0; s < n; ++s) src.p[s] = static_cast<const uint4*>(srcs[s]);
  const long long nvec = elems / 8;
  long long blocks = (nvec + 255) / 256;
  const long long cap = (long long)di.num_sms * 16;
  if (blocks > cap) blocks = cap;
  arcq_sum_partials_kernel<<<(unsigned)blocks, 256, 0, stream>>>(src, n, nvec, static_cast<const uint4*>(residual),
                                                                static_cast<uint4*>(out));
  ARCQ_CUDA_TRY(cudaGetLastError());
  return ARCQ_OK;
}

int launch_rope(void* x, const float* cos_t, const float* sin_t, int64_t tokens, int row_elems, int heads, int dim,
                int seq, cudaStream_t stream) {
  if (tokens == 0 || heads == 0) return ARCQ_OK;
  DeviceInfo di;
  int rc = get_device_info(&di);
  if (rc != ARCQ_OK) return rc;
  const long long total = (long long)tokens * heads * (dim / 16);
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)di.num_sms * 16;
  if (blocks > cap) blocks = cap;
  arcq_rope_kernel<<<(unsigned)blocks, 256, 0, stream>>>(static_cast<uint16_t*>(x), cos_t, sin_t, tokens, row_elems, heads,
                                                         dim, seq);
  ARCQ_CUDA_TRY(cudaGetLastError());
  return ARCQ_OK;
}

int silu_table_ptr(cudaStream_t stream, const uint16_t** out) {
  DeviceInfo di;
  int rc = get_device_info(&di);
  if (rc != ARCQ_OK) return rc;
  rc = ensure_silu_table(di.device, stream);
  if (rc != ARCQ_OK) return rc;
  static std::mutex mu;
  static const uint16_t* addr[64] = {};
  std::lock_guard<std::mutex> lock(mu);
  if (addr[di.device] == nullptr) {
    void* ptr = nullptr;
    ARCQ_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_silu_table));   // with that device current
    addr[di.device] = static_cast<const uint16_t*>(ptr);
  }
  *out = addr[di.device];
  return ARCQ_OK;
}

int launch_silu_mul_grouped(const void* gu, void* out, int64_t rows, int F, const int* tile_group, const int* groups,
                            int ngroups, float* amax, cudaStream_t stream) {
  if (amax) ARCQ_CUDA_TRY(cudaMemsetAsync(amax, 0, sizeof(float) * ngroups, stream));
  if (rows == 0) return ARCQ_OK;
  DeviceInfo di;
  int rc = get_device_info(&di);
  if (rc != ARCQ_OK) return rc;
  const long long total = (long long)rows * (F / 8);
  auto g = static_cast<const uint16_t*>(gu);
  auto o = static_cast<uint16_t*>(out);
  auto am = reinterpret_cast<unsigned int*>(amax);
  if (total >= (1LL << 21) && di.max_smem_optin >= 131072) {
    rc = ensure_silu_table(di.device, stream);
    if (rc != ARCQ_OK) return rc;
    auto kern = arcq_silu_mul_grouped_kernel<true>;
    static thread_local int attr_dev = -1;
    if (attr_dev != di.device) {
      ARCQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 131072));
      attr_dev = di.device;
    }
    kern<<<(unsigned)di.num_sms, 1024, 131072, stream>>>(g, o, rows, F, tile_group, groups, ngroups, am);
  } else {
    long long blocks = (total + 1023) / 1024;
    if (blocks > (long long)di.num_sms * 2) blocks = (long long)di.num_sms * 2;
    arcq_silu_mul_grouped_kernel<false><<<(unsigned)blocks, 1024, 0, stream>>>(g, o, rows, F, tile_group, groups, ngroups, am);
  }
  ARCQ_CUDA_TRY(cudaGetLastError());
  return ARCQ_OK;
}

int launch_silu_mul(const void* gu, void* out, int64_t tokens, int F, float* amax, cudaStream_t stream) {
  if (amax) ARCQ_CUDA_TRY(cudaMemsetAsync(amax, 0, sizeof(float), stream));
  if (tokens == 0) return ARCQ_OK;
  DeviceInfo di;
  int rc = get_device_info(&di);
  if (rc != ARCQ_OK) return rc;
  const long long total = (long long)tokens * (F / 8);
  if (total >= (1LL << 22) && di.max_smem_optin >= 131072) {   // 32 M elements and more: table lookups
    rc = ensure_silu_table(di.device, stream);
    if (rc != ARCQ_OK) return rc;
    auto kern = arcq_silu_mul_table_kernel;
    static thread_local int attr_dev = -1;
    if (attr_dev != di.device) {
      ARCQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 131072));
      attr_dev = di.device;
    }
    kern<<<(unsigned)di.num_sms, 1024, 131072, stream>>>(static_cast<const uint16_t*>(gu), static_cast<uint16_t*>(out),
                                                        tokens, F, reinterpret_cast<unsigned int*>(amax));
    ARCQ_CUDA_TRY(cudaGetLastError());
    return ARCQ_OK;
  }
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)di.num_sms * 16;
  if (blocks > cap) blocks = cap;
  arcq_silu_mul_kernel<<<(unsigned)blocks, 256, 0, stream>>>(static_cast<const uint16_t*>(gu), static_cast<uint16_t*>(out),
                                                             tokens, F, reinterpret_cast<unsigned int*>(amax));
  ARCQ_CUDA_TRY(cudaGetLastError());
  return ARCQ_OK;
}

}  // namespace arcq
