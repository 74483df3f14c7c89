// Block-scaled NVFP4 GEMM for sm_100a:  C[M,N] = bf16(alpha * (A.SFA)(B.SFB)^T), fp32 accumulation
// in tensor memory.  A [M,K/2] and B [N,K/2] hold packed e2m1 codes (K-major, two per byte), SFA/SFB
// hold one ue4m3 scale per 16 elements in 512-byte atoms of 128 rows x 4 scale columns - exactly
// what one 128-row, K=64 tcgen05 block-scaled MMA consumes, so an atom travels
// global -> shared (bulk copy) -> tensor memory (tcgen05.cp) without being touched by a thread.
//
// Organisation (one CTA per SM, persistent over output tiles of 128 x BN):
//   warp 0    producer: per K stage (256 elements = one 128-byte swizzled row) two tiled TMA loads
//             (A box 128 rows, B box BN rows, 128B swizzle) and the bulk copies of the scale atoms,
//             all completing on the stage's "full" mbarrier
//   warp 1    tensor-core issuer: one thread copies the stage's scale atoms into TMEM and issues
//             four tcgen05.mma.kind::mxf4nvf4.block_scale (M128 x BN x K64) per stage;
//             tcgen05.commit releases the stage ("empty") and finally publishes the accumulator
//   warps 2-5 epilogue: tcgen05.ld 32 lanes x 32 columns, scale by alpha, convert to bf16, 64-byte
//             contiguous global stores per thread; then hand the accumulator back
// Replaces the CUTLASS sm_120 instantiation of kernels/src/nvfp4.cu in ARCQuant.
//
// Every wait on an mbarrier is bounded: after ~2 s without progress the waiting thread raises a
// CTA-wide abort flag, records ARCQ_ERR_TIMEOUT in a device word the host can poll, and all roles
// fall through to the common exit, where tensor memory is released.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "arcq_internal.h"

namespace arcq {
namespace {

constexpr int BM = 128;            // rows of A per tile (MMA M)
constexpr int BK_BYTES = 128;      // bytes of packed codes per row per stage (256 elements)
constexpr int KSTEPS = 4;          // MMAs (K=64 each) per stage
constexpr int ATOM = 512;          // bytes of one scale atom
constexpr int NUM_THREADS = 192;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;

__device__ int g_gemm_error = 0;   // sticky until polled

template <int BN>
struct Cfg {
  static constexpr int NB = BN > 128 ? BN / 128 : 1;           // scale atoms of B per K step
  static constexpr int A_BYTES = BM * BK_BYTES;                // 16 KB
  static constexpr int B_BYTES = BN * BK_BYTES;
  static constexpr int SFA_BYTES = KSTEPS * ATOM;              // 2 KB
  static constexpr int SFB_BYTES = NB * KSTEPS * ATOM;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : (BN == 128 ? 6 : 7);
  static constexpr int SF_COLS = KSTEPS * 4 + KSTEPS * 4 * NB;  // TMEM columns of one stage's scales
  static constexpr int TMEM_NEED = BN + 2 * SF_COLS;
  static constexpr int TMEM_COLS = TMEM_NEED <= 128 ? 128 : (TMEM_NEED <= 256 ? 256 : 512);
  // 1 KB alignment slack + stages + barriers; at least ~120 KB so that two CTAs never share an SM
  static constexpr int SMEM_RAW = 1024 + STAGES * STAGE_BYTES + 256;
  static constexpr int SMEM_BYTES = SMEM_RAW < 124 * 1024 ? 124 * 1024 : SMEM_RAW;
};

struct GemmParams {
  const uint8_t* sfa;
  const uint8_t* sfb;
  __nv_bfloat16* c;
  const float* alpha_a;
  const float* alpha_b;
  float alpha;
  int M, N;
  int ksteps_total;   // K_eff / 64
  int natoms;         // ceil((K_eff/16)/4): scale atoms per 128-row tile
  int tiles_m, tiles_n;
  int sfb_tiles;      // ceil(N/128): 128-row scale tiles of B that exist
  float* ws;          // split-K: fp32 partial sums [splits][M][N] (scratch), else nullptr
  int splits;         // K is cut into this many ranges of whole stages (1 = no split)
};

// ----------------------------------------------------------------------------- PTX wrappers

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
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
// Bounded wait.  Returns false if the CTA is aborting (this wait or another one timed out).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 255u) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
        *abort_flag = 1;
        atomicExch(&g_gemm_error, ARCQ_ERR_TIMEOUT);
        return false;
      }
    }
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
// The same for data that is read once (an L2 evict-first policy keeps it from displacing the operands).
__device__ __forceinline__ void tma_load_2d_once(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_cp_sf(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void tc_mma_nvf4(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t tsfa, uint32_t tsfb, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %6, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%4], [%5], p;\n}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(tsfa), "r"(tsfb), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor (sm_100 format): start address, leading/stride byte offsets
// (16-byte units), descriptor version 1, swizzle mode.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t sbo_bytes, uint32_t layout_type) {
  uint32_t lo = (saddr >> 4) & 0x3fffu;                      // LBO = 0: one core matrix along K
  uint32_t hi = ((sbo_bytes >> 4) & 0x3fffu) | (1u << 14) | (layout_type << 29);
  return ((uint64_t)hi << 32) | lo;
}
constexpr uint32_t LAYOUT_SW128 = 2, LAYOUT_NONE = 0;

// Instruction descriptor of kind::mxf4nvf4 block-scaled MMA: e2m1 x e2m1 (format id 1), ue4m3
// scales (bit 23 = 0), both operands K-major, N>>3 at bit 17, M>>4 at bit 24, K=64 (bit 31 = 0).
template <int BN>
__device__ __forceinline__ constexpr uint32_t instr_desc() {
  return (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// ----------------------------------------------------------------------------- kernel

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
arcq_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const GemmParams p) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;   // 128B swizzle needs 1 KB alignment
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar_base = base + C::STAGES * C::STAGE_BYTES;
  volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(base_ptr + C::STAGES * C::STAGE_BYTES + 192);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(misc + 1);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (C::STAGES + s); };
  const uint32_t tmem_full_bar = bar_base + 8u * (2 * C::STAGES);
  const uint32_t tmem_empty_bar = tmem_full_bar + 8u;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    mbar_init(tmem_full_bar, 1);
    mbar_init(tmem_empty_bar, 4);
    misc[1] = 0;  // abort flag
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)misc)),
                 "r"((uint32_t)C::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = misc[0];
  const uint32_t tmem_sf = tmem_base + BN;   // two stage-parity buffers of SF_COLS columns each

  // A work item is (output tile, K range).  Without split-K there is one range per tile.
  const int num_tiles = p.tiles_m * p.tiles_n * p.splits;
  const int kstages_all = (p.ksteps_total + KSTEPS - 1) / KSTEPS;
  const int kstages_per = (kstages_all + p.splits - 1) / p.splits;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_tiles && ok; item += gridDim.x) {
        const int tile = item / p.splits, split = item - tile * p.splits;
        const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
        const int rtb = (tn * BN) / 128;   // first 128-row scale tile of B this output tile touches
        const int ks_end = min(kstages_all, (split + 1) * kstages_per);
        for (int ks = split * kstages_per; ks < ks_end; ++ks, ++it) {
          const int s = it % C::STAGES;
          const uint32_t ph = (it / C::STAGES) & 1u;
          if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag)) { ok = false; break; }
          const int nk = min(KSTEPS, p.ksteps_total - ks * KSTEPS);
          const uint32_t sf_bytes = (uint32_t)nk * ATOM;
          const uint32_t st = base + s * C::STAGE_BYTES;
          // scale tiles of B that exist (a 256-wide tile may hang over the last 128-row scale tile)
          int nb_valid = 0;
#pragma unroll
          for (int a = 0; a < C::NB; ++a) nb_valid += (rtb + a) < p.sfb_tiles ? 1 : 0;
          mbar_expect_tx(full_bar(s), C::A_BYTES + C::B_BYTES + sf_bytes * (1 + nb_valid));
          tma_load_2d(st, &map_a, full_bar(s), ks * BK_BYTES, tm * BM);
          tma_load_2d(st + C::A_BYTES, &map_b, full_bar(s), ks * BK_BYTES, tn * BN);
          const uint8_t* sa = p.sfa + ((size_t)tm * p.natoms + (size_t)ks * KSTEPS) * ATOM;
          bulk_load(st + C::A_BYTES + C::B_BYTES, sa, sf_bytes, full_bar(s));
#pragma unroll
          for (int a = 0; a < C::NB; ++a) {
            if ((rtb + a) < p.sfb_tiles) {
              const uint8_t* sb = p.sfb + ((size_t)(rtb + a) * p.natoms + (size_t)ks * KSTEPS) * ATOM;
              bulk_load(st + C::A_BYTES + C::B_BYTES + C::SFA_BYTES + a * (KSTEPS * ATOM), sb, sf_bytes, full_bar(s));
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc<BN>();
      uint32_t it = 0, tile_it = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_tiles && ok; item += gridDim.x, ++tile_it) {
        const int tile = item / p.splits, split = item - tile * p.splits;
        const int tn = tile / p.tiles_m;
        const int ks_begin = split * kstages_per, ks_end = min(kstages_all, (split + 1) * kstages_per);
        // sub-atom column offset when BN = 64: rows 32j..32j+31 of an atom live in TMEM column j, so
        // the upper half of a 128-row scale atom starts two columns in.  (Tiles narrower than 64
        // would need an odd column offset, which the block-scaled MMA rejects as misaligned.)
        const uint32_t sfb_sub = (BN < 128) ? (uint32_t)(((tn * BN) % 128) / 32) : 0u;
        if (!mbar_wait(tmem_empty_bar, (tile_it & 1u) ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        for (int ks = ks_begin; ks < ks_end; ++ks, ++it) {
          const int s = it % C::STAGES;
          const uint32_t ph = (it / C::STAGES) & 1u;
          if (!mbar_wait(full_bar(s), ph, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const int nk = min(KSTEPS, p.ksteps_total - ks * KSTEPS);
          const uint32_t st = base + s * C::STAGE_BYTES;
          const uint32_t a_s = st, b_s = st + C::A_BYTES;
          const uint32_t sfa_s = b_s + C::B_BYTES, sfb_s = sfa_s + C::SFA_BYTES;
          const uint32_t t_sfa = tmem_sf + (it & 1u) * C::SF_COLS;
          const uint32_t t_sfb = t_sfa + KSTEPS * 4;
          for (int k = 0; k < nk; ++k) {
            tc_cp_sf(t_sfa + k * 4, smem_desc(sfa_s + k * ATOM, 128, LAYOUT_NONE));
#pragma unroll
            for (int a = 0; a < C::NB; ++a)
              tc_cp_sf(t_sfb + k * 4 * C::NB + a * 4,
                       smem_desc(sfb_s + a * (KSTEPS * ATOM) + k * ATOM, 128, LAYOUT_NONE));
          }
          for (int k = 0; k < nk; ++k) {
            const uint64_t adesc = smem_desc(a_s + k * 32, 1024, LAYOUT_SW128);
            const uint64_t bdesc = smem_desc(b_s + k * 32, 1024, LAYOUT_SW128);
            tc_mma_nvf4(tmem_base, adesc, bdesc, idesc, t_sfa + k * 4, t_sfb + k * 4 * C::NB + sfb_sub,
                        ((ks - ks_begin) | k) ? 1u : 0u);
          }
          tc_commit(empty_bar(s));   // stage reusable once these MMAs have read it
        }
        if (ok) tc_commit(tmem_full_bar);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;       // TMEM lanes 32*quad .. 32*quad+31 belong to this warp
    float alpha = p.alpha;
    if (p.alpha_a) alpha *= __ldg(p.alpha_a);
    if (p.alpha_b) alpha *= __ldg(p.alpha_b);
    uint32_t tile_it = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < num_tiles && ok; item += gridDim.x, ++tile_it) {
      const int tile = item / p.splits, split = item - tile * p.splits;
      const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
      ok = mbar_wait(tmem_full_bar, tile_it & 1u, abort_flag);
      ok = __all_sync(0xffffffffu, ok);   // keep the warp converged for the .sync.aligned loads
      if (!ok) break;
      tc_fence_after();
      const int row = tm * BM + quad * 32 + lane;
      __nv_bfloat16* crow = p.c + (size_t)row * p.N;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tc_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, r);
        tc_wait_ld();
        const int col = tn * BN + c0;
        if (p.ws != nullptr) {
          // split-K: raw fp32 partial sums of this K range; the reduction kernel applies alpha
          if (row < p.M && col < p.N) {
            float* wrow = p.ws + ((size_t)split * p.M + row) * p.N + col;
#pragma unroll
            for (int v = 0; v < 8; ++v)
              if (col + v * 4 < p.N)   // N is a multiple of 8, so groups of four are in or out
                *reinterpret_cast<uint4*>(wrow + v * 4) = make_uint4(r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
          }
        } else if (row < p.M && col < p.N) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            if (col + v * 8 < p.N) {   // N is a multiple of 8: whole 16-byte pieces are in or out
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r[v * 8 + 0]) * alpha, __uint_as_float(r[v * 8 + 1]) * alpha);
              o.y = pack_bf16x2(__uint_as_float(r[v * 8 + 2]) * alpha, __uint_as_float(r[v * 8 + 3]) * alpha);
              o.z = pack_bf16x2(__uint_as_float(r[v * 8 + 4]) * alpha, __uint_as_float(r[v * 8 + 5]) * alpha);
              o.w = pack_bf16x2(__uint_as_float(r[v * 8 + 6]) * alpha, __uint_as_float(r[v * 8 + 7]) * alpha);
              *reinterpret_cast<uint4*>(crow + col + v * 8) = o;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty_bar);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)C::TMEM_COLS)
                 : "memory");
  }
}

// ----------------------------------------------------------------------------- 2-CTA kernel
//
// Same dataflow on a pair of SMs (cluster of two CTAs, cta_group::2): the pair owns a 256 x 256
// output tile.  Each CTA loads its own 128 rows of A, its own 128 rows of B (half of N), its own
// scale atoms of A and all scale atoms of B; the even CTA (leader) issues one
// tcgen05.mma.cta_group::2 (M256 x N256 x K64) per K step, which reads A from both CTAs' shared
// memory, the two halves of B likewise, and accumulates 128 rows x 256 columns in each CTA's TMEM.
// Per SM this is 9.5 KB of operands per K step instead of 13.5 KB, and the smaller stage
// (38 KB) lets five stages fit.
//
// Scale factors do not go through tcgen05.cp here: measured on this kernel, the twelve copies of
// a stage execute strictly in sequence with its MMAs in the tensor pipe and cost as much as the
// MMAs themselves.  Instead four "scale" warps per CTA (one per TMEM lane quadrant) read the
// stage's atoms from shared memory and write them to TMEM with tcgen05.st, off the tensor pipe,
// one stage ahead of the MMAs; each stage owns its own 48 TMEM columns.
//
// Synchronisation: A/B loads of either CTA complete on the LEADER's "full" barrier
// (.cta_group::2 form; the barrier address is the CTA-local one with the pair's rank bit cleared);
// scale loads complete on a CTA-local barrier; the scale warps of both CTAs arrive on the leader's
// "scales ready" barrier; tcgen05.commit with a two-CTA mask releases the stage in both CTAs and
// publishes the accumulator to both epilogues; the epilogue warps of both CTAs arrive on the
// leader's "accumulator free" barrier.  No load uses cluster multicast.

constexpr int C2_STAGES = 5;
constexpr int C2_THREADS = 320;                     // producer, MMA, 4 epilogue, 4 scale warps
constexpr int C2_A_BYTES = 128 * BK_BYTES;          // 16 KB
constexpr int C2_B_BYTES = 128 * BK_BYTES;          // 16 KB: this CTA's half of the 256 B rows
constexpr int C2_SFA_BYTES = KSTEPS * ATOM;         // 2 KB
constexpr int C2_SFB_BYTES = 2 * KSTEPS * ATOM;     // 4 KB: both 128-row scale tiles of B
constexpr int C2_STAGE_BYTES = C2_A_BYTES + C2_B_BYTES + C2_SFA_BYTES + C2_SFB_BYTES;   // 38 KB
constexpr int C2_SF_COLS = KSTEPS * 4 + KSTEPS * 8;  // 48 TMEM columns of scales per stage
constexpr int C2_TMEM_COLS = 512;                    // 256 accumulator + 5 x 48 scale columns
constexpr int C2_CSTAGE_BYTES = 4 * 8192;             // output staging: 32 rows x 128 columns of bf16 per epilogue warp
constexpr int C2_SMEM_BYTES = 1024 + C2_STAGES * C2_STAGE_BYTES + C2_CSTAGE_BYTES + 256 + 64;   // + residual barriers
constexpr uint32_t PEER_BIT_MASK = 0xFEFFFFFFu;      // clears the pair-rank bit of a shared address

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Tiled TMA load whose completion is counted on the leader CTA's barrier.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t leader_bar, int x,
                                                 int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(leader_bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {   // arrives on `bar` in both CTAs of the pair
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"((uint16_t)3)
      : "memory");
}
__device__ __forceinline__ void tc_mma_nvf4_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                 uint32_t tsfa, uint32_t tsfb, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %6, 0;\n"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%4], [%5], p;\n}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(tsfa), "r"(tsfb), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_leader(uint32_t bar) {   // remote arrive on the leader's barrier
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar & PEER_BIT_MASK) : "memory");
}
// 32 lanes x 16 columns of 32 bits, registers -> this warp's TMEM lane quadrant.
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

struct Gemm2Params {
  __nv_bfloat16* c;
  const float* alpha_a;
  const float* alpha_b;
  float alpha;
  int M, N;
  int ksteps_total;   // K_eff / 64
  int natoms;         // scale atoms per 128-row tile
  int tiles_m, tiles_n;   // 256 x 256 tiles
  int group_m;            // tile rows per band of the tile order (see pair_tile_coords)
  // Grouped problems (one launch over several weight matrices stacked in B): tile_group[tm] = which
  // matrix the 256-row tile tm of A multiplies, or a negative number for a tile that holds no rows
  // (device memory: the host never learns the split).  Matrix g owns rows [g*N, (g+1)*N) of B and of
  // its scales, and alpha_a[g] * alpha_b[g].
  const int* tile_group;
  // SwiGLU epilogue (template flag of the kernel): B holds gate and up columns interleaved in blocks of 128
  // (tile column tn = gate columns [128 tn, 128 tn + 128) then the same up columns), C is [M, N/2] and
  // receives bf16(bf16(silu(gate)) * up) of the bf16-rounded GEMM outputs; amax[g] (bit pattern of a
  // non-negative float) takes max|.| over the valid rows - rows below M, and for grouped problems below the
  // end of their run, groups[g] + groups[ngroups + g].
  unsigned int* amax;
  const int* groups;
  int ngroups;
  const uint16_t* silu_table;   // bf16(silu(g)) for all 65536 bf16 patterns g (device memory, see silu_table_ptr)
  // Scattered output (0 = off): rows [d * rows_per_dest, (d + 1) * rows_per_dest) of the result go to output
  // map d, a [rows_per_dest, N] buffer of its own - in a tensor-parallel group, this rank's slot in the memory
  // of the rank that owns those rows (a peer's memory over NVLink, or local memory).  A multiple of 32: one
  // bulk store carries 32 rows.
  int rows_per_dest;
};

// Output maps of the CTA-pair kernel: one, or one per destination of a scattered output.
constexpr int MAX_DESTS = 8;
struct OutputMaps {
  CUtensorMap m[MAX_DESTS];
};

// Tile order of the persistent pairs: bands of group_m tile rows, and inside a band column by column.
// The ~74 tiles in flight at any time then cover about group_m x (74 / group_m) tiles, so every strip of
// A and of B that is being streamed is shared by several pairs (one column of tiles would share one
// strip of B and nothing of A), and a band's A rows plus all of B stay in L2 while the band lasts.
__device__ __forceinline__ void pair_tile_coords(int tile, const Gemm2Params& p, int& tm, int& tn) {
  const int per_band = p.group_m * p.tiles_n;
  const int band = tile / per_band, in_band = tile - band * per_band;
  const int first = band * p.group_m;
  const int rows = min(p.group_m, p.tiles_m - first);
  tn = in_band / rows;
  tm = first + (in_band - tn * rows);
}

// RESID: the epilogue adds a residual tile (bf16 [M, N], map_r) to the bf16-rounded result before it stores:
// C = bf16(R + bf16(alpha * A B^T)), what a bf16 addition after the GEMM computes.  The tile arrives by TMA in
// the same staging memory the output leaves from (per-thread loads of 32 different rows per instruction would
// hold up the scale warps' shared-memory loads, as per-thread stores did).
template <bool SWIGLU, bool RESID = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(C2_THREADS, 1)
arcq_gemm2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                  const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_sfb,
                  const __grid_constant__ OutputMaps maps_c, const Gemm2Params p,
                  const __grid_constant__ CUtensorMap map_r) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t cstage_base = base + C2_STAGES * C2_STAGE_BYTES;   // 1024-byte aligned (swizzled boxes)
  const uint32_t bar_base = cstage_base + C2_CSTAGE_BYTES;
  volatile uint32_t* misc =
      reinterpret_cast<volatile uint32_t*>(base_ptr + C2_STAGES * C2_STAGE_BYTES + C2_CSTAGE_BYTES + 192);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(misc + 1);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };                       // A/B landed (leader's is used)
  auto empty_bar = [&](int s) { return bar_base + 8u * (C2_STAGES + s); };        // stage reusable
  auto sf_full_bar = [&](int s) { return bar_base + 8u * (2 * C2_STAGES + s); };  // this CTA's scale atoms landed
  auto sf_ready_bar = [&](int s) { return bar_base + 8u * (3 * C2_STAGES + s); }; // scales in TMEM (leader's is used)
  const uint32_t tmem_full_bar = bar_base + 8u * (4 * C2_STAGES);
  const uint32_t tmem_empty_bar = tmem_full_bar + 8u;
  auto resid_bar = [&](int q, int b) { return bar_base + 256u + 8u * (2 * q + b); };   // residual box landed in slot b of epilogue warp q

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();        // 0 = leader (issues the MMAs), 1 = peer
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C2_STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
      mbar_init(sf_full_bar(s), 1);
      mbar_init(sf_ready_bar(s), 8);              // four scale warps in each of the two CTAs
    }
    mbar_init(tmem_full_bar, 1);
    mbar_init(tmem_empty_bar, 8);                 // four epilogue warps in each of the two CTAs
    for (int q = 0; q < 8; ++q) mbar_init(resid_bar(q >> 1, q & 1), 1);
    misc[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)misc)),
                 "r"((uint32_t)C2_TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                             // both CTAs' barriers exist before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = misc[0];
  const uint32_t tmem_sf = tmem_base + 256;       // stage s: scale columns [256 + 48 s, 256 + 48 s + 48)

  const int num_tiles = p.tiles_m * p.tiles_n;
  const int kstages = (p.ksteps_total + KSTEPS - 1) / KSTEPS;
  constexpr uint32_t AB_TX = 2u * (C2_A_BYTES + C2_B_BYTES);   // A/B bytes both CTAs deliver per stage
  constexpr uint32_t SF_TX = C2_SFA_BYTES + C2_SFB_BYTES;      // scale bytes of one CTA per stage

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        int tm, tn;
        pair_tile_coords(tile, p, tm, tn);
        int grp = 0;
        if (p.tile_group != nullptr) { grp = __ldg(p.tile_group + tm); if (grp < 0) continue; }
        const int row_a = tm * 256 + (int)rank * 128;        // this CTA's rows of A (and of the output)
        const int row_b = grp * p.N + tn * 256 + (int)rank * 128;   // this CTA's rows of B (half of the N tile)
        const int sfa_tile = tm * 2 + (int)rank;             // 128-row scale tiles
        const int sfb_tile = grp * (p.N >> 7) + tn * 2;
        for (int ks = 0; ks < kstages; ++ks, ++it) {
          const int s = it % C2_STAGES;
          const uint32_t ph = (it / C2_STAGES) & 1u;
          if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag)) { ok = false; break; }
          const uint32_t st = base + s * C2_STAGE_BYTES;
          const uint32_t lbar = full_bar(s) & PEER_BIT_MASK;
          if (rank == 0) mbar_expect_tx(full_bar(s), AB_TX);
          mbar_expect_tx(sf_full_bar(s), SF_TX);
          // scale atoms first (the scale warps work one hop ahead of the MMAs): rows of the map are
          // atoms (128 words each); one box = the four K atoms of this stage
          tma_load_2d(st + C2_A_BYTES + C2_B_BYTES, &map_sfa, sf_full_bar(s), 0, sfa_tile * p.natoms + ks * KSTEPS);
          tma_load_2d(st + C2_A_BYTES + C2_B_BYTES + C2_SFA_BYTES, &map_sfb, sf_full_bar(s), 0,
                      sfb_tile * p.natoms + ks * KSTEPS);
          tma_load_2d(st + C2_A_BYTES + C2_B_BYTES + C2_SFA_BYTES + KSTEPS * ATOM, &map_sfb, sf_full_bar(s), 0,
                      (sfb_tile + 1) * p.natoms + ks * KSTEPS);
          tma_load_2d_pair(st, &map_a, lbar, ks * BK_BYTES, row_a);
          tma_load_2d_pair(st + C2_A_BYTES, &map_b, lbar, ks * BK_BYTES, row_b);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = (1u << 7) | (1u << 10) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
      uint32_t it = 0, tile_it = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        if (p.tile_group != nullptr) {
          int tm, tn;
          pair_tile_coords(tile, p, tm, tn);
          if (__ldg(p.tile_group + tm) < 0) continue;      // a tile without rows: every role skips it
        }
        if (!mbar_wait(tmem_empty_bar, (tile_it & 1u) ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        for (int ks = 0; ks < kstages; ++ks, ++it) {
          const int s = it % C2_STAGES;
          const uint32_t ph = (it / C2_STAGES) & 1u;
          if (!mbar_wait(sf_ready_bar(s), ph, abort_flag)) { ok = false; break; }
          if (!mbar_wait(full_bar(s), ph, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const int nk = min(KSTEPS, p.ksteps_total - ks * KSTEPS);
          const uint32_t st = base + s * C2_STAGE_BYTES;
          const uint32_t a_s = st, b_s = st + C2_A_BYTES;
          const uint32_t t_sfa = tmem_sf + s * C2_SF_COLS;
          const uint32_t t_sfb = t_sfa + KSTEPS * 4;
          for (int k = 0; k < nk; ++k) {
            const uint64_t adesc = smem_desc(a_s + k * 32, 1024, LAYOUT_SW128);
            const uint64_t bdesc = smem_desc(b_s + k * 32, 1024, LAYOUT_SW128);
            tc_mma_nvf4_pair(tmem_base, adesc, bdesc, idesc, t_sfa + k * 4, t_sfb + k * 8, (ks | k) ? 1u : 0u);
          }
          tc_commit_pair(empty_bar(s));
        }
        if (ok) tc_commit_pair(tmem_full_bar);
        ++tile_it;
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue (both CTAs)
    const int quad = warp & 3;
    float alpha = p.alpha;
    if (p.tile_group == nullptr) {
      if (p.alpha_a) alpha *= __ldg(p.alpha_a);
      if (p.alpha_b) alpha *= __ldg(p.alpha_b);
    }
    uint32_t tile_it = 0, resid_it = 0;
    bool ok = true;
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
      int tm, tn;
      pair_tile_coords(tile, p, tm, tn);
      int grp = 0;
      if (p.tile_group != nullptr) {
        grp = __ldg(p.tile_group + tm);
        if (grp < 0) continue;
        alpha = p.alpha;
        if (p.alpha_a) alpha *= __ldg(p.alpha_a + grp);
        if (p.alpha_b) alpha *= __ldg(p.alpha_b + grp);
      }
      if (RESID) {
        // the first residual box of this tile is fetched while the tile's MMAs are still running
        const int row0r = tm * 256 + (int)rank * 128 + quad * 32;
        if (lane == 0 && row0r < p.M) {
          asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");     // slot 0 is free again
          mbar_expect_tx(resid_bar(quad, 0), 4096u);
          tma_load_2d_once(cstage_base + (uint32_t)quad * 8192u, &map_r, resid_bar(quad, 0), tn * 256, row0r);
        }
      }
      ok = mbar_wait(tmem_full_bar, tile_it & 1u, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = tm * 256 + (int)rank * 128 + quad * 32 + lane;
      // Drain the accumulator into registers as packed bf16 (128 registers for this thread's 256
      // columns) and hand tensor memory back at once: the stores below then overlap the next tile's MMAs.
      uint32_t o[128];
#pragma unroll
      for (int c0 = 0; c0 < 256; c0 += 64) {
        uint32_t r0[32], r1[32];
        tc_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, r0);
        tc_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(c0 + 32), r1);
        tc_wait_ld();
#pragma unroll
        for (int v = 0; v < 16; ++v) {
          o[c0 / 2 + v] = pack_bf16x2(__uint_as_float(r0[2 * v]) * alpha, __uint_as_float(r0[2 * v + 1]) * alpha);
          o[c0 / 2 + 16 + v] = pack_bf16x2(__uint_as_float(r1[2 * v]) * alpha, __uint_as_float(r1[2 * v + 1]) * alpha);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(tmem_empty_bar);
      if (SWIGLU) {
        // columns 0..127 of the tile are gate, 128..255 the matching up columns: out = silu(gate) * up in
        // the gate registers, and its maximum over the rows that hold data
        int row_end = p.M;
        if (p.groups != nullptr) row_end = __ldg(p.groups + grp) + __ldg(p.groups + p.ngroups + grp);
        uint32_t m = 0;
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          // SiLU of a bf16 value is one of 65536 results: looked up (the table stays in L2; evaluating
          // expf and a division 128 times per row made the epilogue slower than the tile's MMAs)
          const uint32_t g = o[j], u = o[64 + j];
          const float sa = __uint_as_float((uint32_t)__ldg(p.silu_table + (g & 0xffffu)) << 16);
          const float sb = __uint_as_float((uint32_t)__ldg(p.silu_table + (g >> 16)) << 16);
          o[j] = pack_bf16x2(sa * __uint_as_float(u << 16), sb * __uint_as_float(u & 0xffff0000u));
          asm("max.u16x2 %0, %0, %1;" : "+r"(m) : "r"(o[j] & 0x7fff7fffu));
        }
        uint32_t v = row < row_end ? max(m & 0xffffu, m >> 16) : 0u;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, d));
        if (lane == 0 && v) atomicMax(p.amax + grp, v << 16);
      }
      const int col0 = SWIGLU ? tn * 128 : tn * 256;
      const int ncols = SWIGLU ? (p.N >> 1) : p.N;
      {
        // Through shared memory: the warp's 32 rows x 256 columns leave as four boxes of 64 columns
        // (32 rows x 128 bytes, 128-byte swizzle: lane = row, 16-byte chunk c of row r sits at chunk
        // c ^ (r & 7), so a warp's 128-bit stores are conflict free), two boxes per round in the
        // warp's 8 KB of staging.  The bulk stores write whole 128-byte lines, clip rows >= M and
        // columns >= N themselves, and keep the load/store pipe free for the scale warps.
        const int row0 = tm * 256 + (int)rank * 128 + quad * 32;
        const uint32_t cst = cstage_base + (uint32_t)quad * 8192u;
        const CUtensorMap* map_c = &maps_c.m[0];
        int row_st = row0;
        if (p.rows_per_dest) {       // these 32 rows belong to one destination
          const int d = row0 / p.rows_per_dest;
          map_c = &maps_c.m[d];
          row_st = row0 - d * p.rows_per_dest;
        }
        if (RESID && row0 < p.M) {
          // Four boxes of 64 columns, two slots: box k is added and stored from slot k & 1 while box k + 1 is
          // on its way into the other slot (box 0 was requested before the accumulator was ready).
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int col = col0 + 64 * k;
            if (col >= ncols) break;
            const uint32_t slot = cst + (uint32_t)(k & 1) * 4096u;
            if (lane == 0 && k + 1 < 4 && col + 64 < ncols) {
              if (k >= 1) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // box k - 1 has left its slot
              mbar_expect_tx(resid_bar(quad, (k + 1) & 1), 4096u);
              tma_load_2d_once(cst + (uint32_t)((k + 1) & 1) * 4096u, &map_r, resid_bar(quad, (k + 1) & 1), col + 64, row0);
            }
            ok = mbar_wait(resid_bar(quad, k & 1), (resid_it >> (k & 1)) & 1u, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            resid_it ^= 1u << (k & 1);      // (bit b: parity of slot b's next box)
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              const int j = 32 * k + 4 * c;
              const uint32_t addr = slot + (uint32_t)lane * 128u + (uint32_t)((c ^ (lane & 7)) << 4);
              uint32_t r0, r1, r2, r3;
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr) : "memory");
              const uint32_t rr[4] = {r0, r1, r2, r3};
              uint32_t out4[4];
#pragma unroll
              for (int e = 0; e < 4; ++e)
                out4[e] = pack_bf16x2(__uint_as_float(rr[e] << 16) + __uint_as_float(o[j + e] << 16),
                                      __uint_as_float(rr[e] & 0xffff0000u) + __uint_as_float(o[j + e] & 0xffff0000u));
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(out4[0]), "r"(out4[1]), "r"(out4[2]),
                           "r"(out4[3])
                           : "memory");
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map_c),
                           "r"(slot), "r"(col), "r"(row_st)
                           : "memory");
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
          }
        } else if (row0 < p.M) {
#pragma unroll
          for (int h = 0; h < (SWIGLU ? 1 : 2); ++h) {
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // staging is free again
            __syncwarp();
#pragma unroll
            for (int bs = 0; bs < 2; ++bs) {
#pragma unroll
              for (int c = 0; c < 8; ++c) {
                const int j = 32 * (2 * h + bs) + 4 * c;
                const uint32_t addr = cst + (uint32_t)bs * 4096u + (uint32_t)lane * 128u + (uint32_t)((c ^ (lane & 7)) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(o[j]), "r"(o[j + 1]),
                             "r"(o[j + 2]), "r"(o[j + 3])
                             : "memory");
              }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
#pragma unroll
              for (int bs = 0; bs < 2; ++bs) {
                const int col = col0 + 64 * (2 * h + bs);
                if (col < ncols)
                  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map_c),
                               "r"(cst + (uint32_t)bs * 4096u), "r"(col), "r"(row_st)
                               : "memory");
              }
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
          }
        }
      }
      ++tile_it;
    }
    // the last boxes must have left shared memory (and reached global memory) before the CTA goes
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ scale warps (both CTAs)
    // Warp q writes TMEM lanes 32q..32q+31.  An atom is 32 rows x 16 bytes: lane l's 16 bytes are
    // its four TMEM columns (rows l, l+32, l+64, l+96 of the 128-row tile, four K blocks each);
    // every quadrant holds the same copy.
    const int quad = warp & 3;
    uint32_t it = 0;
    bool ok = true;
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
      if (p.tile_group != nullptr) {
        int tm, tn;
        pair_tile_coords(tile, p, tm, tn);
        if (__ldg(p.tile_group + tm) < 0) continue;
      }
      for (int ks = 0; ks < kstages; ++ks, ++it) {
        const int s = it % C2_STAGES;
        const uint32_t ph = (it / C2_STAGES) & 1u;
        ok = mbar_wait(sf_full_bar(s), ph, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const uint4* sf = reinterpret_cast<const uint4*>(base_ptr + s * C2_STAGE_BYTES + C2_A_BYTES + C2_B_BYTES);
        const uint32_t taddr = tmem_sf + s * C2_SF_COLS + ((uint32_t)(quad * 32) << 16);
        // TMEM columns: [SFA k0..k3 (4 each)] [SFB k0: tile0, tile1][k1: ...] ...
        // shared:       [SFA k0..k3][SFB tile0 k0..k3][SFB tile1 k0..k3], 512 bytes each
#pragma unroll
        for (int part = 0; part < 3; ++part) {
          uint32_t r[16];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            int atom;
            if (part == 0) atom = j;                                        // SFA k = j
            else {
              const int k = (part - 1) * 2 + (j >> 1), t = j & 1;           // SFB k, tile t
              atom = KSTEPS + t * KSTEPS + k;
            }
            const uint4 v = sf[atom * 32 + lane];
            r[4 * j + 0] = v.x; r[4 * j + 1] = v.y; r[4 * j + 2] = v.z; r[4 * j + 3] = v.w;
          }
          tc_st16(taddr + part * 16, r);
        }
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_leader(sf_ready_bar(s));
      }
    }
  }

  // Neither CTA may leave (or give back tensor memory) while the other can still touch it.
  tc_fence_before();
  __syncthreads();
  __syncwarp();
  cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)C2_TMEM_COLS)
                 : "memory");
  }
}

// Sum of the split-K partials in a fixed order, times alpha, to bf16.  Eight outputs per thread.
__global__ void arcq_splitk_reduce_kernel(const float* __restrict__ ws, int splits, long long mn, float alpha,
                                          const float* alpha_a, const float* alpha_b, __nv_bfloat16* __restrict__ c) {
  if (alpha_a) alpha *= __ldg(alpha_a);
  if (alpha_b) alpha *= __ldg(alpha_b);
  const long long nvec = mn / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < splits; ++s) {
      const float4* src = reinterpret_cast<const float4*>(ws + (size_t)s * mn + i * 8);
      const float4 a = src[0], b = src[1];
      acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
      acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0] * alpha, acc[1] * alpha);
    o.y = pack_bf16x2(acc[2] * alpha, acc[3] * alpha);
    o.z = pack_bf16x2(acc[4] * alpha, acc[5] * alpha);
    o.w = pack_bf16x2(acc[6] * alpha, acc[7] * alpha);
    reinterpret_cast<uint4*>(c)[i] = o;
  }
}

// ----------------------------------------------------------------------------- host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int get_encode_fn(EncodeTiledFn* out) {
  static std::mutex mu;
  static EncodeTiledFn fn = nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    ARCQ_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres));
    if (qres != cudaDriverEntryPointSuccess || !sym) return cuda_fail(cudaErrorNotSupported);
    fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  *out = fn;
  return ARCQ_OK;
}

// Packed-code operand [rows, kbytes] (uint8, row-major) with a box of 128 bytes x box_rows rows.
int make_operand_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t kbytes, int box_rows) {
  EncodeTiledFn fn;
  int rc = get_encode_fn(&fn);
  if (rc != ARCQ_OK) return rc;
  cuuint64_t dims[2] = {(cuuint64_t)kbytes, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)kbytes};
  cuuint32_t box[2] = {(cuuint32_t)BK_BYTES, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cuda_fail(cudaErrorInvalidValue);
  return ARCQ_OK;
}

// Scale-factor buffer as a 2-D tensor of 32-bit words: one row per 512-byte atom; box = four atoms
// (the four K steps of one stage of one 128-row tile).
int make_sf_map(CUtensorMap* map, const void* ptr, int64_t total_atoms) {
  EncodeTiledFn fn;
  int rc = get_encode_fn(&fn);
  if (rc != ARCQ_OK) return rc;
  cuuint64_t dims[2] = {128, (cuuint64_t)total_atoms};
  cuuint64_t strides[1] = {(cuuint64_t)ATOM};
  cuuint32_t box[2] = {128, (cuuint32_t)KSTEPS};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cuda_fail(cudaErrorInvalidValue);
  return ARCQ_OK;
}

// bf16 output [M, N] with a box of 64 columns x 32 rows, 128-byte swizzle (what one epilogue warp
// hands over per bulk store).
int make_c_map(CUtensorMap* map, const void* ptr, int64_t M, int64_t N) {
  EncodeTiledFn fn;
  int rc = get_encode_fn(&fn);
  if (rc != ARCQ_OK) return rc;
  cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
  cuuint64_t strides[1] = {(cuuint64_t)N * 2};
  cuuint32_t box[2] = {64, 32};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cuda_fail(cudaErrorInvalidValue);
  return ARCQ_OK;
}

// ngroups > 1: B and SFB hold `ngroups` matrices of N rows each, tile_group says which one every
// 256-row tile of A multiplies (see Gemm2Params).
// swiglu_amax != nullptr: SwiGLU epilogue (see Gemm2Params), C is [M, N/2]; groups: the run table of a grouped
// problem (for the maxima).
int launch_pair(const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB, int64_t M, int64_t N,
                int64_t K_eff, const GemmParams& gp, int num_sms, cudaStream_t stream, const int* tile_group = nullptr,
                int ngroups = 1, float* swiglu_amax = nullptr, const int* groups = nullptr,
                void* const* dests = nullptr, int ndests = 0, const void* residual = nullptr) {
  Gemm2Params p;
  p.rows_per_dest = ndests > 0 ? (int)(M / ndests) : 0;
  p.amax = reinterpret_cast<unsigned int*>(swiglu_amax);
  p.groups = groups;
  p.ngroups = ngroups;
  p.c = gp.c;
  p.alpha_a = gp.alpha_a;
  p.alpha_b = gp.alpha_b;
  p.alpha = gp.alpha;
  p.M = gp.M;
  p.N = gp.N;
  p.ksteps_total = gp.ksteps_total;
  p.natoms = gp.natoms;
  p.tiles_m = (int)((M + 255) / 256);
  p.tiles_n = (int)((N + 255) / 256);
  // Column by column (one strip of B shared by the whole wave, A streamed from L2 once per column) unless A
  // alone overflows half of L2: then narrow bands of 4 tile rows, whose A rows stay resident next to B while
  // the band lasts.  Measured on B200 (M 16384, PFLOP/s): the down projection (A 118 MB) 4.32 with bands of 32
  // or 64 tile rows, 4.54 with 8 or 16, 4.62 - 4.65 with 4 (bands of 32 read A three times from HBM: 885 MB
  // where the operands and the residual are 282 MB); gate_up, qkv and o (A 35 MB) within 1.5 % of one another
  // for every band height from 8 to 64.
  p.group_m = (double)M * (double)K_eff / 2.0 > 64e6 ? 4 : p.tiles_m;
  // grouped: tile rows of one matrix are neighbours, so narrow bands keep a strip of B shared by the
  // pairs that are in flight together
  if (tile_group != nullptr) p.group_m = 4;
  if (p.group_m > p.tiles_m) p.group_m = p.tiles_m;
  p.tile_group = tile_group;
  CUtensorMap ma, mb, msa, msb;
  OutputMaps mc;
  p.silu_table = nullptr;
  if (swiglu_amax != nullptr) {
    ARCQ_CUDA_TRY(cudaMemsetAsync(swiglu_amax, 0, sizeof(float) * ngroups, stream));
    int rc_t = silu_table_ptr(stream, &p.silu_table);
    if (rc_t != ARCQ_OK) return rc_t;
  }
  int rc = ARCQ_OK;
  if (ndests > 0) {
    for (int d = 0; d < ndests && rc == ARCQ_OK; ++d) rc = make_c_map(&mc.m[d], dests[d], M / ndests, N);
    for (int d = ndests; d < MAX_DESTS; ++d) mc.m[d] = mc.m[0];
  } else {
    rc = make_c_map(&mc.m[0], gp.c, M, swiglu_amax != nullptr ? N / 2 : N);
    for (int d = 1; d < MAX_DESTS; ++d) mc.m[d] = mc.m[0];
  }
  if (rc != ARCQ_OK) return rc;
  rc = make_operand_map(&ma, A, M, K_eff / 2, 128);
  if (rc != ARCQ_OK) return rc;
  rc = make_operand_map(&mb, B, N * ngroups, K_eff / 2, 128);
  if (rc != ARCQ_OK) return rc;
  rc = make_sf_map(&msa, SFA, ((M + 127) / 128) * (int64_t)gp.natoms);
  if (rc != ARCQ_OK) return rc;
  rc = make_sf_map(&msb, SFB, ((N * ngroups + 127) / 128) * (int64_t)gp.natoms);
  if (rc != ARCQ_OK) return rc;
  CUtensorMap mr = mc.m[0];
  if (residual != nullptr) {
    rc = make_c_map(&mr, residual, M, N);
    if (rc != ARCQ_OK) return rc;
  }
  auto kern = swiglu_amax != nullptr ? arcq_gemm2_kernel<true, false>
                                     : (residual != nullptr ? arcq_gemm2_kernel<false, true> : arcq_gemm2_kernel<false, false>);
  ARCQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C2_SMEM_BYTES));
  long long tiles = (long long)p.tiles_m * p.tiles_n;
  long long clusters = num_sms / 2;
  if (clusters > tiles) clusters = tiles;
  kern<<<(unsigned)(2 * clusters), C2_THREADS, C2_SMEM_BYTES, stream>>>(ma, mb, msa, msb, mc, p, mr);
  ARCQ_CUDA_TRY(cudaGetLastError());
  return ARCQ_OK;
}

template <int BN>
int launch_bn(const CUtensorMap& ma, const CUtensorMap& mb, GemmParams p, int num_sms, cudaStream_t stream) {
  using C = Cfg<BN>;
  auto kern = arcq_gemm_kernel<BN>;
  ARCQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
  p.tiles_n = (p.N + BN - 1) / BN;
  long long tiles = (long long)p.tiles_m * p.tiles_n * p.splits;
  int grid = (int)(tiles < num_sms ? tiles : num_sms);
  kern<<<grid, NUM_THREADS, C::SMEM_BYTES, stream>>>(ma, mb, p);
  ARCQ_CUDA_TRY(cudaGetLastError());
  return ARCQ_OK;
}

}  // namespace

// Narrowest tile width and K split the launcher would use for a skinny problem.
static void plan_splitk(int64_t M, int64_t N, int64_t K_eff, int num_sms, int* bn_out, int* splits_out,
                        bool allow_split = true) {
  const int tiles_m = (int)((M + BM - 1) / BM);
  int bn = 256;
  while (bn > 64 && (long long)tiles_m * ((N + bn - 1) / bn) < num_sms) bn >>= 1;
  const long long tiles = (long long)tiles_m * ((N + bn - 1) / bn);
  const int kstages = (int)((K_eff / 64 + KSTEPS - 1) / KSTEPS);
  int splits = 1;
  if (tiles_m == 1) {
    // One row of tiles (M <= 128: weight streaming).  The K loop is a serial chain of stages whose
    // latency, not bandwidth, sets the time; splitting K shortens the chain at the price of a second
    // kernel that adds the fp32 partial sums.  Pick tile width and split count by a small cost model
    // fitted to measurements on B200 (microseconds: ~5 fixed, 0.35 + 0.65 * bn/256 per stage of the
    // chain, 2 + 0.35 per MB of partial sums when split), among the choices that fit one wave of CTAs
    // and 8 MB of scratch.  Measured: N 6144, M 16: 15.4 -> 9.6 us; N 4096 / K 14464, M 16: 24.7 -> 13.4 us.
    double best = 1e30;
    int best_bn = 64, best_splits = 1;
    for (int cand = 64; cand <= 256; cand <<= 1) {
      const long long t = (N + cand - 1) / cand;
      for (int sp = 1; sp <= (allow_split ? 8 : 1); ++sp) {
        if (t * sp > num_sms && sp > 1) break;
        if (sp > 1 && sp > kstages / 2) break;
        if (sp > 1 && (sp - 1) * ((kstages + sp - 1) / sp) >= kstages) continue;   // an empty range
        const double ws_mb = sp > 1 ? (double)sp * (double)M * (double)N * 4.0 / (1 << 20) : 0.0;
        if (ws_mb > 8.0) break;
        const double waves = (double)((t * sp + num_sms - 1) / num_sms);
        const double cost = 5.0 + waves * ((kstages + sp - 1) / sp) * (0.35 + 0.65 * cand / 256.0) +
                            (sp > 1 ? 2.0 + 0.35 * ws_mb : 0.0);
        if (cost < best) { best = cost; best_bn = cand; best_splits = sp; }
      }
    }
    bn = best_bn;
    splits = best_splits;
  } else if (allow_split && tiles * 2 <= num_sms) {
    splits = (int)(num_sms / tiles);
    if (splits > 8) splits = 8;
    if (splits > kstages / 2) splits = kstages / 2;   // at least two stages per range
    if (splits < 1) splits = 1;
    // ranges of ceil(kstages/splits) stages must all be non-empty
    while (splits > 1 && (splits - 1) * ((kstages + splits - 1) / splits) >= kstages) --splits;
  }
  *bn_out = bn;
  *splits_out = splits;
}

int launch_gemm_grouped(const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB, int64_t M,
                        int64_t N, int64_t K_eff, const int* tile_group, int ngroups, const float* alpha_a,
                        const float* alpha_b, void* Cout, cudaStream_t stream, float* swiglu_amax, const int* groups) {
  DeviceInfo di;
  int rc = get_device_info(&di);
  if (rc != ARCQ_OK) return rc;
  GemmParams p = {};
  p.c = static_cast<__nv_bfloat16*>(Cout);
  p.alpha_a = alpha_a;
  p.alpha_b = alpha_b;
  p.alpha = 1.0f;
  p.M = (int)M;
  p.N = (int)N;
  p.ksteps_total = (int)(K_eff / 64);
  p.natoms = (int)((K_eff / 16 + 3) / 4);
  p.splits = 1;
  return launch_pair(A, B, SFA, SFB, M, N, K_eff, p, di.num_sms, stream, tile_group, ngroups, swiglu_amax, groups);
}

// The GEMM whose result rows are scattered over `ndests` buffers of M / ndests rows each (see
// Gemm2Params::rows_per_dest): always the CTA-pair kernel, whose epilogue stores through tensor maps.
int launch_gemm_scatter(const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB, int64_t M,
                        int64_t N, int64_t K_eff, const float* alpha_a, const float* alpha_b, void* const* dests,
                        int ndests, cudaStream_t stream) {
  if (ndests < 1 || ndests > MAX_DESTS || M % ndests || (M / ndests) % 32) return ARCQ_ERR_BAD_SHAPE;
  DeviceInfo di;
  int rc = get_device_info(&di);
  if (rc != ARCQ_OK) return rc;
  GemmParams p = {};
  p.c = nullptr;
  p.alpha_a = alpha_a;
  p.alpha_b = alpha_b;
  p.alpha = 1.0f;
  p.M = (int)M;
  p.N = (int)N;
  p.ksteps_total = (int)(K_eff / 64);
  p.natoms = (int)((K_eff / 16 + 3) / 4);
  p.splits = 1;
  return launch_pair(A, B, SFA, SFB, M, N, K_eff, p, di.num_sms, stream, nullptr, 1, nullptr, nullptr, dests, ndests);
}

// C = bf16(residual + bf16(alpha_a * alpha_b * A B^T)): always the CTA-pair kernel, whose epilogue fetches the
// residual tile by TMA.
int launch_gemm_residual(const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB, int64_t M,
                         int64_t N, int64_t K_eff, const float* alpha_a, const float* alpha_b, const void* residual,
                         void* Cout, cudaStream_t stream) {
  DeviceInfo di;
  int rc = get_device_info(&di);
  if (rc != ARCQ_OK) return rc;
  GemmParams p = {};
  p.c = static_cast<__nv_bfloat16*>(Cout);
  p.alpha_a = alpha_a;
  p.alpha_b = alpha_b;
  p.alpha = 1.0f;
  p.M = (int)M;
  p.N = (int)N;
  p.ksteps_total = (int)(K_eff / 64);
  p.natoms = (int)((K_eff / 16 + 3) / 4);
  p.splits = 1;
  return launch_pair(A, B, SFA, SFB, M, N, K_eff, p, di.num_sms, stream, nullptr, 1, nullptr, nullptr, nullptr, 0,
                     residual);
}

size_t gemm_workspace_bytes(int64_t M, int64_t N, int64_t K_eff) {
  DeviceInfo di;
  if (get_device_info(&di) != ARCQ_OK) return 0;
  int bn, splits;
  plan_splitk(M, N, K_eff, di.num_sms, &bn, &splits);
  return splits > 1 ? (size_t)splits * (size_t)M * (size_t)N * sizeof(float) : 0;
}

// Problems with enough 256 x 256 tiles to occupy at least half of the SM pairs run on CTA pairs
// (about 1.4x the throughput of the single-CTA kernel).
static bool use_pair_kernel(int64_t M, int64_t N, int num_sms) {
  return (long long)((M + 255) / 256) * ((N + 255) / 256) >= num_sms / 4 && M > 128;
}

int gemm_plan(int64_t M, int64_t N, int64_t K_eff, int* kind, int* tile_n, int* splits) {
  DeviceInfo di;
  int rc = get_device_info(&di);
  if (rc != ARCQ_OK) return rc;
  int k = ARCQ_GEMM_KIND_SINGLE, bn = 256, sp = 1;
  if (use_pair_kernel(M, N, di.num_sms)) {
    k = ARCQ_GEMM_KIND_PAIR;
  } else {
    plan_splitk(M, N, K_eff, di.num_sms, &bn, &sp);
    if (sp > 1) k = ARCQ_GEMM_KIND_SPLIT_K;
  }
  if (kind) *kind = k;
  if (tile_n) *tile_n = bn;
  if (splits) *splits = sp;
  return ARCQ_OK;
}

int launch_gemm(const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB, int64_t M, int64_t N,
                int64_t K_eff, float alpha, const float* alpha_a, const float* alpha_b, void* Cout,
                void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  DeviceInfo di;
  int rc = get_device_info(&di);
  if (rc != ARCQ_OK) return rc;

  GemmParams p;
  p.sfa = SFA;
  p.sfb = SFB;
  p.c = static_cast<__nv_bfloat16*>(Cout);
  p.alpha_a = alpha_a;
  p.alpha_b = alpha_b;
  p.alpha = alpha;
  p.M = (int)M;
  p.N = (int)N;
  p.ksteps_total = (int)(K_eff / 64);
  p.natoms = (int)((K_eff / 16 + 3) / 4);
  p.tiles_m = (int)((M + BM - 1) / BM);
  p.tiles_n = 0;
  p.sfb_tiles = (int)((N + 127) / 128);
  p.ws = nullptr;
  p.splits = 1;

  // Widest tile that still gives every SM work; narrow tiles for skinny problems.  Partial tiles
  // are clipped by the TMA box (zero fill) and by the store guards.
  int bn = 256;
  while (bn > 64 && (long long)p.tiles_m * ((N + bn - 1) / bn) < di.num_sms) bn >>= 1;

  if (use_pair_kernel(M, N, di.num_sms)) return launch_pair(A, B, SFA, SFB, M, N, K_eff, p, di.num_sms, stream);

  // Skinny problems (few output tiles, long K): split K over otherwise idle SMs when the caller
  // provided scratch for the fp32 partial sums.
  {
    int bn2, splits;
    plan_splitk(M, N, K_eff, di.num_sms, &bn2, &splits, workspace != nullptr);
    if (splits > 1 && workspace_bytes < (size_t)splits * (size_t)M * (size_t)N * sizeof(float))
      plan_splitk(M, N, K_eff, di.num_sms, &bn2, &splits, false);   // scratch too small: do not split
    if (splits > 1 && workspace == nullptr) splits = 1;             // (never split without scratch)
    if (splits > 1) {
      bn = bn2;
      p.ws = static_cast<float*>(workspace);
      p.splits = splits;
    } else if (p.tiles_m == 1) {
      bn = bn2;   // single row of tiles: the cost model also picks the width of an unsplit launch
    }
  }

  CUtensorMap ma, mb;
  rc = make_operand_map(&ma, A, M, K_eff / 2, BM);
  if (rc != ARCQ_OK) return rc;
  rc = make_operand_map(&mb, B, N, K_eff / 2, bn);
  if (rc != ARCQ_OK) return rc;

  switch (bn) {
    case 256: rc = launch_bn<256>(ma, mb, p, di.num_sms, stream); break;
    case 128: rc = launch_bn<128>(ma, mb, p, di.num_sms, stream); break;
    default: rc = launch_bn<64>(ma, mb, p, di.num_sms, stream); break;
  }
  if (rc != ARCQ_OK || p.splits == 1) return rc;
  const long long mn = (long long)M * N;
  long long blocks = (mn / 8 + 255) / 256;
  if (blocks > (long long)di.num_sms * 8) blocks = (long long)di.num_sms * 8;
  arcq_splitk_reduce_kernel<<<(unsigned)blocks, 256, 0, stream>>>(p.ws, p.splits, mn, alpha, alpha_a, alpha_b, p.c);
  ARCQ_CUDA_TRY(cudaGetLastError());
  return ARCQ_OK;
}

// ----------------------------------------------------------------------------- no-allocation entry point
//
// Scratch for arcq_matmul_nvfp4_static: a fixed block of device memory that is part of the loaded
// library image (every GPU that loads libarcq.so carries these 2 MiB until the process exits).
// In host code the name below is only a handle; the device address is looked up once per device
// with cudaGetSymbolAddress and that address is what the kernels receive.
constexpr size_t STATIC_SCRATCH_BYTES = (size_t)ARCQ_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];

static int static_scratch_address(void** out) {
  static std::mutex mu;
  static void* addr[64] = {};
  int dev = 0;
  ARCQ_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return ARCQ_ERR_CUDA;
  std::lock_guard<std::mutex> lock(mu);
  if (addr[dev] == nullptr) {
    void* ptr = nullptr;
    ARCQ_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_scratch));   // with device `dev` current
    if (ptr == nullptr) return cuda_fail(cudaErrorInvalidSymbol);
    addr[dev] = ptr;
  }
  *out = addr[dev];
  return ARCQ_OK;
}

int launch_gemm_static(const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB, int64_t M,
                       int64_t N, int64_t K_eff, float alpha, const float* alpha_a, const float* alpha_b, void* Cout,
                       cudaStream_t stream) {
  const size_t need = gemm_workspace_bytes(M, N, K_eff);
  if (need > STATIC_SCRATCH_BYTES) return ARCQ_ERR_SCRATCH_LIMIT;
  void* scratch = nullptr;
  int rc = static_scratch_address(&scratch);
  if (rc != ARCQ_OK) return rc;
  return launch_gemm(A, B, SFA, SFB, M, N, K_eff, alpha, alpha_a, alpha_b, Cout, scratch, STATIC_SCRATCH_BYTES, stream);
}

int gemm_poll_error() {
  ARCQ_CUDA_TRY(cudaDeviceSynchronize());
  int v = 0;
  ARCQ_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(int)));
  if (v != 0) {
    int zero = 0;
    ARCQ_CUDA_TRY(cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int)));
  }
  return v;
}

}  // namespace arcq
