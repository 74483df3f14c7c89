// C-ABI entry points of libarcq.so: argument validation, then the kernel launchers.
#include <cuda_runtime.h>
#include <string.h>
#include <stdint.h>

#include <atomic>
#include <mutex>

#include "arcq_internal.h"

namespace arcq {

static thread_local int g_last_cuda_error = 0;

int cuda_fail(cudaError_t e) {
  g_last_cuda_error = (int)e;
  (void)cudaGetLastError();  // clear the sticky "last error" of non-fatal failures
  return ARCQ_ERR_CUDA;
}

// Upper bound on the SMs the persistent kernels spread over (0 = all of them), see arcq_set_sm_limit.
static std::atomic<int> g_sm_limit{0};

int get_device_info(DeviceInfo* out) {
  static std::mutex mu;
  static DeviceInfo cache[64];
  static bool have[64] = {};
  int dev = 0;
  ARCQ_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return ARCQ_ERR_CUDA;
  std::lock_guard<std::mutex> lock(mu);
  if (!have[dev]) {
    DeviceInfo d;
    d.device = dev;
    ARCQ_CUDA_TRY(cudaDeviceGetAttribute(&d.num_sms, cudaDevAttrMultiProcessorCount, dev));
    ARCQ_CUDA_TRY(cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    cache[dev] = d;
    have[dev] = true;
  }
  *out = cache[dev];
  const int limit = g_sm_limit.load(std::memory_order_relaxed);
  if (limit > 0 && limit < out->num_sms) out->num_sms = limit;
  return ARCQ_OK;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int check_quant_shape(int64_t rows, int KQ, int KE, int mode) {
  if (rows < 0 || KQ <= 0 || KE < 0 || KE > KQ) return ARCQ_ERR_BAD_SHAPE;
  if (mode != ARCQ_MODE_16 && mode != ARCQ_MODE_32) return ARCQ_ERR_BAD_SHAPE;
  if (KQ % 16 || KE % 16) return ARCQ_ERR_BAD_SHAPE;
  if (mode == ARCQ_MODE_32 && (KQ % 32 || KE % 32)) return ARCQ_ERR_BAD_SHAPE;
  if (KQ > 32752) return ARCQ_ERR_UNSUPPORTED_K;  // int16 channel numbers
  return ARCQ_OK;
}

}  // namespace arcq

using namespace arcq;

extern "C" {

const char* arcq_status_string(int status) {
  switch (status) {
    case ARCQ_OK: return "ok";
    case ARCQ_ERR_BAD_SHAPE: return "bad shape";
    case ARCQ_ERR_UNSUPPORTED_K: return "unsupported K";
    case ARCQ_ERR_NULL_POINTER: return "null pointer";
    case ARCQ_ERR_CUDA: return "CUDA error";
    case ARCQ_ERR_ALIGNMENT: return "pointer not 16-byte aligned";
    case ARCQ_ERR_TIMEOUT: return "device-side wait timed out";
    case ARCQ_ERR_SCRATCH_LIMIT:
      return "problem needs more scratch than the built-in 2 MiB block of arcq_matmul_nvfp4_static; "
             "use arcq_matmul_nvfp4_ws with caller-provided scratch";
    default: return "unknown status";
  }
}

int arcq_last_cuda_error(void) { return g_last_cuda_error; }

int arcq_version(void) { return 200; }

int arcq_set_sm_limit(int sms) {
  if (sms < 0) sms = 0;
  return g_sm_limit.exchange(sms, std::memory_order_relaxed);
}

size_t arcq_sf_bytes(int64_t rows, int64_t k_eff) {
  if (rows < 0 || k_eff < 0) return 0;
  int64_t ncols = k_eff / 16;
  int64_t ref = (rows / 128 + 1) * 128 * k_eff / 16;
  int64_t span = ((rows + 127) / 128) * ((ncols + 3) / 4) * 512;
  return (size_t)(ref > span ? ref : span);
}

int arcq_reference_mode(int kq) {
  return (kq == 3584 || kq == 18944 || kq == 27648 || kq == 28672) ? ARCQ_MODE_32 : ARCQ_MODE_16;
}

int arcq_reorder_quantize_x(const void* x, const int16_t* reorder_index, int64_t M, int KQ, int KE, int mode,
                            uint8_t* qx, uint8_t* sfx, void* stream) {
  int rc = check_quant_shape(M, KQ, KE, mode);
  if (rc != ARCQ_OK) return rc;
  if (M == 0) return ARCQ_OK;
  if (!x || !qx || !sfx) return ARCQ_ERR_NULL_POINTER;
  if (!aligned16(x) || !aligned16(qx)) return ARCQ_ERR_ALIGNMENT;
  return launch_quantize(x, nullptr, 0.f, reorder_index, M, KQ, KE, mode, 0, qx, sfx, (cudaStream_t)stream);
}

int arcq_reorder_quantize_x_scaled(const void* x, const float* scale, const int16_t* reorder_index, int64_t M, int KQ,
                                   int KE, int mode, uint8_t* qx, uint8_t* sfx, void* stream) {
  int rc = check_quant_shape(M, KQ, KE, mode);
  if (rc != ARCQ_OK) return rc;
  if (M == 0) return ARCQ_OK;
  if (!x || !scale || !qx || !sfx) return ARCQ_ERR_NULL_POINTER;
  if (!aligned16(x) || !aligned16(qx)) return ARCQ_ERR_ALIGNMENT;
  return launch_quantize(x, nullptr, 0.f, reorder_index, M, KQ, KE, mode, 0, qx, sfx, (cudaStream_t)stream, scale);
}

int arcq_rmsnorm_quantize_x(const void* x, const void* gamma, float eps, const int16_t* reorder_index,
                            int64_t M, int KQ, int KE, uint8_t* qx, uint8_t* sfx, void* stream) {
  int rc = check_quant_shape(M, KQ, KE, ARCQ_MODE_16);
  if (rc != ARCQ_OK) return rc;
  int g = KQ / 16;
  if (g % 32 || g < 64 || g > 512) return ARCQ_ERR_UNSUPPORTED_K;
  if (M == 0) return ARCQ_OK;
  if (!x || !gamma || !qx || !sfx) return ARCQ_ERR_NULL_POINTER;
  if (!aligned16(x) || !aligned16(qx)) return ARCQ_ERR_ALIGNMENT;
  return launch_quantize(x, gamma, eps, reorder_index, M, KQ, KE, ARCQ_MODE_16, 0, qx, sfx,
                         (cudaStream_t)stream);
}

int arcq_rmsnorm_quantize_x_multi(const void* x, const void* gamma, float eps, const int16_t* reorder_index,
                                  int64_t M, int KQ, int KE, uint8_t* const* qx, uint8_t* const* sfx, int ndests,
                                  void* stream) {
  int rc = check_quant_shape(M, KQ, KE, ARCQ_MODE_16);
  if (rc != ARCQ_OK) return rc;
  int g = KQ / 16;
  if (g % 32 || g < 64 || g > 512) return ARCQ_ERR_UNSUPPORTED_K;
  if (ndests < 1 || ndests > 8) return ARCQ_ERR_BAD_SHAPE;
  if (!qx || !sfx) return ARCQ_ERR_NULL_POINTER;
  if (M == 0) return ARCQ_OK;
  if (!x || !gamma) return ARCQ_ERR_NULL_POINTER;
  if (!aligned16(x)) return ARCQ_ERR_ALIGNMENT;
  for (int d = 0; d < ndests; ++d) {
    if (!qx[d] || !sfx[d]) return ARCQ_ERR_NULL_POINTER;
    if (!aligned16(qx[d]) || !aligned16(sfx[d])) return ARCQ_ERR_ALIGNMENT;
  }
  return launch_quantize(x, gamma, eps, reorder_index, M, KQ, KE, ARCQ_MODE_16, 0, qx[0], sfx[0],
                         (cudaStream_t)stream, nullptr, nullptr, 0, nullptr, qx + 1, sfx + 1, ndests - 1);
}

int arcq_ep_send_layout(const int64_t* ids, int n, int e_local, int ep, int cap, int rank, int32_t* slot,
                        void* const* slot_tables, int32_t* overflow, void* stream) {
  if (n < 0 || n > (1 << 20) || e_local < 1 || ep < 1 || ep > 8 || cap < 1 || rank < 0 || rank >= ep ||
      (int64_t)ep * cap > (int64_t)0x3fffffff)
    return ARCQ_ERR_BAD_SHAPE;
  if ((n > 0 && (!ids || !slot)) || !slot_tables || !overflow) return ARCQ_ERR_NULL_POINTER;
  for (int d = 0; d < ep; ++d)
    if (!slot_tables[d]) return ARCQ_ERR_NULL_POINTER;
  return launch_ep_send_layout(reinterpret_cast<const long long*>(ids), n, e_local, ep, cap, rank, slot, slot_tables,
                               overflow, (cudaStream_t)stream);
}

int arcq_ep_rows(const void* src, const int32_t* item_src, int div, int src_limit, const int32_t* item_slot, int n,
                 int row_bytes, int cap, int ep, int rank, void* const* dst, void* stream) {
  if (n < 0 || div < 1 || src_limit < 0 || row_bytes <= 0 || row_bytes % 16 || cap < 1 || ep < 1 || ep > 8 || rank < 0 ||
      rank >= ep || (int64_t)ep * cap > (int64_t)0x3fffffff)
    return ARCQ_ERR_BAD_SHAPE;
  if (n == 0) return ARCQ_OK;
  if (!src || !dst) return ARCQ_ERR_NULL_POINTER;
  if (!aligned16(src)) return ARCQ_ERR_ALIGNMENT;
  for (int d = 0; d < ep; ++d) {
    if (!dst[d]) return ARCQ_ERR_NULL_POINTER;
    if (!aligned16(dst[d])) return ARCQ_ERR_ALIGNMENT;
  }
  return launch_ep_rows(src, item_src, div, src_limit, item_slot, n, row_bytes, cap, ep, rank, dst, (cudaStream_t)stream);
}

int arcq_peer_barrier(void* const* flags, int rank, int world, uint32_t* counter, void* stream) {
  if (world < 1 || world > 8 || rank < 0 || rank >= world) return ARCQ_ERR_BAD_SHAPE;
  if (!flags || !counter) return ARCQ_ERR_NULL_POINTER;
  for (int d = 0; d < world; ++d)
    if (!flags[d]) return ARCQ_ERR_NULL_POINTER;
  return launch_peer_barrier(flags, rank, world, counter, (cudaStream_t)stream);
}

int arcq_peer_poll_error(void) { return peer_poll_error(); }

int arcq_peer_set_wait_limit_ms(int ms) { return peer_set_wait_limit_ms(ms); }

int arcq_reorder_quantize_w(const void* w, const int16_t* reorder_index, int64_t N, int KQ, int KE, int mode,
                            uint8_t* qw, uint8_t* sfw, void* stream) {
  int rc = check_quant_shape(N, KQ, KE, mode);
  if (rc != ARCQ_OK) return rc;
  if (N == 0) return ARCQ_OK;
  if (!w || !qw || !sfw) return ARCQ_ERR_NULL_POINTER;
  if (!aligned16(w) || !aligned16(qw)) return ARCQ_ERR_ALIGNMENT;
  return launch_quantize(w, nullptr, 0.f, reorder_index, N, KQ, KE, mode, 1, qw, sfw, (cudaStream_t)stream);
}

static int check_gemm(const void* A, const void* B, const void* SFA, const void* SFB, int64_t M, int64_t N,
                      int64_t K, const void* C) {
  if (M < 0 || N <= 0 || K <= 0) return ARCQ_ERR_BAD_SHAPE;
  if (K % 64 || N % 8) return ARCQ_ERR_BAD_SHAPE;
  if (M > (int64_t)1 << 30 || N > (int64_t)1 << 30 || K > (int64_t)1 << 20) return ARCQ_ERR_BAD_SHAPE;
  // the kernels count work items (128 x 64 tiles, up to eight K ranges each) in 32-bit integers
  if (((M + 127) / 128) * ((N + 63) / 64) * 8 > (int64_t)0x7fffffff) return ARCQ_ERR_BAD_SHAPE;
  if (M == 0) return ARCQ_OK;
  if (!A || !B || !SFA || !SFB || !C) return ARCQ_ERR_NULL_POINTER;
  if (!aligned16(A) || !aligned16(B) || !aligned16(SFA) || !aligned16(SFB) || !aligned16(C))
    return ARCQ_ERR_ALIGNMENT;
  return ARCQ_OK;
}

int arcq_matmul_nvfp4(const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB, int64_t M,
                      int64_t N, int64_t K_eff, float alpha, void* C, void* stream) {
  int rc = check_gemm(A, B, SFA, SFB, M, N, K_eff, C);
  if (rc != ARCQ_OK || M == 0) return rc;
  return launch_gemm(A, B, SFA, SFB, M, N, K_eff, alpha, nullptr, nullptr, C, nullptr, 0, (cudaStream_t)stream);
}

int arcq_matmul_nvfp4_dev_alpha(const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB,
                                int64_t M, int64_t N, int64_t K_eff, const float* alpha_a,
                                const float* alpha_b, void* C, void* stream) {
  int rc = check_gemm(A, B, SFA, SFB, M, N, K_eff, C);
  if (rc != ARCQ_OK || M == 0) return rc;
  if (!alpha_a) return ARCQ_ERR_NULL_POINTER;
  return launch_gemm(A, B, SFA, SFB, M, N, K_eff, 1.0f, alpha_a, alpha_b, C, nullptr, 0, (cudaStream_t)stream);
}

size_t arcq_matmul_workspace_bytes(int64_t M, int64_t N, int64_t K_eff) {
  if (M <= 0 || N <= 0 || K_eff <= 0) return 0;
  return gemm_workspace_bytes(M, N, K_eff);
}

int arcq_matmul_plan(int64_t M, int64_t N, int64_t K_eff, int* kind, int* tile_n, int* splits) {
  if (M <= 0 || N <= 0 || K_eff <= 0 || K_eff % 64 || N % 8) return ARCQ_ERR_BAD_SHAPE;
  return gemm_plan(M, N, K_eff, kind, tile_n, splits);
}

int arcq_matmul_nvfp4_ws(const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB, int64_t M,
                         int64_t N, int64_t K_eff, float alpha, const float* alpha_a, const float* alpha_b, void* C,
                         void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_gemm(A, B, SFA, SFB, M, N, K_eff, C);
  if (rc != ARCQ_OK || M == 0) return rc;
  if (workspace != nullptr && !aligned16(workspace)) return ARCQ_ERR_ALIGNMENT;
  return launch_gemm(A, B, SFA, SFB, M, N, K_eff, alpha, alpha_a, alpha_b, C, workspace, workspace_bytes,
                     (cudaStream_t)stream);
}

int arcq_matmul_nvfp4_static(const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB, int64_t M,
                             int64_t N, int64_t K_eff, float alpha, const float* alpha_a, const float* alpha_b,
                             void* C, void* stream) {
  int rc = check_gemm(A, B, SFA, SFB, M, N, K_eff, C);
  if (rc != ARCQ_OK || M == 0) return rc;
  return launch_gemm_static(A, B, SFA, SFB, M, N, K_eff, alpha, alpha_a, alpha_b, C, (cudaStream_t)stream);
}

int arcq_gemm_poll_error(void) {
  const int g = gemm_poll_error();
  const int q = quant_poll_error();   // read (and cleared) as well, whatever the first says
  return g != ARCQ_OK ? g : q;
}

int arcq_rope_bf16(void* x, const float* cos_table, const float* sin_table, int64_t tokens, int row_elems, int heads,
                   int head_dim, int seq, void* stream) {
  if (tokens < 0 || heads < 0 || seq <= 0 || head_dim <= 0 || head_dim % 16 || row_elems % 8 ||
      (int64_t)heads * head_dim > row_elems)
    return ARCQ_ERR_BAD_SHAPE;
  if (tokens == 0 || heads == 0) return ARCQ_OK;
  if (!x || !cos_table || !sin_table) return ARCQ_ERR_NULL_POINTER;
  if (!aligned16(x)) return ARCQ_ERR_ALIGNMENT;
  return launch_rope(x, cos_table, sin_table, tokens, row_elems, heads, head_dim, seq, (cudaStream_t)stream);
}

int arcq_silu_mul_bf16(const void* gate_up, void* out, int64_t tokens, int F, float* amax, void* stream) {
  if (tokens < 0 || F <= 0 || F % 8) return ARCQ_ERR_BAD_SHAPE;
  if (tokens == 0) return launch_silu_mul(gate_up, out, 0, F, amax, (cudaStream_t)stream);
  if (!gate_up || !out) return ARCQ_ERR_NULL_POINTER;
  if (!aligned16(gate_up) || !aligned16(out)) return ARCQ_ERR_ALIGNMENT;
  return launch_silu_mul(gate_up, out, tokens, F, amax, (cudaStream_t)stream);
}

int arcq_moe_combine_bf16(const void* y, const int32_t* pos, const void* weights, void* out, int64_t tokens, int hidden,
                          int top_k, void* stream) {
  if (tokens < 0 || hidden <= 0 || hidden % 8 || top_k < 1) return ARCQ_ERR_BAD_SHAPE;
  if (tokens == 0) return ARCQ_OK;
  if (!y || !pos || !weights || !out) return ARCQ_ERR_NULL_POINTER;
  if (!aligned16(y) || !aligned16(out)) return ARCQ_ERR_ALIGNMENT;
  return launch_moe_combine(y, pos, weights, out, tokens, hidden, top_k, (cudaStream_t)stream);
}

int arcq_calib_stats_bf16(const void* x, int64_t rows, int K, float* chan_absmax, unsigned long long* above,
                          void* stream) {
  if (rows < 0 || K <= 0 || K % 8) return ARCQ_ERR_BAD_SHAPE;
  if (K > 32768) return ARCQ_ERR_UNSUPPORTED_K;
  if (rows == 0) return ARCQ_OK;
  if (!x || !chan_absmax) return ARCQ_ERR_NULL_POINTER;
  if (!aligned16(x)) return ARCQ_ERR_ALIGNMENT;
  return launch_calib_stats(x, rows, K, chan_absmax, above, (cudaStream_t)stream);
}

int arcq_moe_layout(const int64_t* slot_group, int n, int ngroups, int tile, int rows_bound, int div, int32_t* dest,
                    int32_t* row_map, int32_t* groups, int32_t* tile_group, void* stream) {
  if (n < 0 || n > (1 << 20) || ngroups < 1 || ngroups > 64 || tile < 1 || div < 1 || rows_bound % tile ||
      (int64_t)rows_bound < ((int64_t)n + tile - 1) / tile * tile + (int64_t)ngroups * tile)
    return ARCQ_ERR_BAD_SHAPE;
  if ((n > 0 && !slot_group) || !dest || !row_map || !groups || !tile_group) return ARCQ_ERR_NULL_POINTER;
  return launch_moe_layout(reinterpret_cast<const long long*>(slot_group), n, ngroups, tile, rows_bound, div, dest,
                           row_map, groups, tile_group, (cudaStream_t)stream);
}

int arcq_silu_mul_grouped_bf16(const void* gate_up, void* out, int64_t rows_bound, int F, const int32_t* tile_group,
                               const int32_t* groups, int ngroups, float* amax, void* stream) {
  if (rows_bound < 0 || rows_bound % 256 || F <= 0 || F % 256 || ngroups < 1 || ngroups > 64) return ARCQ_ERR_BAD_SHAPE;
  if (rows_bound == 0) return ARCQ_OK;
  if (!gate_up || !out || !tile_group || !groups) return ARCQ_ERR_NULL_POINTER;
  if (!aligned16(gate_up) || !aligned16(out)) return ARCQ_ERR_ALIGNMENT;
  return launch_silu_mul_grouped(gate_up, out, rows_bound, F, tile_group, groups, ngroups, amax, (cudaStream_t)stream);
}

int arcq_absmax_grouped_bf16(const void* x, const int32_t* row_map, const int32_t* groups, int ngroups, int K, float* out,
                             void* stream) {
  if (ngroups < 1 || ngroups > 64 || K <= 0 || K % 8) return ARCQ_ERR_BAD_SHAPE;
  if (!x || !groups || !out) return ARCQ_ERR_NULL_POINTER;
  if (!aligned16(x)) return ARCQ_ERR_ALIGNMENT;
  return launch_absmax_grouped(x, row_map, groups, ngroups, K, out, (cudaStream_t)stream);
}

int arcq_reorder_quantize_x_grouped(const void* x, const int32_t* row_map, const float* scales,
                                    const int16_t* reorder_indices, const int32_t* groups, int ngroups,
                                    int64_t rows_bound, int KQ, int KE, int mode, uint8_t* qx, uint8_t* sfx,
                                    void* stream) {
  int rc = check_quant_shape(rows_bound, KQ, KE, mode);
  if (rc != ARCQ_OK) return rc;
  if (ngroups < 1 || ngroups > 64) return ARCQ_ERR_BAD_SHAPE;
  if (rows_bound == 0) return ARCQ_OK;
  if (!x || !scales || !groups || !qx || !sfx) return ARCQ_ERR_NULL_POINTER;
  if (!aligned16(x) || !aligned16(qx)) return ARCQ_ERR_ALIGNMENT;
  return launch_quantize(x, nullptr, 0.f, reorder_indices, rows_bound, KQ, KE, mode, 0, qx, sfx, (cudaStream_t)stream,
                         scales, groups, ngroups, row_map);
}

int arcq_matmul_nvfp4_grouped(const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB,
                              int64_t M_bound, int64_t N, int64_t K_eff, const int32_t* tile_group, int ngroups,
                              const float* alpha_a, const float* alpha_b, void* C, void* stream) {
  int rc = check_gemm(A, B, SFA, SFB, M_bound, N, K_eff, C);
  if (rc != ARCQ_OK || M_bound == 0) return rc;
  if (ngroups < 1 || N % 128 || N * (int64_t)ngroups > ((int64_t)1 << 30)) return ARCQ_ERR_BAD_SHAPE;
  if (!tile_group || !alpha_a) return ARCQ_ERR_NULL_POINTER;
  return launch_gemm_grouped(A, B, SFA, SFB, M_bound, N, K_eff, tile_group, ngroups, alpha_a, alpha_b, C,
                             (cudaStream_t)stream);
}

int arcq_matmul_nvfp4_swiglu(const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB, int64_t M,
                             int64_t N, int64_t K_eff, const float* alpha_a, const float* alpha_b, void* C,
                             float* amax, void* stream) {
  int rc = check_gemm(A, B, SFA, SFB, M, N, K_eff, C);
  if (rc != ARCQ_OK) return rc;
  if (N % 256) return ARCQ_ERR_BAD_SHAPE;
  if (!alpha_a || !amax) return ARCQ_ERR_NULL_POINTER;
  if (M == 0) return ARCQ_OK;
  return launch_gemm_grouped(A, B, SFA, SFB, M, N, K_eff, nullptr, 1, alpha_a, alpha_b, C, (cudaStream_t)stream, amax,
                             nullptr);
}

int arcq_matmul_nvfp4_grouped_swiglu(const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB,
                                     int64_t M_bound, int64_t N, int64_t K_eff, const int32_t* tile_group,
                                     const int32_t* groups, int ngroups, const float* alpha_a, const float* alpha_b,
                                     void* C, float* amax, void* stream) {
  int rc = check_gemm(A, B, SFA, SFB, M_bound, N, K_eff, C);
  if (rc != ARCQ_OK || M_bound == 0) return rc;
  if (ngroups < 1 || ngroups > 64 || N % 256 || N * (int64_t)ngroups > ((int64_t)1 << 30)) return ARCQ_ERR_BAD_SHAPE;
  if (!tile_group || !groups || !alpha_a || !amax) return ARCQ_ERR_NULL_POINTER;
  return launch_gemm_grouped(A, B, SFA, SFB, M_bound, N, K_eff, tile_group, ngroups, alpha_a, alpha_b, C,
                             (cudaStream_t)stream, amax, groups);
}

int arcq_matmul_nvfp4_residual(const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB, int64_t M,
                               int64_t N, int64_t K_eff, const float* alpha_a, const float* alpha_b,
                               const void* residual, void* C, void* stream) {
  int rc = check_gemm(A, B, SFA, SFB, M, N, K_eff, C);
  if (rc != ARCQ_OK || M == 0) return rc;
  if (!alpha_a || !residual) return ARCQ_ERR_NULL_POINTER;
  if (!aligned16(residual)) return ARCQ_ERR_ALIGNMENT;
  return launch_gemm_residual(A, B, SFA, SFB, M, N, K_eff, alpha_a, alpha_b, residual, C, (cudaStream_t)stream);
}

int arcq_matmul_nvfp4_scatter(const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB, int64_t M,
                              int64_t N, int64_t K_eff, const float* alpha_a, const float* alpha_b,
                              void* const* dests, int ndests, void* stream) {
  if (!dests || ndests < 1 || ndests > 8) return dests ? ARCQ_ERR_BAD_SHAPE : ARCQ_ERR_NULL_POINTER;
  int rc = check_gemm(A, B, SFA, SFB, M, N, K_eff, dests[0]);
  if (rc != ARCQ_OK || M == 0) return rc;
  if (M % ndests || (M / ndests) % 32) return ARCQ_ERR_BAD_SHAPE;
  for (int d = 0; d < ndests; ++d) {
    if (!dests[d]) return ARCQ_ERR_NULL_POINTER;
    if (!aligned16(dests[d])) return ARCQ_ERR_ALIGNMENT;
  }
  if (!alpha_a) return ARCQ_ERR_NULL_POINTER;
  return launch_gemm_scatter(A, B, SFA, SFB, M, N, K_eff, alpha_a, alpha_b, dests, ndests, (cudaStream_t)stream);
}

int arcq_sum_partials_bf16(const void* const* srcs, int n, int64_t elems, const void* residual, void* out,
                           void* stream) {
  if (elems < 0 || elems % 8 || n < 1 || n > 8) return ARCQ_ERR_BAD_SHAPE;
  if (elems == 0) return ARCQ_OK;
  if (!srcs || !out) return ARCQ_ERR_NULL_POINTER;
  for (int s = 0; s < n; ++s) {
    if (!srcs[s]) return ARCQ_ERR_NULL_POINTER;
    if (!aligned16(srcs[s])) return ARCQ_ERR_ALIGNMENT;
  }
  if (!aligned16(out) || (residual && !aligned16(residual))) return ARCQ_ERR_ALIGNMENT;
  return launch_sum_partials(srcs, n, elems, residual, out, (cudaStream_t)stream);
}

int arcq_peer_alloc(size_t bytes, void** ptr) {
  if (!ptr) return ARCQ_ERR_NULL_POINTER;
  if (bytes == 0) return ARCQ_ERR_BAD_SHAPE;
  *ptr = nullptr;
  ARCQ_CUDA_TRY(cudaMalloc(ptr, bytes));
  return ARCQ_OK;
}

int arcq_peer_free(void* ptr) {
  if (ptr) ARCQ_CUDA_TRY(cudaFree(ptr));
  return ARCQ_OK;
}

int arcq_peer_export(void* ptr, unsigned char* handle) {
  static_assert(sizeof(cudaIpcMemHandle_t) == ARCQ_PEER_HANDLE_BYTES, "handle size");
  if (!ptr || !handle) return ARCQ_ERR_NULL_POINTER;
  cudaIpcMemHandle_t h;
  ARCQ_CUDA_TRY(cudaIpcGetMemHandle(&h, ptr));
  memcpy(handle, &h, sizeof(h));
  return ARCQ_OK;
}

int arcq_peer_open(const unsigned char* handle, void** ptr) {
  if (!handle || !ptr) return ARCQ_ERR_NULL_POINTER;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  *ptr = nullptr;
  ARCQ_CUDA_TRY(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return ARCQ_OK;
}

int arcq_peer_close(void* ptr) {
  if (ptr) ARCQ_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
  return ARCQ_OK;
}

int arcq_absmax_bf16(const void* x, int64_t n, float* out, int accumulate, void* stream) {
  if (n < 0) return ARCQ_ERR_BAD_SHAPE;
  if (!out || (n > 0 && !x)) return ARCQ_ERR_NULL_POINTER;
  if (n > 0 && !aligned16(x)) return ARCQ_ERR_ALIGNMENT;
  return launch_absmax(x, n, out, accumulate, (cudaStream_t)stream);
}

}  // extern "C"
