// Internal declarations shared by the translation units of libarcq.so.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "arcq.h"

namespace arcq {

// Records a failing CUDA call for arcq_last_cuda_error() and returns ARCQ_ERR_CUDA.
int cuda_fail(cudaError_t e);

#define ARCQ_CUDA_TRY(expr)                                  \
  do {                                                       \
    cudaError_t _e = (expr);                                 \
    if (_e != cudaSuccess) return ::arcq::cuda_fail(_e);     \
  } while (0)

struct DeviceInfo {
  int device;
  int num_sms;
  int max_smem_optin;
};
// Cached properties of the current device (queried once per device).
int get_device_info(DeviceInfo* out);

// Launchers (defined in arcq_quant.cu / arcq_gemm.cu); arguments are validated by the callers
// in arcq_api.cu.
int launch_quantize(const void* x, const void* gamma, float eps, const int16_t* idx, int64_t rows, int KQ,
                    int KE, int mode, int is_weight, uint8_t* q, uint8_t* sf, cudaStream_t stream,
                    const float* scale = nullptr,    // scale (device): x is divided by it first; plain x only
                    const int* groups = nullptr, int ngroups = 0,   // runs of rows with their own order and scale
                    const int* row_map = nullptr,                   // input row of every output row
                    // further copies of the output (e.g. the peers' gathered buffers), see QuantParams
                    uint8_t* const* q_extra = nullptr, uint8_t* const* sf_extra = nullptr, int nextra = 0);
int launch_absmax(const void* x, int64_t n, float* out, int accumulate, cudaStream_t stream);
// workspace (may be null): scratch for split-K partial sums, see gemm_workspace_bytes().
int launch_gemm(const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB, int64_t M,
                int64_t N, int64_t K_eff, float alpha, const float* alpha_a, const float* alpha_b, void* C,
                void* workspace, size_t workspace_bytes, cudaStream_t stream);
size_t gemm_workspace_bytes(int64_t M, int64_t N, int64_t K_eff);
// Kernel choice for a shape (see arcq_matmul_plan).
int gemm_plan(int64_t M, int64_t N, int64_t K_eff, int* kind, int* tile_n, int* splits);
// Split-K GEMM whose scratch is the library's own static device array (no allocation anywhere).
int launch_gemm_static(const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB, int64_t M,
                       int64_t N, int64_t K_eff, float alpha, const float* alpha_a, const float* alpha_b, void* C,
                       cudaStream_t stream);
// Layer glue (arcq_layer.cu).
int launch_rope(void* x, const float* cos_t, const float* sin_t, int64_t tokens, int row_elems, int heads, int dim,
                int seq, cudaStream_t stream);
int launch_silu_mul(const void* gu, void* out, int64_t tokens, int F, float* amax, cudaStream_t stream);
int launch_moe_combine(const void* y, const int* pos, const void* w, void* out, int64_t tokens, int hidden, int k,
                       cudaStream_t stream);
// One launch over `ngroups` weight matrices stacked in B (each N rows): tile_group (device) names the
// matrix of every 256-row tile of A, alpha_a / alpha_b are per-matrix arrays.
int launch_gemm_grouped(const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB, int64_t M,
                        int64_t N, int64_t K_eff, const int* tile_group, int ngroups, const float* alpha_a,
                        const float* alpha_b, void* C, cudaStream_t stream,
                        // SwiGLU epilogue: C is [M, N/2], swiglu_amax[ngroups] takes max|C| per matrix; tile_group
                        // may be null with ngroups 1 (one matrix); groups: run table of a grouped problem
                        float* swiglu_amax = nullptr, const int* groups = nullptr);
int launch_absmax_grouped(const void* x, const int* row_map, const int* groups, int ngroups, int K, float* out,
                          cudaStream_t stream);
int launch_moe_layout(const long long* slot_group, int n, int ngroups, int tile, int rows_bound, int div, int* dest,
                      int* row_map, int* groups, int* tile_group, cudaStream_t stream);
int launch_calib_stats(const void* x, int64_t rows, int K, float* chan_absmax, unsigned long long* above,
                       cudaStream_t stream);
int launch_silu_mul_grouped(const void* gu, void* out, int64_t rows, int F, const int* tile_group, const int* groups,
                            int ngroups, float* amax, cudaStream_t stream);
// GEMM whose result rows go to `ndests` buffers of M / ndests rows each (host array of device addresses; peers'
// memory allowed), and the sum of `n` partial results plus an optional residual (arcq_layer.cu).
int launch_gemm_scatter(const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB, int64_t M,
                        int64_t N, int64_t K_eff, const float* alpha_a, const float* alpha_b, void* const* dests,
                        int ndests, cudaStream_t stream);
int launch_gemm_residual(const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB, int64_t M,
                         int64_t N, int64_t K_eff, const float* alpha_a, const float* alpha_b, const void* residual,
                         void* C, cudaStream_t stream);
// Expert-parallel dispatch through peer memory (arcq_layer.cu): places of this rank's routed copies in the peers'
// receive buffers, and rows into the peers' buffers (both directions).
int launch_ep_send_layout(const long long* ids, int n, int e_local, int ep, int cap, int rank, int* slot,
                          void* const* meta, int* overflow, cudaStream_t stream);
int launch_ep_rows(const void* src, const int* item_src, int div, int src_limit, const int* item_slot, int n, int row_bytes,
                   int cap, int ep, int rank, void* const* dst, cudaStream_t stream);
int launch_peer_barrier(void* const* flags, int rank, int world, unsigned int* counter, cudaStream_t stream);
int peer_poll_error();
int peer_set_wait_limit_ms(int ms);
int launch_sum_partials(const void* const* srcs, int n, int64_t elems, const void* residual, void* out,
                        cudaStream_t stream);
// Device address of the 65536-entry table bf16(silu(g)) on the current device; the first call per device
// builds it on `stream`, later calls on other streams wait for that (arcq_layer.cu).
int silu_table_ptr(cudaStream_t stream, const uint16_t** out);
int gemm_poll_error();
// Same for the bounded waits of the warp-specialised quantizer.
int quant_poll_error();

}  // namespace arcq
