/*
 * arcq.h - C ABI of libarcq.so, the sm_100a (B200) implementation of the
 * ARC-NVFP4 quantized-linear hot path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream
 * handle (a cudaStream_t passed as void*; NULL = legacy default stream) and
 * returns an int status (ARCQ_OK = 0).  Nothing here allocates device memory
 * unless its comment says so; outputs are caller-allocated.  The library has
 * no CPU fallback: without a CUDA device every compute call returns
 * ARCQ_ERR_CUDA.
 *
 * Each function names the reference interface it replaces (paths relative to
 * the ARCQuant source tree).
 *
 * Data formats (identical to the reference's):
 *   - activations / weights in: bf16, row-major [rows, KQ]
 *   - reorder_index: int16 [KQ], ascending-by-importance channel order; the
 *     LAST KE entries are the critical channels whose quantization residual is
 *     appended (ARC)
 *   - packed codes out: uint8 [rows, (KQ+KE)/2]; element 2i in the low nibble;
 *     bytes [0, 8*G0) hold the G0=(KQ-KE)/16 plain groups, then per critical
 *     group 16 bytes [8 B main codes][8 B residual codes]
 *   - scale factors out: one ue4m3 byte per 16 elements in the 512-byte
 *     128-row x 4-column atom layout of block-scaled tensor-core GEMMs:
 *       offset(r,c) = ((r/128)*ceil(C/4) + c/4)*512 + (r%32)*16 + ((r/32)%4)*4 + c%4,
 *     C = (KQ+KE)/16.  Padding bytes are left unwritten.
 */
#ifndef ARCQ_H_
#define ARCQ_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ARCQ_OK 0
#define ARCQ_ERR_BAD_SHAPE 1      /* sizes that the data layout cannot express */
#define ARCQ_ERR_UNSUPPORTED_K 2  /* KQ outside what the kernels cover */
#define ARCQ_ERR_NULL_POINTER 3
#define ARCQ_ERR_CUDA 4           /* a CUDA runtime/driver call failed; see arcq_last_cuda_error() */
#define ARCQ_ERR_ALIGNMENT 5      /* a pointer is not 16-byte aligned */
#define ARCQ_ERR_TIMEOUT 6        /* a bounded device-side wait expired (reported by arcq_gemm_poll_error) */
#define ARCQ_ERR_SCRATCH_LIMIT 7  /* arcq_matmul_nvfp4_static: the shape needs more than its built-in scratch */

/* Channel-layout family of the critical groups.
 * 16: one group per slot  - [main][residual] per critical group
 *     (kernels/src/reorder.cu:68-203).
 * 32: groups in pairs     - [main1][main2][res1][res2], residual taken against
 *     the un-rounded fp32 block scale (kernels/src/reorder.cu:381-555,
 *     kernels/src/down.cu:71-236). */
#define ARCQ_MODE_16 16
#define ARCQ_MODE_32 32

/* Human-readable text for a status code. */
const char* arcq_status_string(int status);

/* cudaError_t value of the last failing CUDA call made by this library on the
 * calling thread (0 if none). */
int arcq_last_cuda_error(void);

/* Library version: major*10000 + minor*100 + patch. */
int arcq_version(void);

/* The quantizer and GEMM kernels are persistent: by default every launch spreads over all SMs of the
 * device, with one CTA that fills its SM.  A collective that should run at the same time on another
 * stream (an NCCL all-gather or reduce-scatter under the next GEMM) then finds no SM to start on.
 * arcq_set_sm_limit(n) makes every later launch of this process use at most n SMs (0 = all), leaving the
 * rest to whatever else runs; it returns the previous limit.  Process-wide, not per stream; a CUDA graph
 * keeps the grid sizes it was captured with.  No counterpart in the reference (it has no collectives). */
int arcq_set_sm_limit(int sms);

/* Bytes to allocate for the scale-factor buffer of `rows` rows and K_eff =
 * KQ+KE columns.  Never smaller than the reference's own size
 * (rows/128+1)*128*K_eff/16 (kernels/src/bindings.cpp:83-95) and never smaller
 * than what the atom layout spans. */
size_t arcq_sf_bytes(int64_t rows, int64_t k_eff);

/* Which family the reference dispatches a given KQ to
 * (kernels/src/bindings.cpp:141-160): ARCQ_MODE_32 for 3584, 18944, 27648,
 * 28672, else ARCQ_MODE_16. */
int arcq_reference_mode(int kq);

/* Replaces agemm.reorder_quantize_x (kernels/src/bindings.cpp:122-163 ->
 * run_reorder_x_bf16_nvfp4 kernels/src/reorder.cu:332-351, and the 32-wide /
 * pre-gathered variants reorder.cu:698-717, down.cu:363-381).
 * x: bf16 [M,KQ]; reorder_index: int16 [KQ] on the device, or NULL for the
 * identity order (an input gathered beforehand).  KQ % 16 == 0, KE % 16 == 0
 * (mode 32: % 32), 0 <= KE <= KQ, KQ <= 32752. */
int arcq_reorder_quantize_x(const void* x, const int16_t* reorder_index, int64_t M, int KQ, int KE,
                            int mode, uint8_t* qx, uint8_t* sfx, void* stream);

/* arcq_reorder_quantize_x on x / *scale: the division by the per-tensor scale that the reference's
 * callers do in torch before the operator (`x / scale` in NVFP4_reorder_quantize_x,
 * model/qLlamaLayer.py:73-77) is done while the rows are staged.  No counterpart in the reference's
 * bindings.  scale: one fp32 in device memory (so no host round trip is needed to produce it).
 * Every element becomes bf16(fp32(x) / fp32(bf16(*scale))), round to nearest even - what torch's CUDA
 * kernel gives for (bf16 tensor) / (fp32 0-dim tensor), which loads the divisor in the tensor's type -
 * and is then quantized as by arcq_reorder_quantize_x.
 * Returns ARCQ_ERR_UNSUPPORTED_K for row widths the staging kernel does not cover (KQ from 512 to
 * 16384 is covered); the caller then divides first. */
int arcq_reorder_quantize_x_scaled(const void* x, const float* scale, const int16_t* reorder_index, int64_t M, int KQ,
                                   int KE, int mode, uint8_t* qx, uint8_t* sfx, void* stream);

/* Replaces agemm.rmsnorm_quantize_x (kernels/src/bindings.cpp:216-254 ->
 * kernels/src/rmsnorm.cu:68-281): RMSNorm with gain `gamma` (bf16 [KQ]) fused
 * in front of the mode-16 quantizer.  The sum of squares is accumulated in the
 * reference's order; the reciprocal root is the correctly rounded fp32
 * 1/sqrt(ss/KQ + eps).  KQ/16 must be a multiple of 32 between 64 and 512 (KQ 1024..8192). */
int arcq_rmsnorm_quantize_x(const void* x, const void* gamma, float eps, const int16_t* reorder_index,
                            int64_t M, int KQ, int KE, uint8_t* qx, uint8_t* sfx, void* stream);

/* Replaces agemm.reorder_quantize_w (kernels/src/bindings.cpp:170-210 ->
 * kernels/src/reorder.cu:353-372, 719-738, down.cu:383-401): the offline
 * weight packer.  The residual slot of each critical group is a copy of its
 * main codes and scale, so the GEMM needs no knowledge of ARC. */
int arcq_reorder_quantize_w(const void* w, const int16_t* reorder_index, int64_t N, int KQ, int KE,
                            int mode, uint8_t* qw, uint8_t* sfw, void* stream);

/* Replaces agemm.matmul (kernels/src/bindings.cpp:99-120 ->
 * matmul_host_nvfp4_bf16 kernels/src/nvfp4.cu:35-132):
 *   C[m,n] = bf16( alpha * sum_k val(A[m,k])*SFA[m,k/16] * val(B[n,k])*SFB[n,k/16] ),
 * fp32 accumulation.  A: [M,K_eff/2], B: [N,K_eff/2] packed e2m1; C: bf16 [M,N]
 * row-major.  K_eff % 64 == 0, N % 8 == 0, all pointers 16-byte aligned. */
int arcq_matmul_nvfp4(const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB,
                      int64_t M, int64_t N, int64_t K_eff, float alpha, void* C, void* stream);

/* Same as arcq_matmul_nvfp4 with alpha = (*alpha_a) * (*alpha_b) read on the
 * device (fp32 scalars in device memory; alpha_b may be NULL = 1), so the
 * per-tensor global scales never travel to the host.  Replaces the
 * `scale * self.scale` host round trip of model/qLinearLayer.py:69. */
int arcq_matmul_nvfp4_dev_alpha(const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB,
                                int64_t M, int64_t N, int64_t K_eff, const float* alpha_a,
                                const float* alpha_b, void* C, void* stream);

/* Skinny problems (M <= 128 with a long K leave most SMs without an output tile) run faster when K
 * is split over the idle SMs; that needs scratch for the fp32 partial sums.
 * arcq_matmul_workspace_bytes: how much scratch the split-K path would use for this shape on the
 * current device (0 = the shape is not split).  arcq_matmul_nvfp4_ws: arcq_matmul_nvfp4 /
 * _dev_alpha (alpha = alpha * *alpha_a * *alpha_b, the pointers may be NULL) with caller-provided
 * scratch; with workspace == NULL or too small it behaves exactly like arcq_matmul_nvfp4.  The
 * partials are summed in a fixed order, so results are reproducible.  Same reference interface
 * as arcq_matmul_nvfp4 (kernels/src/bindings.cpp:99-120). */
size_t arcq_matmul_workspace_bytes(int64_t M, int64_t N, int64_t K_eff);
int arcq_matmul_nvfp4_ws(const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB,
                         int64_t M, int64_t N, int64_t K_eff, float alpha, const float* alpha_a,
                         const float* alpha_b, void* C, void* workspace, size_t workspace_bytes, void* stream);

/* Which kernel arcq_matmul_nvfp4* would run for this shape on the current device (no counterpart in the
 * reference, whose CUTLASS template picks nothing at run time): *kind = ARCQ_GEMM_KIND_PAIR (persistent
 * CTA pairs, 256 x 256 tiles), ARCQ_GEMM_KIND_SINGLE (one CTA per 128 x tile_n tile) or
 * ARCQ_GEMM_KIND_SPLIT_K (single-CTA tiles over *splits ranges of K; needs scratch).  *tile_n: tile
 * width; *splits: 1 unless split.  Any output pointer may be NULL. */
#define ARCQ_GEMM_KIND_SINGLE 0
#define ARCQ_GEMM_KIND_SPLIT_K 1
#define ARCQ_GEMM_KIND_PAIR 2
int arcq_matmul_plan(int64_t M, int64_t N, int64_t K_eff, int* kind, int* tile_n, int* splits);

/* No counterpart in the reference.  The split-K GEMM for callers that must not allocate device
 * memory: code that runs where an allocation would fail or stall - an inference-server plugin
 * whose enqueue hook is forbidden to call the allocator, a process whose whole device memory has
 * been handed to another framework's pool, a latency-critical loop where a cudaMalloc would
 * serialise the device.  Same arithmetic and same split as arcq_matmul_nvfp4_ws, but the fp32
 * partial sums live in a block of ARCQ_STATIC_SCRATCH_BYTES (2 MiB) that is part of the library
 * image itself; every GPU that loads the library holds that block until the process exits.  Inputs
 * and the output are still the caller's.  The call allocates nothing: no cudaMalloc / cudaFree, no
 * allocating library routine.
 *   - Shapes whose partial sums exceed the block (arcq_matmul_workspace_bytes(M,N,K_eff) >
 *     ARCQ_STATIC_SCRATCH_BYTES, e.g. M 128 x N 4096 x K_eff 14464) are refused with
 *     ARCQ_ERR_SCRATCH_LIMIT; shapes that are not split at all run without touching the block.
 *   - The first call on each device looks up the block's device address (one cudaGetSymbolAddress,
 *     with that device current); make that first call outside any stream capture.
 *   - All calls share the one block and it keeps whatever the previous call left.  Nothing in it
 *     needs clearing: every partial sum that is read was written earlier in the same call.  For the
 *     same reason two calls that overlap on the GPU (different streams, or different host threads
 *     on one device) race on it - serialise them on one stream. */
#define ARCQ_STATIC_SCRATCH_BYTES (2u << 20)
int arcq_matmul_nvfp4_static(const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB,
                             int64_t M, int64_t N, int64_t K_eff, float alpha, const float* alpha_a,
                             const float* alpha_b, void* C, void* stream);

/* The GEMM kernels and the quantizer bound every wait on a barrier; if one
 * ever expires the kernel records it and returns.  This reads (and clears)
 * those records for the current device: ARCQ_OK or ARCQ_ERR_TIMEOUT.
 * Synchronises the device. */
int arcq_gemm_poll_error(void);

/* One pass max|x| over n bf16 elements into *out (fp32, device memory; the
 * caller zero-fills it first or passes accumulate=0 to have it cleared by the
 * call).  Replaces the torch.max(x.abs()) pass of model/qLlamaLayer.py:74. */
int arcq_absmax_bf16(const void* x, int64_t n, float* out, int accumulate, void* stream);

/* Layer glue between the quantized linears.  No counterpart in the reference's bindings: its layers
 * call torch for these (Hugging Face apply_rotary_pos_emb and act_fn(gate) * up in
 * model/qLlamaLayer.py).  Results equal eager torch bit for bit FOR THE FORMULAS WRITTEN BELOW.  For the
 * rotary embedding that formula keeps cos and sin in fp32 and rounds once; Hugging Face's
 * apply_rotary_pos_emb, which the reference layer calls, multiplies by bf16 cos / sin and rounds each
 * product and the sum to bf16, so a layer output agrees with the reference layer's within bf16 rounding
 * at this step, not bit for bit.
 *
 * arcq_rope_bf16: rotate-half rotary embedding, in place, on the first `heads` heads of `head_dim`
 *   elements of every row of x [tokens, row_elems] (bf16; e.g. the q and k columns of a fused qkv
 *   output).  cos_table / sin_table: fp32 [seq, head_dim], row = token % seq.
 *   out = bf16(fp32(x * cos) + fp32(rotate_half(x) * sin)).  head_dim % 16 == 0.
 * arcq_silu_mul_bf16: out [tokens, F] = bf16(bf16(silu(gate)) * up) for gate_up [tokens, 2F] = [gate | up]
 *   (bf16); if amax is not NULL it receives max |out| (fp32, device memory) - the per-tensor maximum the
 *   next activation quantizer's global scale is made of.  F % 8 == 0. */
int arcq_rope_bf16(void* x, const float* cos_table, const float* sin_table, int64_t tokens, int row_elems, int heads,
                   int head_dim, int seq, void* stream);
int arcq_silu_mul_bf16(const void* gate_up, void* out, int64_t tokens, int F, float* amax, void* stream);

/* Weighted sum of the routed copies of each token after the experts of a sparse MoE block (the
 * `final_hidden_states.index_add_(0, top_x, expert_out * routing_weight)` of the reference's
 * model/qMixtralLayer.py:466-471, as one gather instead of one scatter-add per expert; no counterpart
 * in the reference's bindings).  y [rows, hidden] bf16: expert outputs; pos [tokens, top_k] int32: the
 * row of y holding copy j of token t; weights [tokens, top_k] bf16; out [tokens, hidden] bf16 =
 * sum_j bf16(y[pos[t][j]] * weights[t][j]), products and running sum rounded to bf16.  hidden % 8 == 0. */
int arcq_moe_combine_bf16(const void* y, const int32_t* pos, const void* weights, void* out, int64_t tokens, int hidden,
                          int top_k, void* stream);

/* Calibration statistics of a batch of activations x [rows, K] (bf16) in one pass, accumulated into
 * running values in device memory (the caller zero-fills them before the first batch):
 *   chan_absmax [K] fp32: per-channel max |x| - the statistic the reference's get_act_stats keeps with its
 *     max metric (utilize.py:108) and reorders the channels by (utilize.py:42);
 *   above (may be NULL): number of elements larger than an eighth of their row's (signed) maximum - the
 *     numerator of the select_num rule (utilize.py:546-547); the caller divides by rows * K.
 * Replaces torch's abs / amax / max / compare passes over the same tensor.  K % 8 == 0, K <= 32768. */
int arcq_calib_stats_bf16(const void* x, int64_t rows, int K, float* chan_absmax, unsigned long long* above,
                          void* stream);

/* ---- Grouped forms: all experts of a sparse MoE block in one launch ---------------------------------
 * The reference runs its experts one after another from Python, each with its own quantize and GEMM
 * calls on that expert's batch of tokens (model/qMixtralLayer.py:458-471, 524-543).  Here the routed
 * rows of all experts lie in ONE buffer, expert after expert ("runs"), every run starting at a multiple
 * of 256 rows; how many rows each run holds is known on the device only:
 *   groups    int32 [2*ngroups] in device memory: groups[e] = first row of run e (a multiple of 256),
 *             groups[ngroups + e] = its number of rows.  Rows between runs are padding: never read as
 *             results, their content is unspecified.
 *   row_map   int32 per (padded) row, or NULL: the row of x that row holds (the dispatch gather is
 *             folded into the loads).
 * No counterpart in the reference's bindings.
 *
 * arcq_absmax_grouped_bf16: out[e] = max|x| over the rows of run e (the per-call global scale of
 *   NVFP4_reorder_quantize_x, per expert).
 * arcq_reorder_quantize_x_grouped: arcq_reorder_quantize_x_scaled on every run with its own divisor
 *   scales[e] and its own channel order reorder_indices + e*KQ (int16 [ngroups, KQ]).  rows_bound: rows of
 *   the output buffers (>= end of the last run).  Row widths as arcq_reorder_quantize_x_scaled.
 * arcq_matmul_nvfp4_grouped: C[r, :] = alpha_a[e]*alpha_b[e] * A[r, :] . B_e^T for the rows r of run e;
 *   B [ngroups*N, K_eff/2] and SFB hold the experts' packed weights one after another (N % 128 == 0);
 *   tile_group int32 [ceil(M_bound/256)] in device memory: the run that owns each 256-row tile of A, or
 *   a negative number for a tile without rows (skipped).  alpha_b may be NULL. */
/* The padded layout itself, computed on the device in one small launch (no counterpart in the reference,
 * whose Python loop asks torch.where for every expert's rows, model/qMixtralLayer.py:458-466).
 * slot_group int64 [n]: the run (local expert) of every slot - a routed copy (token, j) or a row of the
 * receive buffer - or a value outside [0, ngroups) for a slot that belongs to nobody.  Outputs, all int32
 * in device memory: dest [n] = padded row of every slot (rows_bound for nobody); row_map [rows_bound] =
 * slot / div of the slot every padded row holds (0 for padding; div = top_k turns copies into tokens);
 * groups [2*ngroups]; tile_group [rows_bound / tile].  Slots of one run keep their order.
 * rows_bound must be a multiple of tile and at least n rounded up to a tile plus ngroups * tile;
 * n <= 1 << 20, ngroups <= 64. */
int arcq_moe_layout(const int64_t* slot_group, int n, int ngroups, int tile, int rows_bound, int div, int32_t* dest,
                    int32_t* row_map, int32_t* groups, int32_t* tile_group, void* stream);
/* arcq_silu_mul_grouped_bf16: arcq_silu_mul_bf16 over grouped rows: 256-row tiles that tile_group marks
 *   as empty are skipped altogether, and amax[e] (fp32 [ngroups], may be NULL) receives max|out| over the
 *   rows of run e - the down projection's per-expert global scale - in the same pass.  F % 256 == 0. */
int arcq_silu_mul_grouped_bf16(const void* gate_up, void* out, int64_t rows_bound, int F, const int32_t* tile_group,
                               const int32_t* groups, int ngroups, float* amax, void* stream);
int arcq_absmax_grouped_bf16(const void* x, const int32_t* row_map, const int32_t* groups, int ngroups, int K,
                             float* out, void* stream);
int arcq_reorder_quantize_x_grouped(const void* x, const int32_t* row_map, const float* scales,
                                    const int16_t* reorder_indices, const int32_t* groups, int ngroups,
                                    int64_t rows_bound, int KQ, int KE, int mode, uint8_t* qx, uint8_t* sfx,
                                    void* stream);
int arcq_matmul_nvfp4_grouped(const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB,
                              int64_t M_bound, int64_t N, int64_t K_eff, const int32_t* tile_group, int ngroups,
                              const float* alpha_a, const float* alpha_b, void* C, void* stream);

/* ---- Gate/up projection with the SwiGLU fused into the GEMM's epilogue -------------------------------
 * The reference runs gate_proj and up_proj as two GEMMs and then `act_fn(gate) * up` in torch
 * (model/qLlamaLayer.py:432-436, model/qMixtralLayer.py:536-539).  Here B holds both weights, interleaved
 * in blocks of 128 output channels - rows [256 t, 256 t + 128) of B are gate channels [128 t, 128 t + 128),
 * rows [256 t + 128, 256 t + 256) the same up channels - so one output tile holds matching gate and up
 * columns and the epilogue writes C [M, N/2] = bf16(bf16(silu(g)) * u) directly, g and u being the
 * bf16-rounded GEMM results: the same bits as arcq_matmul_nvfp4 followed by arcq_silu_mul_bf16, without the
 * [M, N] round trip through memory.  amax (fp32, device) receives max|C| over the valid rows - the
 * per-tensor maximum the down projection's quantizer needs.  N % 256 == 0.  Always runs the CTA-pair
 * kernel (meant for prefill-sized M).
 * arcq_matmul_nvfp4_grouped_swiglu: the same over the runs of a grouped problem (see above); amax has one
 * entry per run and `groups` says where each run's valid rows end. */
int arcq_matmul_nvfp4_swiglu(const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB,
                             int64_t M, int64_t N, int64_t K_eff, const float* alpha_a, const float* alpha_b,
                             void* C, float* amax, void* stream);
int arcq_matmul_nvfp4_grouped_swiglu(const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB,
                                     int64_t M_bound, int64_t N, int64_t K_eff, const int32_t* tile_group,
                                     const int32_t* groups, int ngroups, const float* alpha_a, const float* alpha_b,
                                     void* C, float* amax, void* stream);

/* ---- Projection with the residual addition in the GEMM's epilogue ---------------------------------------
 * The reference adds the residual stream in torch after o_proj and down_proj (`residual + hidden_states`,
 * model/qLlamaLayer.py:162, 168).  arcq_matmul_nvfp4_residual writes C = bf16(R + bf16(alpha_a * alpha_b *
 * A B^T)) - the bits of that addition - with R (bf16 [M, N], may be C itself) fetched tile by tile in the
 * epilogue instead of a pass of its own over [M, N].  Always the CTA-pair kernel (meant for prefill-sized M). */
int arcq_matmul_nvfp4_residual(const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB, int64_t M,
                               int64_t N, int64_t K_eff, const float* alpha_a, const float* alpha_b,
                               const void* residual, void* C, void* stream);

/* ---- Row-parallel projection fused with its reduce-scatter over peer memory -----------------------------
 * No counterpart in the reference (it runs on one GPU: o_proj and down_proj at model/qLlamaLayer.py:363-366, 439-443); these serve the
 * tensor-parallel form of its decoder layer, where the o and down projections are sharded by K and their
 * partial results must be added over the ranks, each rank keeping the token rows it owns.
 *
 * arcq_matmul_nvfp4_scatter: the GEMM of arcq_matmul_nvfp4_dev_alpha whose epilogue stores rows
 *   [d * M / ndests, (d + 1) * M / ndests) of the result into dests[d], a bf16 [M / ndests, N] buffer of its
 *   own (host array of ndests <= 8 device addresses).  In a tensor-parallel group dests[d] is this rank's
 *   receive slot in the memory of rank d (an address obtained with arcq_peer_open, or local memory for
 *   d == this rank): every output tile leaves for its owner over NVLink as soon as it is computed, while the
 *   tensor cores work on the next tile.  M % ndests == 0, (M / ndests) % 32 == 0.  Always the CTA-pair kernel.
 * arcq_sum_partials_bf16: out = residual + bf16(srcs[0] + ... + srcs[n-1]) over `elems` bf16 elements
 *   (fp32 accumulation in the order given, one rounding, then the bf16 residual addition; residual may be
 *   NULL): what a rank runs over its n receive slots once every peer's GEMM has finished (the caller orders
 *   that, e.g. with a barrier of its communication library on the same stream).  srcs: host array of n <= 8
 *   device addresses; elems % 8 == 0.
 * arcq_peer_alloc / _free: device memory from cudaMalloc (not from a framework's pool), which is what
 *   arcq_peer_export can describe; _export writes the 64-byte handle another process on the same machine
 *   passes to arcq_peer_open, which maps the block into the calling process and enables peer access from the
 *   current device; _close unmaps it.  Handles travel by any host channel (the Python layer uses its process
 *   group's all_gather_object).
 * arcq_rmsnorm_quantize_x_multi: arcq_rmsnorm_quantize_x into (qx[0], sfx[0]), followed on the same stream by
 *   a copy of the codes and of the rows' scale tiles to (qx[d], sfx[d]), 0 < d < ndests <= 8 - host arrays of
 *   device addresses; in a sequence-parallel group the places of this rank's token rows in every rank's
 *   gathered code and scale buffers (M a multiple of 128, so that the rows' scale tiles are whole).  With a
 *   barrier behind it this is the all-gather in front of a column-parallel projection, written as stores
 *   into the peers' memory.
 * arcq_peer_barrier: all ranks of the group have finished the work that precedes the call in their streams
 *   before work that follows it in any rank's stream starts.  flags: host array of `world` device addresses,
 *   flags[d] = rank d's block of `world` 32-bit words (zeroed once, before the handles are exchanged; peers'
 *   blocks opened with arcq_peer_open); counter: a zero-initialised 32-bit word in this rank's memory that
 *   counts its barriers (every rank must issue the same sequence of barriers).  One small kernel; its wait is
 *   bounded (10 s; arcq_peer_set_wait_limit_ms changes the limit for later launches of this process and
 *   returns the previous one), after which the kernel returns and arcq_peer_poll_error() reports
 *   ARCQ_ERR_TIMEOUT (it synchronises the device and clears the record): a rank that never arrives costs its
 *   peers that wait, not the GPU.
 * arcq_ep_send_layout / arcq_ep_rows: the dispatch of an expert-parallel MoE block (the loop over experts of
 *   model/qMixtralLayer.py:458-471 spread over `ep` ranks with e_local experts each) as stores into the peers'
 *   memory instead of all-to-all collectives.  _send_layout (one small launch): copy i of this rank's n routed
 *   copies, global expert ids[i], gets the next free place j of this rank's block of `cap` places in the receive
 *   buffer of rank d = ids[i] / e_local: slot[i] = d * cap + j, and the place's local expert goes into rank d's
 *   slot table, slot_tables[d][rank * cap + j] (int64; free places of the block receive e_local = nobody - the
 *   form arcq_moe_layout reads).  Copies beyond the capacity are dropped (slot[i] = ep * cap, *overflow = 1).
 *   _rows: one warp per item copies a row of `row_bytes` from src to place rank * cap + s % cap of the buffer
 *   dst[s / cap], s = item_slot ? item_slot[i] : i (skipped when s >= ep * cap), reading row item_src ?
 *   item_src[i] : i / div (skipped when >= src_limit): token rows to the experts' ranks, and the experts' output
 *   rows back to the ranks of their tokens.  A barrier (arcq_peer_barrier) follows each. */
#define ARCQ_PEER_HANDLE_BYTES 64
int arcq_ep_send_layout(const int64_t* ids, int n, int e_local, int ep, int cap, int rank, int32_t* slot,
                        void* const* slot_tables, int32_t* overflow, void* stream);
int arcq_ep_rows(const void* src, const int32_t* item_src, int div, int src_limit, const int32_t* item_slot, int n,
                 int row_bytes, int cap, int ep, int rank, void* const* dst, void* stream);
int arcq_rmsnorm_quantize_x_multi(const void* x, const void* gamma, float eps, const int16_t* reorder_index,
                                  int64_t M, int KQ, int KE, uint8_t* const* qx, uint8_t* const* sfx, int ndests,
                                  void* stream);
int arcq_peer_barrier(void* const* flags, int rank, int world, uint32_t* counter, void* stream);
int arcq_peer_poll_error(void);
int arcq_peer_set_wait_limit_ms(int ms);
int arcq_matmul_nvfp4_scatter(const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB, int64_t M,
                              int64_t N, int64_t K_eff, const float* alpha_a, const float* alpha_b,
                              void* const* dests, int ndests, void* stream);
int arcq_sum_partials_bf16(const void* const* srcs, int n, int64_t elems, const void* residual, void* out,
                           void* stream);
int arcq_peer_alloc(size_t bytes, void** ptr);
int arcq_peer_free(void* ptr);
int arcq_peer_export(void* ptr, unsigned char* handle);
int arcq_peer_open(const unsigned char* handle, void** ptr);
int arcq_peer_close(void* ptr);

#ifdef __cplusplus
}
#endif
#endif /* ARCQ_H_ */
