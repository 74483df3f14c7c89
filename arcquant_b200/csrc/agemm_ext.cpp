// Python extension module `agemm`: the operator surface of ARCQuant's torch extension
// (kernels/src/bindings.cpp:551-582) on top of libarcq.so's C ABI.  Same function names, argument
// order and return types for the four quantized-linear operators; outputs are allocated here with
// torch::empty, inputs are borrowed, kernels run on torch's current CUDA stream.  The reference's
// KV-cache operators (batch_decode_*, init_kv_*, append_kv_*) are not part of this library.
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include <sstream>
#include <stdexcept>
#include <tuple>

#include "arcq.h"

namespace {

void check_status(int status, const char* where) {
  if (status == ARCQ_OK) return;
  std::ostringstream os;
  os << "Value error in " << where << ": " << arcq_status_string(status);
  if (status == ARCQ_ERR_CUDA) os << " (cudaError " << arcq_last_cuda_error() << ")";
  throw std::runtime_error(os.str());
}

void* current_stream(const torch::Tensor& t) {
  return static_cast<void*>(c10::cuda::getCurrentCUDAStream(t.device().index()).stream());
}

void require_cuda(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor (this library has no CPU path)");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}
// Every tensor a kernel will dereference: on the device of `like`, contiguous, of the given type.
void require_on(const torch::Tensor& t, const torch::Tensor& like, at::ScalarType type, const char* name) {
  require_cuda(t, name);
  TORCH_CHECK(t.device() == like.device(), name, " must be on the same device as the first operand");
  TORCH_CHECK(t.scalar_type() == type, name, ": expected ", type, ", got ", t.scalar_type());
}
void require_scalar_f32(const torch::Tensor& t, const torch::Tensor& like, const char* name) {
  require_on(t, like, at::kFloat, name);
  TORCH_CHECK(t.numel() == 1, name, " must hold one fp32 value");
}
// Shapes of a block-scaled GEMM's operands; returns M, N, K_eff.
std::tuple<int64_t, int64_t, int64_t> check_gemm_operands(const torch::Tensor& A, const torch::Tensor& B,
                                                          const torch::Tensor& SFA, const torch::Tensor& SFB) {
  require_cuda(A, "A");
  TORCH_CHECK(A.scalar_type() == at::kByte, "A: expected uint8 packed codes");
  require_on(B, A, at::kByte, "B");
  require_on(SFA, A, at::kByte, "SFA");
  require_on(SFB, A, at::kByte, "SFB");
  TORCH_CHECK(A.dim() == 2 && B.dim() == 2, "A and B must be 2-D [rows, K_eff/2]");
  TORCH_CHECK(A.size(1) == B.size(1), "A and B disagree on K");
  const int64_t M = A.size(0), N = B.size(0), K = A.size(1) * 2;
  // what the kernels read: whole 512-byte atoms of every 128-row tile
  const int64_t atoms = (K / 16 + 3) / 4;
  TORCH_CHECK(SFA.numel() >= ((M + 127) / 128) * atoms * 512, "SFA is smaller than the scale layout of A");
  TORCH_CHECK(SFB.numel() >= ((N + 127) / 128) * atoms * 512, "SFB is smaller than the scale layout of B");
  return std::make_tuple(M, N, K);
}

std::tuple<torch::Tensor, torch::Tensor> quantize_common(const torch::Tensor& X, const torch::Tensor* gamma,
                                                         float eps, const torch::Tensor& reorder_index, int KE,
                                                         bool is_weight, const char* where) {
  require_cuda(X, "input");
  require_on(reorder_index, X, at::kShort, "reorder_index");
  TORCH_CHECK(X.dim() == 2, "input must be 2-D");
  const int64_t rows = X.size(0);
  const int KQ = static_cast<int>(X.size(1));
  const int K = KQ + KE;
  TORCH_CHECK(KE >= 0 && KE <= KQ, "KE must lie in [0, KQ]");
  TORCH_CHECK(reorder_index.numel() == KQ, "reorder_index must have KQ entries");
  c10::cuda::CUDAGuard guard(X.device());
  auto options = torch::dtype(torch::kUInt8).device(X.device());
  auto Q = torch::empty({rows, K / 2}, options);
  auto SF = torch::empty({static_cast<int64_t>(arcq_sf_bytes(rows, K))}, options);
  const void* px = X.data_ptr<at::BFloat16>();                 // throws on a wrong dtype, as the reference does
  const int16_t* pidx = reorder_index.data_ptr<int16_t>();
  int status;
  if (gamma) {
    require_on(*gamma, X, at::kBFloat16, "weight");
    TORCH_CHECK(gamma->numel() == KQ, "weight must have KQ entries");
    status = arcq_rmsnorm_quantize_x(px, gamma->data_ptr<at::BFloat16>(), eps, pidx, rows, KQ, KE,
                                     Q.data_ptr<uint8_t>(), SF.data_ptr<uint8_t>(), current_stream(X));
  } else if (is_weight) {
    status = arcq_reorder_quantize_w(px, pidx, rows, KQ, KE, arcq_reference_mode(KQ), Q.data_ptr<uint8_t>(),
                                     SF.data_ptr<uint8_t>(), current_stream(X));
  } else {
    status = arcq_reorder_quantize_x(px, pidx, rows, KQ, KE, arcq_reference_mode(KQ), Q.data_ptr<uint8_t>(),
                                     SF.data_ptr<uint8_t>(), current_stream(X));
  }
  check_status(status, where);
  return std::make_tuple(Q, SF);
}

torch::Tensor matmul(const torch::Tensor& A, const torch::Tensor& B, const torch::Tensor& SFA,
                     const torch::Tensor& SFB, const float scale) {
  int64_t M, N, K;
  std::tie(M, N, K) = check_gemm_operands(A, B, SFA, SFB);
  c10::cuda::CUDAGuard guard(A.device());
  auto C = torch::empty({M, N}, torch::dtype(torch::kBFloat16).device(A.device()));
  // skinny problems split K over idle SMs; the fp32 partial sums need scratch
  const int64_t ws_bytes = static_cast<int64_t>(arcq_matmul_workspace_bytes(M, N, K));
  torch::Tensor ws;
  if (ws_bytes > 0) ws = torch::empty({ws_bytes}, torch::dtype(torch::kUInt8).device(A.device()));
  int status = arcq_matmul_nvfp4_ws(A.data_ptr<uint8_t>(), B.data_ptr<uint8_t>(), SFA.data_ptr<uint8_t>(),
                                    SFB.data_ptr<uint8_t>(), M, N, K, scale, nullptr, nullptr,
                                    C.data_ptr<at::BFloat16>(), ws_bytes > 0 ? ws.data_ptr() : nullptr,
                                    static_cast<size_t>(ws_bytes), current_stream(A));
  check_status(status, "matmul_host_nvfp4_bf16");
  return C;
}

// Extra: alpha = alpha_a * alpha_b read on the device (0-dim fp32 CUDA tensors), no host sync.
torch::Tensor matmul_dev_alpha(const torch::Tensor& A, const torch::Tensor& B, const torch::Tensor& SFA,
                               const torch::Tensor& SFB, const torch::Tensor& alpha_a,
                               const c10::optional<torch::Tensor>& alpha_b) {
  int64_t M, N, K;
  std::tie(M, N, K) = check_gemm_operands(A, B, SFA, SFB);
  require_scalar_f32(alpha_a, A, "alpha_a");
  if (alpha_b.has_value()) require_scalar_f32(*alpha_b, A, "alpha_b");
  c10::cuda::CUDAGuard guard(A.device());
  auto C = torch::empty({M, N}, torch::dtype(torch::kBFloat16).device(A.device()));
  // skinny problems split K over idle SMs; the fp32 partial sums need scratch
  const int64_t ws_bytes = static_cast<int64_t>(arcq_matmul_workspace_bytes(M, N, K));
  torch::Tensor ws;
  if (ws_bytes > 0) ws = torch::empty({ws_bytes}, torch::dtype(torch::kUInt8).device(A.device()));
  int status = arcq_matmul_nvfp4_ws(
      A.data_ptr<uint8_t>(), B.data_ptr<uint8_t>(), SFA.data_ptr<uint8_t>(), SFB.data_ptr<uint8_t>(), M, N, K, 1.0f,
      alpha_a.data_ptr<float>(), alpha_b.has_value() ? alpha_b->data_ptr<float>() : nullptr,
      C.data_ptr<at::BFloat16>(), ws_bytes > 0 ? ws.data_ptr() : nullptr, static_cast<size_t>(ws_bytes),
      current_stream(A));
  check_status(status, "matmul_host_nvfp4_bf16");
  return C;
}

std::tuple<torch::Tensor, torch::Tensor> reorder_quantize_x(const torch::Tensor& X,
                                                            const torch::Tensor& reorder_index, const int KE) {
  return quantize_common(X, nullptr, 0.f, reorder_index, KE, false, "run_reorder_x_bf16_nvfp4");
}

std::tuple<torch::Tensor, torch::Tensor> reorder_quantize_w(const torch::Tensor& W,
                                                            const torch::Tensor& reorder_index, const int KE) {
  return quantize_common(W, nullptr, 0.f, reorder_index, KE, true, "run_reorder_w_bf16_nvfp4");
}

std::tuple<torch::Tensor, torch::Tensor> rmsnorm_quantize_x(const torch::Tensor& X, const torch::Tensor& W,
                                                            const float eps, const torch::Tensor& reorder_index,
                                                            const int KE) {
  return quantize_common(X, &W, eps, reorder_index, KE, false, "run_rmsnorm_x_bf16_nvfp4");
}

// ---- extras without a counterpart in the reference's bindings (its layers call torch for these) ----

// reorder_quantize_x on X / scale (scale: 0-dim fp32 CUDA tensor), the division fused into the kernel
// where the row width allows it, done with torch first where it does not.  mode < 0: the reference's
// choice for this KQ.
std::tuple<torch::Tensor, torch::Tensor> reorder_quantize_x_scaled(const torch::Tensor& X, const torch::Tensor& scale,
                                                                   const torch::Tensor& reorder_index, const int KE,
                                                                   int mode) {
  require_cuda(X, "input");
  require_on(reorder_index, X, at::kShort, "reorder_index");
  require_scalar_f32(scale, X, "scale");
  TORCH_CHECK(X.dim() == 2, "input must be 2-D");
  const int64_t rows = X.size(0);
  const int KQ = static_cast<int>(X.size(1));
  const int K = KQ + KE;
  TORCH_CHECK(KE >= 0 && KE <= KQ, "KE must lie in [0, KQ]");
  TORCH_CHECK(reorder_index.numel() == KQ, "reorder_index must have KQ entries");
  if (mode < 0) mode = arcq_reference_mode(KQ);
  c10::cuda::CUDAGuard guard(X.device());
  auto options = torch::dtype(torch::kUInt8).device(X.device());
  auto Q = torch::empty({rows, K / 2}, options);
  auto SF = torch::empty({static_cast<int64_t>(arcq_sf_bytes(rows, K))}, options);
  int status = arcq_reorder_quantize_x_scaled(X.data_ptr<at::BFloat16>(), scale.data_ptr<float>(),
                                              reorder_index.data_ptr<int16_t>(), rows, KQ, KE, mode,
                                              Q.data_ptr<uint8_t>(), SF.data_ptr<uint8_t>(), current_stream(X));
  if (status == ARCQ_ERR_UNSUPPORTED_K) {
    auto Xs = X / scale;
    status = arcq_reorder_quantize_x(Xs.data_ptr<at::BFloat16>(), reorder_index.data_ptr<int16_t>(), rows, KQ, KE, mode,
                                     Q.data_ptr<uint8_t>(), SF.data_ptr<uint8_t>(), current_stream(X));
  }
  check_status(status, "run_reorder_x_bf16_nvfp4");
  return std::make_tuple(Q, SF);
}

std::tuple<torch::Tensor, torch::Tensor> silu_mul(const torch::Tensor& GU) {
  require_cuda(GU, "gate_up");
  TORCH_CHECK(GU.dim() == 2 && GU.size(1) % 16 == 0, "gate_up must be [tokens, 2F] with F a multiple of 8");
  c10::cuda::CUDAGuard guard(GU.device());
  const int64_t tokens = GU.size(0);
  const int F = static_cast<int>(GU.size(1) / 2);
  auto out = torch::empty({tokens, F}, torch::dtype(torch::kBFloat16).device(GU.device()));
  auto amax = torch::empty({}, torch::dtype(torch::kFloat32).device(GU.device()));
  check_status(arcq_silu_mul_bf16(GU.data_ptr<at::BFloat16>(), out.data_ptr<at::BFloat16>(), tokens, F,
                                  amax.data_ptr<float>(), current_stream(GU)),
               "silu_mul");
  return std::make_tuple(out, amax);
}

torch::Tensor rope_inplace(torch::Tensor X, const torch::Tensor& cos_t, const torch::Tensor& sin_t, int heads,
                           int head_dim) {
  require_cuda(X, "x");
  require_on(cos_t, X, at::kFloat, "cos");
  require_on(sin_t, X, at::kFloat, "sin");
  TORCH_CHECK(X.dim() == 2 && cos_t.dim() == 2 && cos_t.size(1) == head_dim && cos_t.sizes() == sin_t.sizes(),
              "x must be [tokens, row]; cos / sin [seq, head_dim]");
  c10::cuda::CUDAGuard guard(X.device());
  check_status(arcq_rope_bf16(X.data_ptr<at::BFloat16>(), cos_t.data_ptr<float>(), sin_t.data_ptr<float>(), X.size(0),
                              static_cast<int>(X.size(1)), heads, head_dim, static_cast<int>(cos_t.size(0)),
                              current_stream(X)),
               "rope");
  return X;
}

torch::Tensor absmax(const torch::Tensor& X) {
  require_cuda(X, "input");
  c10::cuda::CUDAGuard guard(X.device());
  auto out = torch::empty({}, torch::dtype(torch::kFloat32).device(X.device()));
  check_status(arcq_absmax_bf16(X.data_ptr<at::BFloat16>(), X.numel(), out.data_ptr<float>(), 0, current_stream(X)),
               "absmax");
  return out;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("matmul", &matmul, "our ARC gemm (sm_100a)", py::arg("A"), py::arg("B"), py::arg("SFA"), py::arg("SFB"),
        py::arg("scale"));
  m.def("reorder_quantize_x", &reorder_quantize_x, "Reorder and quantize activation.", py::arg("X"),
        py::arg("reorder_index"), py::arg("KE"));
  m.def("reorder_quantize_w", &reorder_quantize_w, "Reorder and quantize weight.", py::arg("W"),
        py::arg("reorder_index"), py::arg("KE"));
  m.def("rmsnorm_quantize_x", &rmsnorm_quantize_x, "RMSNorm, reorder and quantize activation.", py::arg("X"),
        py::arg("W"), py::arg("eps"), py::arg("reorder_index"), py::arg("KE"));
  m.def("matmul_dev_alpha", &matmul_dev_alpha, "gemm with device-resident global scales", py::arg("A"),
        py::arg("B"), py::arg("SFA"), py::arg("SFB"), py::arg("alpha_a"), py::arg("alpha_b") = py::none());
  m.def("reorder_quantize_x_scaled", &reorder_quantize_x_scaled, "reorder_quantize_x of X / scale (device scalar)",
        py::arg("X"), py::arg("scale"), py::arg("reorder_index"), py::arg("KE"), py::arg("mode") = -1);
  m.def("silu_mul", &silu_mul, "(silu(gate) * up, max|.|) of [gate | up]", py::arg("gate_up"));
  m.def("rope_inplace", &rope_inplace, "rotate-half rotary embedding in place on the first heads of each row",
        py::arg("X"), py::arg("cos"), py::arg("sin"), py::arg("heads"), py::arg("head_dim"));
  m.def("absmax", &absmax, "max|x| of a bf16 tensor as a 0-dim fp32 tensor", py::arg("X"));
  m.def("sf_bytes", [](int64_t rows, int64_t k_eff) { return static_cast<int64_t>(arcq_sf_bytes(rows, k_eff)); },
        "bytes of a scale-factor buffer");
}
