// torch.library shim: registers the `tensorrt::` operators of the quantized-linear hot
// path on top of the b200q C ABI.  No kernels live here; every op validates its
// arguments the way the reference converters do, allocates outputs through the torch
// caching allocator, and enqueues one or more b200q_* calls on the current CUDA stream.
//
// The reference's C++ runtime owns TORCH_LIBRARY(tensorrt, ...)
// (core/runtime/register_jit_hooks.cpp:193-194), and its Python side adds further ops to
// the same namespace through FRAGMENT libraries
// (py/torch_tensorrt/dynamo/lowering/passes/fuse_distributed_ops.py:57), so this file
// uses TORCH_LIBRARY_FRAGMENT.  The two quantize ops keep the positional schemas the
// reference calls them with (tests/py/dynamo/models/test_models_export.py:789;
// py/torch_tensorrt/dynamo/conversion/aten_ops_converters.py:948-960); they are defined
// here only when no other package has defined them already.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <ATen/core/dispatch/Dispatcher.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <cmath>
#include <optional>
#include <tuple>

#include "b200q.h"

namespace {

using at::Tensor;

void check_status(int rc, const char* what) {
  TORCH_CHECK(rc == B200Q_OK, what, " failed: ", b200q_status_string(rc), " (status ", rc, ")");
}

int dtype_code(const Tensor& t, const char* op) {
  switch (t.scalar_type()) {
    case at::kFloat: return B200Q_F32;
    case at::kHalf: return B200Q_F16;
    case at::kBFloat16: return B200Q_BF16;
    default:
      TORCH_CHECK_VALUE(false, op, " received an input of ", t.scalar_type(),
                        " type. Supported types: float32 | float16 | bfloat16");
  }
}

b200q_stream_t current_stream() { return static_cast<b200q_stream_t>(at::cuda::getCurrentCUDAStream().stream()); }

Tensor as_f32_cuda(const Tensor& t, const Tensor& like) {
  return t.to(like.device(), at::kFloat).contiguous();
}

int64_t rows_of(const Tensor& x) { return x.dim() == 0 ? 1 : x.numel() / std::max<int64_t>(x.size(-1), 1); }
int64_t cols_of(const Tensor& x) { return x.dim() == 0 ? 1 : x.size(-1); }

// amax granularity: 1 value -> per tensor; one value per row of the flattened [rows, cols] view.
int64_t amax_numel_for(const Tensor& x, const Tensor& amax, const char* op) {
  const int64_t n = amax.numel();
  if (n == 1) return 1;
  TORCH_CHECK(n == rows_of(x), op, ": amax must hold one value (per-tensor) or one value per row of the input (",
              rows_of(x), "), got shape ", amax.sizes());
  return n;
}

// ------------------------------------------------------------------ reference-schema ops (fake quant)
Tensor quantize_op_cuda(const Tensor& input, const Tensor& amax, int64_t num_bits, int64_t exponent_bits,
                        bool /*unsigned_*/, bool /*narrow_range*/) {
  const int dt = dtype_code(input, "quantize_op");
  TORCH_CHECK_VALUE(num_bits == 8 && exponent_bits == 4,
                    "quantize_op on this device path only accepts FP8 E4M3 (num_bits=8, exponent_bits=4), got num_bits=",
                    num_bits, ", exponent_bits=", exponent_bits);
  c10::cuda::CUDAGuard guard(input.device());
  Tensor x = input.contiguous();
  Tensor out = at::empty_like(x);
  if (x.numel() == 0) return out;
  TORCH_CHECK(cols_of(x) % 8 == 0, "quantize_op: last dimension must be a multiple of 8, got ", cols_of(x));
  Tensor a = as_f32_cuda(amax, x);
  check_status(b200q_fp8_fake_quantize(x.data_ptr(), dt, rows_of(x), cols_of(x), a.data_ptr<float>(),
                                       amax_numel_for(x, a, "quantize_op"), out.data_ptr(), current_stream()),
               "b200q_fp8_fake_quantize");
  return out;
}

Tensor quantize_op_meta(const Tensor& input, const Tensor&, int64_t, int64_t, bool, bool) { return at::empty_like(input); }

void check_nvfp4_args(int64_t block_size, int64_t num_bits, int64_t exponent_bits, int64_t scale_num_bits,
                      int64_t scale_exponent_bits) {
  TORCH_CHECK_VALUE(block_size == 16 && num_bits == 4 && exponent_bits == 2 && scale_num_bits == 8 && scale_exponent_bits == 4,
                    "dynamic_block_quantize_op only accepts NVFP4: block_size=16, (num_bits, exponent_bits)=(4, 2), "
                    "(scale_num_bits, scale_exponent_bits)=(8, 4); got block_size=",
                    block_size, ", (", num_bits, ", ", exponent_bits, "), (", scale_num_bits, ", ", scale_exponent_bits, ")");
}

Tensor dynamic_block_quantize_op_cuda(const Tensor& input, int64_t block_size, const Tensor& amax, int64_t num_bits,
                                      int64_t exponent_bits, int64_t scale_num_bits, int64_t scale_exponent_bits) {
  const int dt = dtype_code(input, "dynamic_block_quantize_op");
  check_nvfp4_args(block_size, num_bits, exponent_bits, scale_num_bits, scale_exponent_bits);
  TORCH_CHECK(amax.numel() == 1, "dynamic_block_quantize_op: amax should be a scalar, got shape ", amax.sizes());
  c10::cuda::CUDAGuard guard(input.device());
  Tensor x = input.contiguous();
  Tensor out = at::empty_like(x);
  if (x.numel() == 0) return out;
  TORCH_CHECK_VALUE(cols_of(x) % 16 == 0, "dynamic_block_quantize_op: last dimension (", cols_of(x),
                    ") must be a multiple of the block size 16");
  Tensor a = as_f32_cuda(amax, x);
  check_status(b200q_nvfp4_fake_quantize(x.data_ptr(), dt, rows_of(x), cols_of(x), a.data_ptr<float>(), out.data_ptr(),
                                         current_stream()),
               "b200q_nvfp4_fake_quantize");
  return out;
}

Tensor dynamic_block_quantize_op_meta(const Tensor& input, int64_t, const Tensor&, int64_t, int64_t, int64_t, int64_t) {
  return at::empty_like(input);
}

// ------------------------------------------------------------------ real-quant building blocks
Tensor amax_cuda(const Tensor& input) {
  const int dt = dtype_code(input, "b200_amax");
  c10::cuda::CUDAGuard guard(input.device());
  Tensor x = input.contiguous();
  Tensor out = at::zeros({}, x.options().dtype(at::kFloat));
  if (x.numel() == 0) return out;
  Tensor ws = at::zeros({static_cast<int64_t>(b200q_amax_workspace_bytes())}, x.options().dtype(at::kByte));
  check_status(b200q_amax(x.data_ptr(), dt, x.numel(), out.data_ptr<float>(), ws.data_ptr(), ws.numel(), current_stream()),
               "b200q_amax");
  return out;
}
Tensor amax_meta(const Tensor& input) { return at::empty({}, input.options().dtype(at::kFloat)); }

std::tuple<Tensor, Tensor> fp8_quantize_cuda(const Tensor& input, const std::optional<Tensor>& amax) {
  const int dt = dtype_code(input, "b200_fp8_quantize");
  c10::cuda::CUDAGuard guard(input.device());
  Tensor x = input.contiguous();
  const int64_t rows = rows_of(x), cols = cols_of(x);
  TORCH_CHECK(cols % 16 == 0, "b200_fp8_quantize: last dimension must be a multiple of 16, got ", cols);
  Tensor codes = at::empty(x.sizes(), x.options().dtype(at::kByte));
  int64_t n = 0;
  Tensor a;
  if (amax.has_value()) {
    a = as_f32_cuda(*amax, x);
    n = amax_numel_for(x, a, "b200_fp8_quantize");
  }
  Tensor scales = at::empty({n == 1 ? 1 : rows}, x.options().dtype(at::kFloat));
  if (x.numel() == 0) return {codes, scales};
  check_status(b200q_fp8_quantize(x.data_ptr(), dt, rows, cols, n ? a.data_ptr<float>() : nullptr, n,
                                  codes.data_ptr<uint8_t>(), scales.data_ptr<float>(), current_stream()),
               "b200q_fp8_quantize");
  return {codes, scales};
}
std::tuple<Tensor, Tensor> fp8_quantize_meta(const Tensor& input, const std::optional<Tensor>& amax) {
  const int64_t n = (amax.has_value() && amax->numel() == 1) ? 1 : rows_of(input);
  return {at::empty(input.sizes(), input.options().dtype(at::kByte)), at::empty({n}, input.options().dtype(at::kFloat))};
}

std::tuple<Tensor, Tensor, Tensor> nvfp4_quantize_cuda(const Tensor& input, const Tensor& amax) {
  const int dt = dtype_code(input, "b200_nvfp4_quantize");
  TORCH_CHECK(input.dim() >= 1, "b200_nvfp4_quantize: input must have at least one dimension");
  TORCH_CHECK(amax.numel() == 1, "b200_nvfp4_quantize: amax should be a scalar, got shape ", amax.sizes());
  c10::cuda::CUDAGuard guard(input.device());
  Tensor x = input.contiguous();
  const int64_t rows = rows_of(x), cols = cols_of(x);
  TORCH_CHECK_VALUE(cols % 16 == 0, "b200_nvfp4_quantize: last dimension (", cols, ") must be a multiple of the block size 16");
  auto shape = x.sizes().vec();
  shape.back() = cols / 2;
  Tensor codes = at::empty(shape, x.options().dtype(at::kByte));
  Tensor scales = at::empty({static_cast<int64_t>(b200q_nvfp4_scale_bytes(rows, cols))}, x.options().dtype(at::kByte));
  Tensor g = at::empty({}, x.options().dtype(at::kFloat));
  Tensor a = as_f32_cuda(amax, x);
  if (x.numel() == 0) {
    g.fill_(1.0);
    return {codes, scales, g};
  }
  check_status(b200q_nvfp4_quantize(x.data_ptr(), dt, rows, cols, a.data_ptr<float>(), codes.data_ptr<uint8_t>(),
                                    scales.data_ptr<uint8_t>(), g.data_ptr<float>(), current_stream()),
               "b200q_nvfp4_quantize");
  return {codes, scales, g};
}
std::tuple<Tensor, Tensor, Tensor> nvfp4_quantize_meta(const Tensor& input, const Tensor&) {
  auto shape = input.sizes().vec();
  const int64_t rows = rows_of(input), cols = cols_of(input);
  shape.back() = cols / 2;
  const int64_t sb = ((rows + 127) / 128) * ((cols / 16 + 3) / 4) * 512;
  return {at::empty(shape, input.options().dtype(at::kByte)), at::empty({sb}, input.options().dtype(at::kByte)),
          at::empty({}, input.options().dtype(at::kFloat))};
}

// out[M, N] = dequant(a) @ dequant(b)^T + bias, bf16
Tensor fp8_gemm_cuda(const Tensor& a_codes, const Tensor& a_scales, const Tensor& b_codes, const Tensor& b_scales,
                     const std::optional<Tensor>& bias) {
  TORCH_CHECK(a_codes.scalar_type() == at::kByte && b_codes.scalar_type() == at::kByte, "b200_fp8_gemm: codes must be uint8");
  TORCH_CHECK(b_codes.dim() == 2 && a_codes.dim() >= 1 && a_codes.size(-1) == b_codes.size(1),
              "b200_fp8_gemm: a [.., K] and b [N, K] must share K, got ", a_codes.sizes(), " and ", b_codes.sizes());
  c10::cuda::CUDAGuard guard(a_codes.device());
  Tensor a = a_codes.contiguous(), b = b_codes.contiguous();
  Tensor sa = a_scales.contiguous(), sb = b_scales.contiguous();
  TORCH_CHECK(sa.scalar_type() == at::kFloat && sb.scalar_type() == at::kFloat, "b200_fp8_gemm: scales must be float32");
  const int64_t K = b.size(1), N = b.size(0), M = a.numel() / std::max<int64_t>(K, 1);
  TORCH_CHECK((sa.numel() == 1 || sa.numel() == M) && (sb.numel() == 1 || sb.numel() == N),
              "b200_fp8_gemm: scales must be per-tensor or per-row");
  auto shape = a.sizes().vec();
  shape.back() = N;
  Tensor out = at::empty(shape, a.options().dtype(at::kBFloat16));
  Tensor bs;
  if (bias.has_value()) {
    bs = bias->to(at::kBFloat16).contiguous();
    TORCH_CHECK(bs.numel() == N, "b200_fp8_gemm: bias must have N elements");
  }
  if (out.numel() == 0) return out;
  check_status(b200q_fp8_gemm(a.data_ptr<uint8_t>(), sa.data_ptr<float>(), sa.numel(), b.data_ptr<uint8_t>(),
                              sb.data_ptr<float>(), sb.numel(), bias.has_value() ? bs.data_ptr() : nullptr, out.data_ptr(),
                              M, N, K, current_stream(), nullptr),
               "b200q_fp8_gemm");
  return out;
}
Tensor fp8_gemm_meta(const Tensor& a_codes, const Tensor&, const Tensor& b_codes, const Tensor&, const std::optional<Tensor>&) {
  auto shape = a_codes.sizes().vec();
  shape.back() = b_codes.size(0);
  return at::empty(shape, a_codes.options().dtype(at::kBFloat16));
}

Tensor nvfp4_gemm_cuda(const Tensor& a_codes, const Tensor& a_scales, const Tensor& a_global, const Tensor& b_codes,
                       const Tensor& b_scales, const Tensor& b_global, const std::optional<Tensor>& bias) {
  TORCH_CHECK(a_codes.scalar_type() == at::kByte && b_codes.scalar_type() == at::kByte, "b200_nvfp4_gemm: codes must be uint8");
  TORCH_CHECK(b_codes.dim() == 2 && a_codes.dim() >= 1 && a_codes.size(-1) == b_codes.size(1),
              "b200_nvfp4_gemm: a [.., K/2] and b [N, K/2] must share K, got ", a_codes.sizes(), " and ", b_codes.sizes());
  c10::cuda::CUDAGuard guard(a_codes.device());
  Tensor a = a_codes.contiguous(), b = b_codes.contiguous();
  Tensor sa = a_scales.contiguous(), sb = b_scales.contiguous();
  Tensor ga = a_global.to(at::kFloat).contiguous(), gb = b_global.to(at::kFloat).contiguous();
  const int64_t K = b.size(1) * 2, N = b.size(0), M = a.numel() / std::max<int64_t>(K / 2, 1);
  TORCH_CHECK(sa.numel() >= static_cast<int64_t>(b200q_nvfp4_scale_bytes(M, K)) &&
                  sb.numel() >= static_cast<int64_t>(b200q_nvfp4_scale_bytes(N, K)),
              "b200_nvfp4_gemm: block-scale buffers are smaller than the swizzled layout needs");
  auto shape = a.sizes().vec();
  shape.back() = N;
  Tensor out = at::empty(shape, a.options().dtype(at::kBFloat16));
  Tensor bs;
  if (bias.has_value()) {
    bs = bias->to(at::kBFloat16).contiguous();
    TORCH_CHECK(bs.numel() == N, "b200_nvfp4_gemm: bias must have N elements");
  }
  if (out.numel() == 0) return out;
  check_status(b200q_nvfp4_gemm(a.data_ptr<uint8_t>(), sa.data_ptr<uint8_t>(), ga.data_ptr<float>(), b.data_ptr<uint8_t>(),
                                sb.data_ptr<uint8_t>(), gb.data_ptr<float>(), bias.has_value() ? bs.data_ptr() : nullptr,
                                out.data_ptr(), M, N, K, current_stream(), nullptr),
               "b200q_nvfp4_gemm");
  return out;
}
Tensor nvfp4_gemm_meta(const Tensor& a_codes, const Tensor&, const Tensor&, const Tensor& b_codes, const Tensor&, const Tensor&,
                       const std::optional<Tensor>&) {
  auto shape = a_codes.sizes().vec();
  shape.back() = b_codes.size(0);
  return at::empty(shape, a_codes.options().dtype(at::kBFloat16));
}

// Schema variants without optional arguments: the reference's plugin generator accepts only
// Tensor / float / int / bool / str arguments
// (py/torch_tensorrt/dynamo/conversion/plugins/_generate_plugin.py:131-158).
Tensor fp8_gemm_nobias_cuda(const Tensor& a, const Tensor& sa, const Tensor& b, const Tensor& sb) {
  return fp8_gemm_cuda(a, sa, b, sb, std::nullopt);
}
Tensor fp8_gemm_bias_cuda(const Tensor& a, const Tensor& sa, const Tensor& b, const Tensor& sb, const Tensor& bias) {
  return fp8_gemm_cuda(a, sa, b, sb, bias);
}
Tensor fp8_gemm_nobias_meta(const Tensor& a, const Tensor& sa, const Tensor& b, const Tensor& sb) {
  return fp8_gemm_meta(a, sa, b, sb, std::nullopt);
}
Tensor fp8_gemm_bias_meta(const Tensor& a, const Tensor& sa, const Tensor& b, const Tensor& sb, const Tensor&) {
  return fp8_gemm_meta(a, sa, b, sb, std::nullopt);
}
// Gate/up linear of a gated MLP with the activation in the GEMM epilogue: b = [F gate rows; F up rows],
// out [.., F] = silu(g) * u.  Fewer than 256 tokens (a decode step) take the GEMM and the activation
// kernel one after the other: the same bits.
Tensor fp8_gemm_silu_mul_cuda(const Tensor& a_codes, const Tensor& a_scales, const Tensor& b_codes, const Tensor& b_scales) {
  TORCH_CHECK(a_codes.scalar_type() == at::kByte && b_codes.scalar_type() == at::kByte, "b200_fp8_gemm_silu_mul: codes must be uint8");
  TORCH_CHECK(b_codes.dim() == 2 && a_codes.dim() >= 1 && a_codes.size(-1) == b_codes.size(1) && b_codes.size(0) % 256 == 0,
              "b200_fp8_gemm_silu_mul: a [.., K] and b [2F, K] with F a multiple of 128, got ", a_codes.sizes(), " and ", b_codes.sizes());
  c10::cuda::CUDAGuard guard(a_codes.device());
  Tensor a = a_codes.contiguous(), b = b_codes.contiguous();
  Tensor sa = a_scales.contiguous(), sb = b_scales.contiguous();
  TORCH_CHECK(sa.scalar_type() == at::kFloat && sb.scalar_type() == at::kFloat, "b200_fp8_gemm_silu_mul: scales must be float32");
  const int64_t K = b.size(1), N = b.size(0), M = a.numel() / std::max<int64_t>(K, 1);
  TORCH_CHECK((sa.numel() == 1 || sa.numel() == M) && (sb.numel() == 1 || sb.numel() == N),
              "b200_fp8_gemm_silu_mul: scales must be per-tensor or per-row");
  auto shape = a.sizes().vec();
  shape.back() = N / 2;
  Tensor out = at::empty(shape, a.options().dtype(at::kBFloat16));
  if (out.numel() == 0) return out;
  if (M >= 256) {
    check_status(b200q_fp8_gemm_silu_mul(a.data_ptr<uint8_t>(), sa.data_ptr<float>(), sa.numel(), b.data_ptr<uint8_t>(), sb.data_ptr<float>(),
                                         sb.numel(), nullptr, out.data_ptr(), M, N, K, current_stream(), nullptr),
                 "b200q_fp8_gemm_silu_mul");
  } else {
    Tensor gu = at::empty({M, N}, a.options().dtype(at::kBFloat16));
    check_status(b200q_fp8_gemm(a.data_ptr<uint8_t>(), sa.data_ptr<float>(), sa.numel(), b.data_ptr<uint8_t>(), sb.data_ptr<float>(), sb.numel(),
                                nullptr, gu.data_ptr(), M, N, K, current_stream(), nullptr),
                 "b200q_fp8_gemm");
    check_status(b200q_silu_mul(gu.data_ptr(), out.data_ptr(), M, N / 2, current_stream()), "b200q_silu_mul");
  }
  return out;
}
Tensor fp8_gemm_silu_mul_meta(const Tensor& a_codes, const Tensor&, const Tensor& b_codes, const Tensor&) {
  auto shape = a_codes.sizes().vec();
  shape.back() = b_codes.size(0) / 2;
  return at::empty(shape, a_codes.options().dtype(at::kBFloat16));
}
// ... and with the static per-tensor FP8 quantizer of the activation in the epilogue too: (codes, scale)
std::tuple<Tensor, Tensor> fp8_gemm_silu_mul_quant_cuda(const Tensor& a_codes, const Tensor& a_scales, const Tensor& b_codes,
                                                        const Tensor& b_scales, const Tensor& amax) {
  TORCH_CHECK(amax.numel() == 1, "b200_fp8_gemm_silu_mul_quant: amax must hold one value");
  c10::cuda::CUDAGuard guard(a_codes.device());
  const int64_t K = b_codes.size(1), N = b_codes.size(0), M = a_codes.numel() / std::max<int64_t>(K, 1);
  Tensor am = amax.to(a_codes.device(), at::kFloat).reshape({1}).contiguous();
  if (M < 256) {   // a decode step: the kernels one after the other give the same bits
    Tensor act = fp8_gemm_silu_mul_cuda(a_codes, a_scales, b_codes, b_scales);
    auto shape = act.sizes().vec();
    Tensor codes = at::empty(shape, act.options().dtype(at::kByte));
    Tensor scale = at::empty({1}, act.options().dtype(at::kFloat));
    if (act.numel() > 0)
      check_status(b200q_fp8_quantize(act.data_ptr(), B200Q_BF16, M, N / 2, am.data_ptr<float>(), 1, codes.data_ptr<uint8_t>(),
                                      scale.data_ptr<float>(), current_stream()),
                   "b200q_fp8_quantize");
    return {codes, scale};
  }
  TORCH_CHECK(a_codes.scalar_type() == at::kByte && b_codes.scalar_type() == at::kByte && b_codes.dim() == 2 &&
                  a_codes.size(-1) == K && N % 256 == 0,
              "b200_fp8_gemm_silu_mul_quant: a [.., K] and b [2F, K] uint8 with F a multiple of 128");
  Tensor a = a_codes.contiguous(), b = b_codes.contiguous();
  Tensor sa = a_scales.contiguous(), sb = b_scales.contiguous();
  TORCH_CHECK(sa.scalar_type() == at::kFloat && sb.scalar_type() == at::kFloat && (sa.numel() == 1 || sa.numel() == M) &&
                  (sb.numel() == 1 || sb.numel() == N),
              "b200_fp8_gemm_silu_mul_quant: float32 scales, per-tensor or per-row");
  auto shape = a.sizes().vec();
  shape.back() = N / 2;
  Tensor codes = at::empty(shape, a.options().dtype(at::kByte));
  Tensor scale = at::empty({1}, a.options().dtype(at::kFloat));
  check_status(b200q_fp8_gemm_silu_mul_quantize(a.data_ptr<uint8_t>(), sa.data_ptr<float>(), sa.numel(), b.data_ptr<uint8_t>(),
                                                sb.data_ptr<float>(), sb.numel(), nullptr, am.data_ptr<float>(), codes.data_ptr<uint8_t>(),
                                                scale.data_ptr<float>(), M, N, K, current_stream(), nullptr),
               "b200q_fp8_gemm_silu_mul_quantize");
  return {codes, scale};
}
std::tuple<Tensor, Tensor> fp8_gemm_silu_mul_quant_meta(const Tensor& a_codes, const Tensor&, const Tensor& b_codes, const Tensor&,
                                                        const Tensor&) {
  auto shape = a_codes.sizes().vec();
  shape.back() = b_codes.size(0) / 2;
  return {at::empty(shape, a_codes.options().dtype(at::kByte)), at::empty({1}, a_codes.options().dtype(at::kFloat))};
}
Tensor nvfp4_gemm_nobias_cuda(const Tensor& a, const Tensor& sa, const Tensor& ga, const Tensor& b, const Tensor& sb, const Tensor& gb) {
  return nvfp4_gemm_cuda(a, sa, ga, b, sb, gb, std::nullopt);
}
Tensor nvfp4_gemm_bias_cuda(const Tensor& a, const Tensor& sa, const Tensor& ga, const Tensor& b, const Tensor& sb, const Tensor& gb,
                            const Tensor& bias) {
  return nvfp4_gemm_cuda(a, sa, ga, b, sb, gb, bias);
}
Tensor nvfp4_gemm_nobias_meta(const Tensor& a, const Tensor& sa, const Tensor& ga, const Tensor& b, const Tensor& sb, const Tensor& gb) {
  return nvfp4_gemm_meta(a, sa, ga, b, sb, gb, std::nullopt);
}
Tensor nvfp4_gemm_bias_meta(const Tensor& a, const Tensor& sa, const Tensor& ga, const Tensor& b, const Tensor& sb, const Tensor& gb,
                            const Tensor&) {
  return nvfp4_gemm_meta(a, sa, ga, b, sb, gb, std::nullopt);
}

// ------------------------------------------------------------------ one-node quantized linears (the plugin form)
// y = linear(Q(x), W_hat, bias) with the weight already reduced to codes and scales: what the three
// nodes quantize_op(x), quantize_op(W), aten.linear collapse to once the weight is a constant.
// All arguments are tensors and the activation comes first, so the generated TensorRT plugin's
// output descriptor (`tensor_args[0].like()`, plugins/_generate_plugin.py:263) has the right
// dtype: the result is returned in x's dtype, like the DQ output of the reference
// (impl/quantize.py:132-134).  x_amax: one value (per-tensor, impl/quantize.py:96-100), one per
// token, or an empty tensor (per-token abs-max measured by the quantize kernel).
Tensor fp8_linear_impl(const Tensor& x_in, const Tensor& x_amax, const Tensor& w_codes, const Tensor& w_scales,
                       const std::optional<Tensor>& bias) {
  const int dt = dtype_code(x_in, "b200_fp8_linear");
  TORCH_CHECK(w_codes.dim() == 2 && x_in.dim() >= 1 && x_in.size(-1) == w_codes.size(1),
              "b200_fp8_linear: x [.., K] and w_codes [N, K] must share K, got ", x_in.sizes(), " and ", w_codes.sizes());
  c10::cuda::CUDAGuard guard(x_in.device());
  Tensor x = x_in.contiguous();
  const int64_t rows = rows_of(x), cols = cols_of(x);
  TORCH_CHECK(cols % 16 == 0, "b200_fp8_linear: K must be a multiple of 16, got ", cols);
  int64_t n = 0;
  Tensor a;
  if (x_amax.numel() > 0) {
    a = as_f32_cuda(x_amax, x);
    n = amax_numel_for(x, a, "b200_fp8_linear");
  }
  Tensor codes = at::empty(x.sizes(), x.options().dtype(at::kByte));
  Tensor scales = at::empty({n == 1 ? 1 : rows}, x.options().dtype(at::kFloat));
  if (x.numel() > 0)
    check_status(b200q_fp8_quantize(x.data_ptr(), dt, rows, cols, n ? a.data_ptr<float>() : nullptr, n,
                                    codes.data_ptr<uint8_t>(), scales.data_ptr<float>(), current_stream()),
                 "b200q_fp8_quantize");
  Tensor out = fp8_gemm_cuda(codes, scales, w_codes, w_scales, bias);
  return out.scalar_type() == x.scalar_type() ? out : out.to(x.scalar_type());
}
Tensor fp8_linear_cuda(const Tensor& x, const Tensor& x_amax, const Tensor& w_codes, const Tensor& w_scales) {
  return fp8_linear_impl(x, x_amax, w_codes, w_scales, std::nullopt);
}
Tensor fp8_linear_bias_cuda(const Tensor& x, const Tensor& x_amax, const Tensor& w_codes, const Tensor& w_scales, const Tensor& bias) {
  return fp8_linear_impl(x, x_amax, w_codes, w_scales, bias);
}
Tensor linear_meta_like(const Tensor& x, const Tensor& w_codes) {
  auto shape = x.sizes().vec();
  shape.back() = w_codes.size(0);
  return at::empty(shape, x.options());
}
Tensor fp8_linear_meta(const Tensor& x, const Tensor&, const Tensor& w_codes, const Tensor&) { return linear_meta_like(x, w_codes); }
Tensor fp8_linear_bias_meta(const Tensor& x, const Tensor&, const Tensor& w_codes, const Tensor&, const Tensor&) {
  return linear_meta_like(x, w_codes);
}

Tensor nvfp4_linear_impl(const Tensor& x_in, const Tensor& x_amax, const Tensor& w_codes, const Tensor& w_scales,
                         const Tensor& w_global, const std::optional<Tensor>& bias) {
  TORCH_CHECK(w_codes.dim() == 2 && x_in.dim() >= 1 && x_in.size(-1) == 2 * w_codes.size(1),
              "b200_nvfp4_linear: x [.., K] and w_codes [N, K/2] must share K, got ", x_in.sizes(), " and ", w_codes.sizes());
  TORCH_CHECK_VALUE(cols_of(x_in) % 32 == 0, "b200_nvfp4_linear: K must be a multiple of 32, got ", cols_of(x_in));
  auto q = nvfp4_quantize_cuda(x_in, x_amax);
  Tensor out = nvfp4_gemm_cuda(std::get<0>(q), std::get<1>(q), std::get<2>(q), w_codes, w_scales, w_global, bias);
  return out.scalar_type() == x_in.scalar_type() ? out : out.to(x_in.scalar_type());
}
Tensor nvfp4_linear_cuda(const Tensor& x, const Tensor& x_amax, const Tensor& w_codes, const Tensor& w_scales, const Tensor& w_global) {
  return nvfp4_linear_impl(x, x_amax, w_codes, w_scales, w_global, std::nullopt);
}
Tensor nvfp4_linear_bias_cuda(const Tensor& x, const Tensor& x_amax, const Tensor& w_codes, const Tensor& w_scales,
                              const Tensor& w_global, const Tensor& bias) {
  return nvfp4_linear_impl(x, x_amax, w_codes, w_scales, w_global, bias);
}
Tensor nvfp4_linear_meta(const Tensor& x, const Tensor&, const Tensor& w_codes, const Tensor&, const Tensor&) {
  return linear_meta_like(x, w_codes);
}
Tensor nvfp4_linear_bias_meta(const Tensor& x, const Tensor&, const Tensor& w_codes, const Tensor&, const Tensor&, const Tensor&) {
  return linear_meta_like(x, w_codes);
}

// ------------------------------------------------------------------ FP8 attention (Q, K, V from quantize_op)
Tensor fp8_sdpa_cuda(const Tensor& q_in, const Tensor& k_in, const Tensor& v_in, const Tensor& amax_q, const Tensor& amax_k,
                     const Tensor& amax_v, bool is_causal, double scale) {
  const int dt = dtype_code(q_in, "b200_fp8_sdpa");
  TORCH_CHECK(q_in.dim() == 4 && k_in.dim() == 4 && v_in.dim() == 4 && k_in.sizes() == v_in.sizes() && q_in.size(0) == k_in.size(0) &&
                  q_in.size(3) == k_in.size(3),
              "b200_fp8_sdpa: expected q [B, Hq, Sq, D] and k, v [B, Hkv, Sk, D], got ", q_in.sizes(), ", ", k_in.sizes(), ", ", v_in.sizes());
  TORCH_CHECK(k_in.scalar_type() == q_in.scalar_type() && v_in.scalar_type() == q_in.scalar_type(), "b200_fp8_sdpa: q, k, v must share a dtype");
  TORCH_CHECK(amax_q.numel() == 1 && amax_k.numel() == 1 && amax_v.numel() == 1, "b200_fp8_sdpa: amax must be per-tensor (one value each)");
  const int64_t B = q_in.size(0), Hq = q_in.size(1), Sq = q_in.size(2), D = q_in.size(3), Hkv = k_in.size(1), Sk = k_in.size(2);
  TORCH_CHECK_VALUE(Hq % Hkv == 0 && D % 16 == 0 && D <= 128, "b200_fp8_sdpa: need Hq % Hkv == 0 and a head dimension that is a multiple of 16 up to 128");
  c10::cuda::CUDAGuard guard(q_in.device());
  Tensor q = q_in.contiguous(), k = k_in.contiguous(), v = v_in.contiguous();
  Tensor out = at::empty_like(q);
  if (out.numel() == 0) return out;
  auto bytes = q.options().dtype(at::kByte);
  auto f32 = q.options().dtype(at::kFloat);
  Tensor aq = as_f32_cuda(amax_q, q).reshape({1}), ak = as_f32_cuda(amax_k, q).reshape({1}), av = as_f32_cuda(amax_v, q).reshape({1});
  Tensor qc = at::empty(q.sizes(), bytes), kc = at::empty(k.sizes(), bytes);
  Tensor sq = at::empty({1}, f32), sk = at::ones({1}, f32), sv = at::ones({1}, f32);
  const int64_t stride = std::max<int64_t>((Sk + 15) / 16 * 16, 16);
  Tensor vt = at::empty({B, Hkv, D, stride}, bytes);
  check_status(b200q_fp8_quantize(q.data_ptr(), dt, B * Hq * Sq, D, aq.data_ptr<float>(), 1, qc.data_ptr<uint8_t>(), sq.data_ptr<float>(),
                                  current_stream()), "b200q_fp8_quantize");
  if (Sk > 0) {
    check_status(b200q_fp8_quantize(k.data_ptr(), dt, B * Hkv * Sk, D, ak.data_ptr<float>(), 1, kc.data_ptr<uint8_t>(), sk.data_ptr<float>(),
                                    current_stream()), "b200q_fp8_quantize");
    check_status(b200q_fp8_quantize_transpose(v.data_ptr(), dt, B * Hkv, Sk, D, av.data_ptr<float>(), vt.data_ptr<uint8_t>(), stride,
                                              sv.data_ptr<float>(), current_stream()), "b200q_fp8_quantize_transpose");
  }
  const float sm = scale > 0.0 ? static_cast<float>(scale) : 1.0f / std::sqrt(static_cast<float>(D));
  check_status(b200q_fp8_sdpa(qc.data_ptr<uint8_t>(), kc.data_ptr<uint8_t>(), vt.data_ptr<uint8_t>(), sq.data_ptr<float>(), sk.data_ptr<float>(),
                              sv.data_ptr<float>(), out.data_ptr(), dt, B, Hq, Hkv, Sq, Sk, stride, D, sm, is_causal ? 1 : 0, current_stream()),
               "b200q_fp8_sdpa");
  return out;
}
Tensor fp8_sdpa_meta(const Tensor& q, const Tensor&, const Tensor&, const Tensor&, const Tensor&, const Tensor&, bool, double) {
  return at::empty_like(q);
}

bool schema_exists(const char* name) {
  return c10::Dispatcher::singleton().findSchema({name, ""}).has_value();
}

}  // namespace

TORCH_LIBRARY_FRAGMENT(tensorrt, m) {
  // Reference-schema ops: only defined (and implemented) here when nobody else has.
  if (!schema_exists("tensorrt::quantize_op")) {
    m.def("quantize_op(Tensor input, Tensor amax, int num_bits, int exponent_bits, bool unsigned, bool narrow_range) -> Tensor");
    m.impl("quantize_op", c10::DispatchKey::CUDA, TORCH_FN(quantize_op_cuda));
    m.impl("quantize_op", c10::DispatchKey::Meta, TORCH_FN(quantize_op_meta));
  }
  if (!schema_exists("tensorrt::dynamic_block_quantize_op")) {
    m.def(
        "dynamic_block_quantize_op(Tensor input, int block_size, Tensor amax, int num_bits, int exponent_bits, "
        "int scale_num_bits, int scale_exponent_bits) -> Tensor");
    m.impl("dynamic_block_quantize_op", c10::DispatchKey::CUDA, TORCH_FN(dynamic_block_quantize_op_cuda));
    m.impl("dynamic_block_quantize_op", c10::DispatchKey::Meta, TORCH_FN(dynamic_block_quantize_op_meta));
  }
  // The same two kernels under names that never collide, plus the real-quant building blocks.
  m.def("b200_quantize_op(Tensor input, Tensor amax, int num_bits, int exponent_bits, bool unsigned, bool narrow_range) -> Tensor");
  m.impl("b200_quantize_op", c10::DispatchKey::CUDA, TORCH_FN(quantize_op_cuda));
  m.impl("b200_quantize_op", c10::DispatchKey::Meta, TORCH_FN(quantize_op_meta));
  m.def(
      "b200_dynamic_block_quantize_op(Tensor input, int block_size, Tensor amax, int num_bits, int exponent_bits, "
      "int scale_num_bits, int scale_exponent_bits) -> Tensor");
  m.impl("b200_dynamic_block_quantize_op", c10::DispatchKey::CUDA, TORCH_FN(dynamic_block_quantize_op_cuda));
  m.impl("b200_dynamic_block_quantize_op", c10::DispatchKey::Meta, TORCH_FN(dynamic_block_quantize_op_meta));

  m.def("b200_amax(Tensor input) -> Tensor");
  m.impl("b200_amax", c10::DispatchKey::CUDA, TORCH_FN(amax_cuda));
  m.impl("b200_amax", c10::DispatchKey::Meta, TORCH_FN(amax_meta));

  m.def("b200_fp8_quantize(Tensor input, Tensor? amax) -> (Tensor, Tensor)");
  m.impl("b200_fp8_quantize", c10::DispatchKey::CUDA, TORCH_FN(fp8_quantize_cuda));
  m.impl("b200_fp8_quantize", c10::DispatchKey::Meta, TORCH_FN(fp8_quantize_meta));

  m.def("b200_nvfp4_quantize(Tensor input, Tensor amax) -> (Tensor, Tensor, Tensor)");
  m.impl("b200_nvfp4_quantize", c10::DispatchKey::CUDA, TORCH_FN(nvfp4_quantize_cuda));
  m.impl("b200_nvfp4_quantize", c10::DispatchKey::Meta, TORCH_FN(nvfp4_quantize_meta));

  // GEMMs on quantized operands: a variant with and one without bias, no optional arguments
  m.def("b200_fp8_gemm(Tensor a_codes, Tensor a_scales, Tensor b_codes, Tensor b_scales) -> Tensor");
  m.impl("b200_fp8_gemm", c10::DispatchKey::CUDA, TORCH_FN(fp8_gemm_nobias_cuda));
  m.impl("b200_fp8_gemm", c10::DispatchKey::Meta, TORCH_FN(fp8_gemm_nobias_meta));
  m.def("b200_fp8_gemm_bias(Tensor a_codes, Tensor a_scales, Tensor b_codes, Tensor b_scales, Tensor bias) -> Tensor");
  m.impl("b200_fp8_gemm_bias", c10::DispatchKey::CUDA, TORCH_FN(fp8_gemm_bias_cuda));
  m.impl("b200_fp8_gemm_bias", c10::DispatchKey::Meta, TORCH_FN(fp8_gemm_bias_meta));
  m.def("b200_fp8_gemm_silu_mul(Tensor a_codes, Tensor a_scales, Tensor b_codes, Tensor b_scales) -> Tensor");
  m.impl("b200_fp8_gemm_silu_mul", c10::DispatchKey::CUDA, TORCH_FN(fp8_gemm_silu_mul_cuda));
  m.impl("b200_fp8_gemm_silu_mul", c10::DispatchKey::Meta, TORCH_FN(fp8_gemm_silu_mul_meta));
  m.def("b200_fp8_gemm_silu_mul_quant(Tensor a_codes, Tensor a_scales, Tensor b_codes, Tensor b_scales, Tensor amax) -> (Tensor, Tensor)");
  m.impl("b200_fp8_gemm_silu_mul_quant", c10::DispatchKey::CUDA, TORCH_FN(fp8_gemm_silu_mul_quant_cuda));
  m.impl("b200_fp8_gemm_silu_mul_quant", c10::DispatchKey::Meta, TORCH_FN(fp8_gemm_silu_mul_quant_meta));
  m.def("b200_nvfp4_gemm(Tensor a_codes, Tensor a_scales, Tensor a_global, Tensor b_codes, Tensor b_scales, Tensor b_global) -> Tensor");
  m.impl("b200_nvfp4_gemm", c10::DispatchKey::CUDA, TORCH_FN(nvfp4_gemm_nobias_cuda));
  m.impl("b200_nvfp4_gemm", c10::DispatchKey::Meta, TORCH_FN(nvfp4_gemm_nobias_meta));
  m.def(
      "b200_nvfp4_gemm_bias(Tensor a_codes, Tensor a_scales, Tensor a_global, Tensor b_codes, Tensor b_scales, Tensor b_global, "
      "Tensor bias) -> Tensor");
  m.impl("b200_nvfp4_gemm_bias", c10::DispatchKey::CUDA, TORCH_FN(nvfp4_gemm_bias_cuda));
  m.impl("b200_nvfp4_gemm_bias", c10::DispatchKey::Meta, TORCH_FN(nvfp4_gemm_bias_meta));

  // SDPA whose Q, K, V are FP8 fake-quantized with per-tensor amax; scale <= 0 = 1 / sqrt(head_dim)
  m.def("b200_fp8_sdpa(Tensor q, Tensor k, Tensor v, Tensor amax_q, Tensor amax_k, Tensor amax_v, bool is_causal, float scale) -> Tensor");
  m.impl("b200_fp8_sdpa", c10::DispatchKey::CUDA, TORCH_FN(fp8_sdpa_cuda));
  m.impl("b200_fp8_sdpa", c10::DispatchKey::Meta, TORCH_FN(fp8_sdpa_meta));

  // One-node quantized linears (activation first, result in the activation's dtype): the ops handed
  // to torch_tensorrt.dynamo.conversion.plugins.custom_op.
  m.def("b200_fp8_linear(Tensor x, Tensor x_amax, Tensor w_codes, Tensor w_scales) -> Tensor");
  m.impl("b200_fp8_linear", c10::DispatchKey::CUDA, TORCH_FN(fp8_linear_cuda));
  m.impl("b200_fp8_linear", c10::DispatchKey::Meta, TORCH_FN(fp8_linear_meta));
  m.def("b200_fp8_linear_bias(Tensor x, Tensor x_amax, Tensor w_codes, Tensor w_scales, Tensor bias) -> Tensor");
  m.impl("b200_fp8_linear_bias", c10::DispatchKey::CUDA, TORCH_FN(fp8_linear_bias_cuda));
  m.impl("b200_fp8_linear_bias", c10::DispatchKey::Meta, TORCH_FN(fp8_linear_bias_meta));
  m.def("b200_nvfp4_linear(Tensor x, Tensor x_amax, Tensor w_codes, Tensor w_scales, Tensor w_global) -> Tensor");
  m.impl("b200_nvfp4_linear", c10::DispatchKey::CUDA, TORCH_FN(nvfp4_linear_cuda));
  m.impl("b200_nvfp4_linear", c10::DispatchKey::Meta, TORCH_FN(nvfp4_linear_meta));
  m.def("b200_nvfp4_linear_bias(Tensor x, Tensor x_amax, Tensor w_codes, Tensor w_scales, Tensor w_global, Tensor bias) -> Tensor");
  m.impl("b200_nvfp4_linear_bias", c10::DispatchKey::CUDA, TORCH_FN(nvfp4_linear_bias_cuda));
  m.impl("b200_nvfp4_linear_bias", c10::DispatchKey::Meta, TORCH_FN(nvfp4_linear_bias_meta));
}
