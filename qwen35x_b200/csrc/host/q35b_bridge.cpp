// Binding of libq35b into the qwen35x runtime: the file a maintainer of the reference adds as
// src/runtime/q35b_bridge.cpp and links with -lq35b.
//
// It keeps the reference's calling convention (namespace qwen35x::cuda, bool + std::string & error_message,
// include/qwen35x/runtime/cuda_bench.h:7-283) and maps each NVFP4 projection seam onto the C ABI of
// include/q35b_nvfp4.h:
//   load time   load_modelopt_nvfp4_state's pad/swizzle/pack steps (src/runtime/qwen35x_cuda_backend.cpp:1582-1695)
//               -> q35b_load_weight / q35b_load_gate_up
//   decode      run_nvfp4_scalar_*_device and matvec_nvfp4_bf16 call sites (qwen35x_cuda_backend.cpp:2323-2478)
//               -> q35b_decode_projection, q35b_decode_mlp
//   prefill     run_nvfp4_cublaslt_prefill_projection_device_bf16 (cuda_bench.h:70-83) as called by
//               cublas_nvfp4_prefill_gemm_or_bf16 (src/kernels/cuda/prefill.cu:606-645)
//               -> run_nvfp4_q35b_prefill_projection_device_bf16: same arguments up to the weight, BF16 output
//               directly (the pf_f32_to_bf16 pass at prefill.cu:639 goes away)
//
// This file is compiled (syntax and types) against the reference's headers by tests/test_bridge_compiles.py, so a
// drift of either interface is caught; it is not part of libq35b itself.
#include <cstdint>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "q35b_nvfp4.h"
#include "qwen35x/runtime/cuda_bench.h"

namespace qwen35x::cuda {
namespace {

bool ok(int status, std::string & error_message) {
  if (status == Q35B_OK) return true;
  error_message = q35b_last_error();  // same convention: false + human-readable message
  return false;
}

}  // namespace

// ---- load time ----------------------------------------------------------------------------------------------

bool q35b_load_weight(const std::vector<std::uint8_t> & packed_weights, const std::vector<std::uint8_t> & weight_scales_e4m3,
                      float input_scale, float weight_scale_2, int rows, int cols, q35b_weight ** out,
                      std::string & error_message) {
  if (packed_weights.size() != static_cast<std::size_t>(rows) * (cols / 2) ||
      weight_scales_e4m3.size() != static_cast<std::size_t>(rows) * (cols / 16)) {
    error_message = "NVFP4 packed weight or scale size does not match matrix dimensions.";
    return false;
  }
  return ok(q35b_weight_create(packed_weights.data(), weight_scales_e4m3.data(), weight_scale_2, input_scale, rows, cols,
                               0, 1, out),
            error_message);
}

bool q35b_load_gate_up(const std::vector<std::uint8_t> & gate_packed, const std::vector<std::uint8_t> & gate_scales,
                       float gate_weight_scale_2, const std::vector<std::uint8_t> & up_packed,
                       const std::vector<std::uint8_t> & up_scales, float up_weight_scale_2, int intermediate, int hidden,
                       q35b_weight ** out, std::string & error_message) {
  return ok(q35b_weight_create_gate_up(gate_packed.data(), gate_scales.data(), gate_weight_scale_2, up_packed.data(),
                                       up_scales.data(), up_weight_scale_2, intermediate, hidden, out),
            error_message);
}

// ---- decode -------------------------------------------------------------------------------------------------

bool q35b_decode_projection(const q35b_weight * weight, const void * input_bf16, int tokens, void * output_bf16,
                            cudaStream_t stream, std::string & error_message) {
  return ok(q35b_gemv_w4a16_bf16(weight, input_bf16, tokens, output_bf16, Q35B_GEMV_AUTO, stream), error_message);
}

// The MLP of one layer as one launch: silu(gate x) * up x into `intermediate_bf16`, then down + residual, the role of
// run_nvfp4_scalar_mlp_residual_device (src/runtime/cuda_bench.cu:1707-1800).  The work list is built once per layer.
bool q35b_decode_mlp_create(const q35b_weight * gate_up, const q35b_weight * down, const void * input_bf16,
                            void * intermediate_bf16, const void * residual_bf16, void * output_bf16, int tokens,
                            q35b_gemv_batch ** out, std::string & error_message) {
  const q35b_gemv_item items[2] = {
    {gate_up, input_bf16, intermediate_bf16, nullptr, 0},
    {down, intermediate_bf16, output_bf16, residual_bf16, 1},  // runs after item 0 of the same launch
  };
  return ok(q35b_gemv_batch_create(items, 2, tokens, out), error_message);
}

bool q35b_decode_mlp(const q35b_gemv_batch * mlp, cudaStream_t stream, std::string & error_message) {
  return ok(q35b_gemv_batch_run(mlp, stream), error_message);
}

// ---- prefill ------------------------------------------------------------------------------------------------

// Drop-in for run_nvfp4_cublaslt_prefill_projection_device_bf16: same scratch arguments (sized by the reference's
// rule, cuda_bench.cu:2616-2619), the repacked weight instead of the three cuBLASLt pointers, BF16 output.
// input_scale_scratch: one float; quant_workspace: q35b_quant_workspace_bytes() bytes, zeroed once.
bool run_nvfp4_q35b_prefill_projection_device_bf16(const void * input_bf16, const q35b_weight * weight, int sequence_length,
                                                   int rows, int cols, std::uint8_t * activation_scratch,
                                                   std::uint8_t * activation_scale_scratch, float * input_scale_scratch,
                                                   void * quant_workspace, void * output_bf16, cudaStream_t stream,
                                                   std::string & error_message) {
  if (weight == nullptr || q35b_weight_rows(weight) != rows || q35b_weight_cols(weight) != cols) {
    error_message = "Invalid dimensions for NVFP4 prefill projection.";
    return false;
  }
  return ok(q35b_quantize_nvfp4_bf16(input_bf16, sequence_length, cols, 0.0f, activation_scratch, activation_scale_scratch,
                                     input_scale_scratch, quant_workspace, stream),
            error_message) &&
         ok(q35b_gemm_w4a4_bf16(weight, activation_scratch, activation_scale_scratch, input_scale_scratch, sequence_length,
                                output_bf16, rows, nullptr, stream),
            error_message);
}

// The check and benchmark entry points keep their reference signatures exactly; these wrappers only show that the
// types line up (the implementations that run on libq35b are in nvfp4_runtime.cpp of the q35b command line).
bool q35b_matvec_check(const std::vector<std::uint8_t> & packed_weights, const std::vector<std::uint8_t> & weight_scales_e4m3,
                       float input_scale, float weight_scale_2, int rows, int cols, int sample_rows,
                       double & max_abs_error, std::string & error_message) {
  bool (*reference_signature)(const std::vector<std::uint8_t> &, const std::vector<std::uint8_t> &, float, float, int, int,
                              int, double &, std::string &) = &run_nvfp4_matvec_check;
  (void)reference_signature;
  (void)input_scale;
  (void)sample_rows;
  max_abs_error = 0.0;
  q35b_weight * w = nullptr;
  if (!q35b_load_weight(packed_weights, weight_scales_e4m3, 1.0f, weight_scale_2, rows, cols, &w, error_message)) return false;
  q35b_weight_destroy(w);
  return true;
}

}  // namespace qwen35x::cuda
