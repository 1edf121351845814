// Host-side mirror of the reference's NVFP4 projection entry points on top of the q35b C ABI.
//
// Same names, argument meaning and error convention (`bool` + `std::string & error_message`) as
// qwen35x::cuda::run_nvfp4_matvec_check / run_nvfp4_custom_projection_benchmark /
// run_nvfp4_cublaslt_prefill_projection (include/qwen35x/runtime/cuda_bench.h:18-54,85-98) and the kernel-name
// selector of run_nvfp4_projection_benchmark (src/runtime/runtime.cpp:378-390), so that runtime.cpp-style callers and
// the CLI flags --check-nvfp4-tensor / --bench-nvfp4-projection / --bench-nvfp4-prefill-projection /
// --nvfp4-projection-kernel keep working.
#pragma once

#include <cstdint>
#include <string>
#include <vector>

namespace q35b::runtime {

// Kernel selector: the reference's names map onto the engine's decode kernels (row, warp, scale-group: the
// vectorised SIMT kernel; blackwell-fp4: activation quantisation + tcgen05 W4A4 GEMM at M = 1) and two new names
// select them directly.
enum KernelVariant : int {
  kRow = 0,
  kWarp = 1,
  kScaleGroup = 2,
  kBlackwellFp4 = 3,
  kB200Simt = 10,
  kB200Stream = 11,
};

bool parse_projection_kernel(const std::string & name, int & kernel_variant, std::string & error_message);
const char * projection_kernel_note(int kernel_variant);

bool run_nvfp4_matvec_check(const std::vector<std::uint8_t> & packed_weights,
                            const std::vector<std::uint8_t> & weight_scales_e4m3, float input_scale,
                            float weight_scale_2, int rows, int cols, int sample_rows, double & max_abs_error,
                            std::string & error_message);

bool run_nvfp4_custom_projection_benchmark(const std::vector<std::uint8_t> & packed_weights,
                                           const std::vector<std::uint8_t> & weight_scales_e4m3, float input_scale,
                                           float weight_scale_2, int rows, int cols, int kernel_variant,
                                           int warmup_iterations, int benchmark_iterations, double & avg_iteration_ms,
                                           double & max_abs_error, std::string & error_message);

// The prefill W4A4 projection benchmark: host fp32 input [sequence_length, cols] quantised from fp32 on the device
// (the reference's benchmark contract), checkpoint-order host weights; per iteration activation quantisation + GEMM.  max_abs_error compares 2 tokens x
// 8 rows against the unquantised-activation host projection, exactly what the reference reports
// (src/runtime/cuda_bench.cu:2571-2585).
bool run_nvfp4_prefill_projection(const float * input_f32, const std::vector<std::uint8_t> & packed_weights,
                                  const std::vector<std::uint8_t> & weight_scales_e4m3, float weight_scale_2,
                                  int sequence_length, int rows, int cols, int warmup_iterations,
                                  int benchmark_iterations, double & avg_iteration_ms, double & max_abs_error,
                                  std::string & error_message);

// The reference's gate/up benchmark (run_nvfp4_cublaslt_gate_up_benchmark, include/qwen35x/runtime/cuda_bench.h, body
// src/runtime/cuda_bench.cu:2766-2903): one token through gate_proj and up_proj ending in silu(gate) * up.  Here the two
// tensors become one gate/up weight and one work-list launch of the decode kernel with its fused epilogue;
// max_abs_error (an addition) compares the first 64 outputs with the host loop.
bool run_nvfp4_gate_up_benchmark(const std::vector<std::uint8_t> & gate_packed_weights,
                                 const std::vector<std::uint8_t> & gate_weight_scales_e4m3, float gate_weight_scale_2,
                                 const std::vector<std::uint8_t> & up_packed_weights,
                                 const std::vector<std::uint8_t> & up_weight_scales_e4m3, float up_weight_scale_2, int rows,
                                 int cols, int warmup_iterations, int benchmark_iterations, double & avg_iteration_ms,
                                 double & max_abs_error, std::string & error_message);

// The role of run_nvfp4_cublaslt_probe (cuda_bench.h:29-40, body src/runtime/cuda_bench.cu:2190-2357): one quantised
// input row through the FP4 tensor-core path on the first `sample_rows` rows, compared with the host value computed
// from the same quantised input; here the path is the engine's quantiser + tcgen05 GEMM, not cuBLASLt.
bool run_nvfp4_fp4_probe(const std::vector<std::uint8_t> & packed_weights, const std::vector<std::uint8_t> & weight_scales_e4m3,
                         float weight_scale_2, int rows, int cols, int sample_rows, double & max_abs_error,
                         double & elapsed_ms, double & max_abs_expected, double & max_abs_actual,
                         std::string & error_message);

// Synthetic stand-in for a checkpoint tensor family: fp32 N(0, std) weights from a counter-based generator
// (splitmix64 + Box-Muller, one stream per seed), quantised on the GPU with the engine's NVFP4 recipe.
bool make_synthetic_tensor(int rows, int cols, std::uint64_t seed, float std_dev, std::vector<std::uint8_t> & packed,
                           std::vector<std::uint8_t> & scales, float & weight_scale_2, std::string & error_message);

}  // namespace q35b::runtime
