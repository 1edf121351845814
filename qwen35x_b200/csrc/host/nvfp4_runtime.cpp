#include "nvfp4_runtime.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <string>

#include "../../../include/q35b_nvfp4.h"
#include "../nvfp4_codec.cuh"

namespace q35b::runtime {
namespace {

bool ok(int status, std::string & error_message) {
  if (status == Q35B_OK) return true;
  error_message = q35b_last_error();
  return false;
}

bool cuda_ok(cudaError_t e, const char * what, std::string & error_message) {
  if (e == cudaSuccess) return true;
  error_message = std::string(what) + " failed: " + cudaGetErrorString(e);
  return false;
}

// Frees everything it was given when it goes out of scope.
struct DeviceBuffers {
  std::vector<void *> ptrs;
  q35b_weight * weight = nullptr;
  cudaEvent_t start = nullptr, stop = nullptr;
  ~DeviceBuffers() {
    for (void * p : ptrs) cudaFree(p);
    if (weight) q35b_weight_destroy(weight);
    if (start) cudaEventDestroy(start);
    if (stop) cudaEventDestroy(stop);
  }
  template <typename T>
  bool alloc(T ** p, size_t bytes, const char * what, std::string & err) {
    void * q = nullptr;
    if (!cuda_ok(cudaMalloc(&q, bytes), what, err)) return false;
    ptrs.push_back(q);
    *p = static_cast<T *>(q);
    return true;
  }
};

// The reference's fixed benchmark input, x[i] = ((i % 17) - 8) / 17 (src/runtime/cuda_bench.cu:2085-2088).
std::vector<float> fixed_input(int cols) {
  std::vector<float> x(static_cast<size_t>(cols));
  for (int i = 0; i < cols; ++i) x[static_cast<size_t>(i)] = static_cast<float>((i % 17) - 8) / 17.0f;
  return x;
}

// Host expected value of the first `check_rows` rows: the loop at src/runtime/cuda_bench.cu:2091-2100.
std::vector<float> host_expected(const std::vector<std::uint8_t> & packed, const std::vector<std::uint8_t> & scales,
                                 float input_scale, float s2, int cols, int check_rows, const float * x) {
  const int packed_cols = cols / 2, scale_cols = cols / 16;
  std::vector<float> expected(static_cast<size_t>(check_rows), 0.0f);
  for (int row = 0; row < check_rows; ++row) {
    for (int c = 0; c < cols; ++c) {
      const std::uint8_t p = packed[static_cast<size_t>(row) * packed_cols + c / 2];
      const std::uint8_t nibble = (c & 1) == 0 ? (p & 0x0fu) : static_cast<std::uint8_t>(p >> 4u);
      const float scale = decode_e4m3(scales[static_cast<size_t>(row) * scale_cols + c / 16]) * s2;
      expected[static_cast<size_t>(row)] += decode_e2m1(nibble) * scale * (x[c] * input_scale);
    }
  }
  return expected;
}

bool check_dims(const std::vector<std::uint8_t> & packed, const std::vector<std::uint8_t> & scales, int rows, int cols,
                const char * what, std::string & error_message) {
  if (rows <= 0 || cols <= 0 || (cols % 16) != 0 || (cols % 2) != 0) {
    error_message = std::string("Invalid matrix dimensions for ") + what + ".";
    return false;
  }
  if (packed.size() != static_cast<size_t>(rows) * (cols / 2) || scales.size() != static_cast<size_t>(rows) * (cols / 16)) {
    error_message = "NVFP4 packed weight or scale size does not match matrix dimensions.";
    return false;
  }
  return true;
}

}  // namespace

bool parse_projection_kernel(const std::string & name, int & kernel_variant, std::string & error_message) {
  if (name == "row") kernel_variant = kRow;
  else if (name == "warp") kernel_variant = kWarp;
  else if (name == "scale-group") kernel_variant = kScaleGroup;
  else if (name == "blackwell-fp4") kernel_variant = kBlackwellFp4;
  else if (name == "b200-simt") kernel_variant = kB200Simt;
  else if (name == "b200-stream") kernel_variant = kB200Stream;
  else {
    error_message = "unknown custom NVFP4 projection kernel: " + name +
                    " (expected row|warp|scale-group|blackwell-fp4|b200-simt|b200-stream).";
    return false;
  }
  return true;
}

const char * projection_kernel_note(int kernel_variant) {
  switch (kernel_variant) {
    case kBlackwellFp4: return "sm_100a tcgen05 mxf4nvf4 block-scale path (activation quantised to NVFP4 on the GPU)";
    case kB200Stream: return "sm_100a persistent TMA-fed streaming decode kernel";
    default: return "sm_100a vectorised SIMT decode kernel (128-bit loads, in-register dequant, warp-shuffle reduction)";
  }
}

bool run_nvfp4_matvec_check(const std::vector<std::uint8_t> & packed_weights,
                            const std::vector<std::uint8_t> & weight_scales_e4m3, float input_scale,
                            float weight_scale_2, int rows, int cols, int sample_rows, double & max_abs_error,
                            std::string & error_message) {
  (void)input_scale;  // the reference's check runs with input_scale = 1 (src/runtime/cuda_bench.cu:1984,2019)
  if (rows <= 0 || cols <= 0 || (cols % 16) != 0) {
    error_message = "Invalid matrix dimensions for NVFP4 check.";
    return false;
  }
  if (!check_dims(packed_weights, weight_scales_e4m3, rows, cols, "NVFP4 check", error_message)) return false;
  sample_rows = std::max(1, std::min(sample_rows, rows));
  const std::vector<float> x = fixed_input(cols);
  const std::vector<float> expected = host_expected(packed_weights, weight_scales_e4m3, 1.0f, weight_scale_2, cols, sample_rows, x.data());

  DeviceBuffers d;
  float * d_x = nullptr;
  float * d_y = nullptr;
  if (!ok(q35b_weight_create(packed_weights.data(), weight_scales_e4m3.data(), weight_scale_2, 1.0f, rows, cols, 0, 1, &d.weight), error_message) ||
      !d.alloc(&d_x, x.size() * sizeof(float), "cudaMalloc(nvfp4 input)", error_message) ||
      !d.alloc(&d_y, static_cast<size_t>(rows) * sizeof(float), "cudaMalloc(nvfp4 output)", error_message) ||
      !cuda_ok(cudaMemcpy(d_x, x.data(), x.size() * sizeof(float), cudaMemcpyHostToDevice), "cudaMemcpy(nvfp4 input)", error_message) ||
      !ok(q35b_gemv_w4a16_f32(d.weight, d_x, 1.0f, d_y, Q35B_GEMV_SIMT, nullptr), error_message)) {
    return false;
  }
  std::vector<float> actual(static_cast<size_t>(sample_rows));
  if (!cuda_ok(cudaMemcpy(actual.data(), d_y, actual.size() * sizeof(float), cudaMemcpyDeviceToHost), "cudaMemcpy(nvfp4 output)", error_message)) {
    return false;
  }
  max_abs_error = 0.0;
  for (int r = 0; r < sample_rows; ++r) {
    max_abs_error = std::max(max_abs_error, static_cast<double>(std::fabs(actual[static_cast<size_t>(r)] - expected[static_cast<size_t>(r)])));
  }
  return true;
}

bool run_nvfp4_custom_projection_benchmark(const std::vector<std::uint8_t> & packed_weights,
                                           const std::vector<std::uint8_t> & weight_scales_e4m3, float input_scale,
                                           float weight_scale_2, int rows, int cols, int kernel_variant,
                                           int warmup_iterations, int benchmark_iterations, double & avg_iteration_ms,
                                           double & max_abs_error, std::string & error_message) {
  if (rows <= 0 || cols <= 0 || (cols % 16) != 0 || (cols % 2) != 0) {
    error_message = "Invalid matrix dimensions for custom NVFP4 projection benchmark.";
    return false;
  }
  if (warmup_iterations < 0 || benchmark_iterations <= 0) {
    error_message = "warmup_iterations must be >= 0 and benchmark_iterations must be > 0.";
    return false;
  }
  if (!check_dims(packed_weights, weight_scales_e4m3, rows, cols, "custom NVFP4 projection benchmark", error_message)) return false;
  const std::vector<float> x = fixed_input(cols);
  const int check_rows = std::min(rows, 64);
  const std::vector<float> expected = host_expected(packed_weights, weight_scales_e4m3, input_scale, weight_scale_2, cols, check_rows, x.data());

  DeviceBuffers d;
  if (!ok(q35b_weight_create(packed_weights.data(), weight_scales_e4m3.data(), weight_scale_2, input_scale, rows, cols, 0, 1, &d.weight), error_message)) {
    return false;
  }
  if (!cuda_ok(cudaEventCreate(&d.start), "cudaEventCreate", error_message) ||
      !cuda_ok(cudaEventCreate(&d.stop), "cudaEventCreate", error_message)) {
    return false;
  }
  std::vector<float> actual(static_cast<size_t>(check_rows));

  if (kernel_variant == kBlackwellFp4 || kernel_variant == kB200Stream) {
    // BF16 activation paths: x * input_scale rounded to BF16 on the host, BF16 output.
    std::vector<std::uint16_t> xb(x.size());
    for (size_t i = 0; i < x.size(); ++i) xb[i] = f32_to_bf16_bits(x[i] * input_scale);
    std::uint16_t * d_x = nullptr;
    std::uint16_t * d_y = nullptr;
    std::uint8_t * d_codes = nullptr;
    std::uint8_t * d_scales = nullptr;
    float * d_g = nullptr;
    void * d_ws = nullptr;
    if (!d.alloc(&d_x, xb.size() * 2, "cudaMalloc(nvfp4 input)", error_message) ||
        !d.alloc(&d_y, static_cast<size_t>(rows) * 2, "cudaMalloc(nvfp4 output)", error_message) ||
        !d.alloc(&d_codes, q35b_act_codes_bytes(1, cols), "cudaMalloc(fp4 activation)", error_message) ||
        !d.alloc(&d_scales, q35b_act_scales_bytes(1, cols), "cudaMalloc(fp4 activation scales)", error_message) ||
        !d.alloc(&d_g, sizeof(float), "cudaMalloc(fp4 input scale)", error_message) ||
        !d.alloc(&d_ws, q35b_quant_workspace_bytes(), "cudaMalloc(quantiser workspace)", error_message) ||
        !cuda_ok(cudaMemset(d_ws, 0, q35b_quant_workspace_bytes()), "cudaMemset(quantiser workspace)", error_message) ||
        !cuda_ok(cudaMemcpy(d_x, xb.data(), xb.size() * 2, cudaMemcpyHostToDevice), "cudaMemcpy(nvfp4 input)", error_message)) {
      return false;
    }
    auto launch = [&]() -> bool {
      if (kernel_variant == kB200Stream) {
        return ok(q35b_gemv_w4a16_bf16(d.weight, d_x, 1, d_y, Q35B_GEMV_STREAM, nullptr), error_message);
      }
      return ok(q35b_quantize_nvfp4_bf16(d_x, 1, cols, 0.0f, d_codes, d_scales, d_g, d_ws, nullptr), error_message) &&
             ok(q35b_gemm_w4a4_bf16(d.weight, d_codes, d_scales, d_g, 1, d_y, rows, nullptr, nullptr), error_message);
    };
    for (int i = 0; i < warmup_iterations; ++i) {
      if (!launch()) return false;
    }
    if (!cuda_ok(cudaEventRecord(d.start), "cudaEventRecord", error_message)) return false;
    for (int i = 0; i < benchmark_iterations; ++i) {
      if (!launch()) return false;
    }
    float ms = 0.0f;
    if (!cuda_ok(cudaEventRecord(d.stop), "cudaEventRecord", error_message) ||
        !cuda_ok(cudaEventSynchronize(d.stop), "cudaEventSynchronize", error_message) ||
        !cuda_ok(cudaEventElapsedTime(&ms, d.start, d.stop), "cudaEventElapsedTime", error_message)) {
      return false;
    }
    avg_iteration_ms = static_cast<double>(ms) / benchmark_iterations;
    std::vector<std::uint16_t> yb(static_cast<size_t>(check_rows));
    if (!cuda_ok(cudaMemcpy(yb.data(), d_y, yb.size() * 2, cudaMemcpyDeviceToHost), "cudaMemcpy(nvfp4 output)", error_message)) return false;
    for (int r = 0; r < check_rows; ++r) actual[static_cast<size_t>(r)] = bf16_bits_to_f32(yb[static_cast<size_t>(r)]);
  } else {
    float * d_x = nullptr;
    float * d_y = nullptr;
    if (!d.alloc(&d_x, x.size() * sizeof(float), "cudaMalloc(nvfp4 input)", error_message) ||
        !d.alloc(&d_y, static_cast<size_t>(rows) * sizeof(float), "cudaMalloc(nvfp4 output)", error_message) ||
        !cuda_ok(cudaMemcpy(d_x, x.data(), x.size() * sizeof(float), cudaMemcpyHostToDevice), "cudaMemcpy(nvfp4 input)", error_message)) {
      return false;
    }
    for (int i = 0; i < warmup_iterations; ++i) {
      if (!ok(q35b_gemv_w4a16_f32(d.weight, d_x, input_scale, d_y, Q35B_GEMV_SIMT, nullptr), error_message)) return false;
    }
    if (!cuda_ok(cudaEventRecord(d.start), "cudaEventRecord", error_message)) return false;
    for (int i = 0; i < benchmark_iterations; ++i) {
      if (!ok(q35b_gemv_w4a16_f32(d.weight, d_x, input_scale, d_y, Q35B_GEMV_SIMT, nullptr), error_message)) return false;
    }
    float ms = 0.0f;
    if (!cuda_ok(cudaEventRecord(d.stop), "cudaEventRecord", error_message) ||
        !cuda_ok(cudaEventSynchronize(d.stop), "cudaEventSynchronize", error_message) ||
        !cuda_ok(cudaEventElapsedTime(&ms, d.start, d.stop), "cudaEventElapsedTime", error_message)) {
      return false;
    }
    avg_iteration_ms = static_cast<double>(ms) / benchmark_iterations;
    if (!cuda_ok(cudaMemcpy(actual.data(), d_y, actual.size() * sizeof(float), cudaMemcpyDeviceToHost), "cudaMemcpy(nvfp4 output)", error_message)) return false;
  }
  max_abs_error = 0.0;
  for (int r = 0; r < check_rows; ++r) {
    max_abs_error = std::max(max_abs_error, static_cast<double>(std::fabs(actual[static_cast<size_t>(r)] - expected[static_cast<size_t>(r)])));
  }
  return true;
}

bool run_nvfp4_prefill_projection(const float * input_f32, const std::vector<std::uint8_t> & packed_weights,
                                  const std::vector<std::uint8_t> & weight_scales_e4m3, float weight_scale_2,
                                  int sequence_length, int rows, int cols, int warmup_iterations,
                                  int benchmark_iterations, double & avg_iteration_ms, double & max_abs_error,
                                  std::string & error_message) {
  if (input_f32 == nullptr) {
    error_message = "NVFP4 prefill projection received a null input buffer.";
    return false;
  }
  if (sequence_length <= 0 || rows <= 0 || cols <= 0 || (cols % 16) != 0 || (cols % 2) != 0) {
    error_message = "Invalid dimensions for NVFP4 prefill projection.";
    return false;
  }
  if (warmup_iterations < 0 || benchmark_iterations <= 0) {
    error_message = "warmup_iterations must be >= 0 and benchmark_iterations must be > 0.";
    return false;
  }
  if (!check_dims(packed_weights, weight_scales_e4m3, rows, cols, "NVFP4 prefill projection", error_message)) return false;
  const size_t n_in = static_cast<size_t>(sequence_length) * cols;

  DeviceBuffers d;
  float * d_x = nullptr;
  std::uint16_t * d_y = nullptr;
  std::uint8_t * d_codes = nullptr;
  std::uint8_t * d_scales = nullptr;
  float * d_g = nullptr;
  void * d_ws = nullptr;
  if (!ok(q35b_weight_create(packed_weights.data(), weight_scales_e4m3.data(), weight_scale_2, 1.0f, rows, cols, 0, 1, &d.weight), error_message) ||
      !d.alloc(&d_x, n_in * sizeof(float), "cudaMalloc(prefill input)", error_message) ||
      !d.alloc(&d_y, static_cast<size_t>(sequence_length) * rows * 2, "cudaMalloc(prefill output)", error_message) ||
      !d.alloc(&d_codes, q35b_act_codes_bytes(sequence_length, cols), "cudaMalloc(prefill fp4 activation)", error_message) ||
      !d.alloc(&d_scales, q35b_act_scales_bytes(sequence_length, cols), "cudaMalloc(prefill fp4 activation scales)", error_message) ||
      !d.alloc(&d_g, sizeof(float), "cudaMalloc(prefill input scale)", error_message) ||
      !d.alloc(&d_ws, q35b_quant_workspace_bytes(), "cudaMalloc(quantiser workspace)", error_message) ||
      !cuda_ok(cudaMemset(d_ws, 0, q35b_quant_workspace_bytes()), "cudaMemset(quantiser workspace)", error_message) ||
      !cuda_ok(cudaMemcpy(d_x, input_f32, n_in * sizeof(float), cudaMemcpyHostToDevice), "cudaMemcpy(prefill input)", error_message) ||
      !cuda_ok(cudaEventCreate(&d.start), "cudaEventCreate", error_message) ||
      !cuda_ok(cudaEventCreate(&d.stop), "cudaEventCreate", error_message)) {
    return false;
  }
  auto launch = [&]() -> bool {
    // fp32 activations, as the reference's benchmark feeds its quantiser (src/runtime/cuda_bench.cu:141-176)
    return ok(q35b_quantize_nvfp4_f32(d_x, sequence_length, cols, 0.0f, d_codes, d_scales, d_g, d_ws, nullptr), error_message) &&
           ok(q35b_gemm_w4a4_bf16(d.weight, d_codes, d_scales, d_g, sequence_length, d_y, rows, nullptr, nullptr), error_message);
  };
  for (int i = 0; i < warmup_iterations; ++i) {
    if (!launch()) return false;
  }
  if (!cuda_ok(cudaEventRecord(d.start), "cudaEventRecord", error_message)) return false;
  for (int i = 0; i < benchmark_iterations; ++i) {
    if (!launch()) return false;
  }
  float ms = 0.0f;
  if (!cuda_ok(cudaEventRecord(d.stop), "cudaEventRecord", error_message) ||
      !cuda_ok(cudaEventSynchronize(d.stop), "cudaEventSynchronize", error_message) ||
      !cuda_ok(cudaEventElapsedTime(&ms, d.start, d.stop), "cudaEventElapsedTime", error_message)) {
    return false;
  }
  avg_iteration_ms = static_cast<double>(ms) / benchmark_iterations;
  const int check_tokens = std::min(sequence_length, 2), check_rows = std::min(rows, 8);
  std::vector<std::uint16_t> yb(static_cast<size_t>(check_tokens) * rows);
  if (!cuda_ok(cudaMemcpy(yb.data(), d_y, yb.size() * 2, cudaMemcpyDeviceToHost), "cudaMemcpy(prefill output)", error_message)) return false;
  max_abs_error = 0.0;
  for (int tok = 0; tok < check_tokens; ++tok) {
    const std::vector<float> expected = host_expected(packed_weights, weight_scales_e4m3, 1.0f, weight_scale_2, cols, check_rows,
                                                      input_f32 + static_cast<size_t>(tok) * cols);
    for (int r = 0; r < check_rows; ++r) {
      const float actual = bf16_bits_to_f32(yb[static_cast<size_t>(tok) * rows + r]);
      max_abs_error = std::max(max_abs_error, static_cast<double>(std::fabs(actual - expected[static_cast<size_t>(r)])));
    }
  }
  return true;
}

bool run_nvfp4_gate_up_benchmark(const std::vector<std::uint8_t> & gate_packed_weights,
                                 const std::vector<std::uint8_t> & gate_weight_scales_e4m3, float gate_weight_scale_2,
                                 const std::vector<std::uint8_t> & up_packed_weights,
                                 const std::vector<std::uint8_t> & up_weight_scales_e4m3, float up_weight_scale_2, int rows,
                                 int cols, int warmup_iterations, int benchmark_iterations, double & avg_iteration_ms,
                                 double & max_abs_error, std::string & error_message) {
  if (rows <= 0 || cols <= 0 || (cols % 16) != 0 || (cols % 2) != 0) {
    error_message = "Invalid matrix dimensions for NVFP4 gate/up benchmark.";
    return false;
  }
  if (warmup_iterations < 0 || benchmark_iterations <= 0) {
    error_message = "warmup_iterations must be >= 0 and benchmark_iterations must be > 0.";
    return false;
  }
  const size_t weight_bytes = static_cast<size_t>(rows) * (cols / 2), scale_bytes = static_cast<size_t>(rows) * (cols / 16);
  if (gate_packed_weights.size() != weight_bytes || up_packed_weights.size() != weight_bytes ||
      gate_weight_scales_e4m3.size() != scale_bytes || up_weight_scales_e4m3.size() != scale_bytes) {
    error_message = "NVFP4 gate/up benchmark tensor sizes do not match dimensions.";
    return false;
  }
  // one token, the reference's fixed input, BF16 on the device; output silu(gate x) * up x [rows]
  const std::vector<float> x = fixed_input(cols);
  std::vector<std::uint16_t> xb(x.size());
  std::vector<float> xr(x.size());
  for (size_t i = 0; i < x.size(); ++i) {
    xb[i] = f32_to_bf16_bits(x[i]);
    xr[i] = bf16_bits_to_f32(xb[i]);
  }
  DeviceBuffers d;
  std::uint16_t * d_x = nullptr;
  std::uint16_t * d_y = nullptr;
  q35b_gemv_batch * batch = nullptr;
  if (!ok(q35b_weight_create_gate_up(gate_packed_weights.data(), gate_weight_scales_e4m3.data(), gate_weight_scale_2,
                                     up_packed_weights.data(), up_weight_scales_e4m3.data(), up_weight_scale_2, rows, cols,
                                     &d.weight), error_message) ||
      !d.alloc(&d_x, xb.size() * 2, "cudaMalloc(gate/up input)", error_message) ||
      !d.alloc(&d_y, static_cast<size_t>(rows) * 2, "cudaMalloc(gate/up output)", error_message) ||
      !cuda_ok(cudaMemcpy(d_x, xb.data(), xb.size() * 2, cudaMemcpyHostToDevice), "cudaMemcpy(gate/up input)", error_message) ||
      !cuda_ok(cudaEventCreate(&d.start), "cudaEventCreate(gate/up start)", error_message) ||
      !cuda_ok(cudaEventCreate(&d.stop), "cudaEventCreate(gate/up stop)", error_message)) {
    return false;
  }
  const q35b_gemv_item item{d.weight, d_x, d_y, nullptr, 0};
  if (!ok(q35b_gemv_batch_create(&item, 1, 1, &batch), error_message)) return false;
  bool good = true;
  for (int i = 0; i < warmup_iterations && good; ++i) good = ok(q35b_gemv_batch_run(batch, nullptr), error_message);
  good = good && cuda_ok(cudaEventRecord(d.start), "cudaEventRecord(gate/up start)", error_message);
  for (int i = 0; i < benchmark_iterations && good; ++i) good = ok(q35b_gemv_batch_run(batch, nullptr), error_message);
  float ms = 0.0f;
  good = good && cuda_ok(cudaEventRecord(d.stop), "cudaEventRecord(gate/up stop)", error_message) &&
         cuda_ok(cudaEventSynchronize(d.stop), "cudaEventSynchronize(gate/up stop)", error_message) &&
         cuda_ok(cudaEventElapsedTime(&ms, d.start, d.stop), "cudaEventElapsedTime(gate/up)", error_message);
  unsigned int wait_code = 0;
  good = good && ok(q35b_gemv_batch_status(batch, &wait_code), error_message);
  q35b_gemv_batch_destroy(batch);
  if (!good) return false;
  if (wait_code != 0) {
    error_message = "A device-side wait of the NVFP4 gate/up projection expired (code " + std::to_string(wait_code) + ").";
    return false;
  }
  avg_iteration_ms = static_cast<double>(ms) / benchmark_iterations;
  const int check_rows = std::min(rows, 64);
  std::vector<std::uint16_t> yb(static_cast<size_t>(check_rows));
  if (!cuda_ok(cudaMemcpy(yb.data(), d_y, yb.size() * 2, cudaMemcpyDeviceToHost), "cudaMemcpy(gate/up output)", error_message)) return false;
  const std::vector<float> gate = host_expected(gate_packed_weights, gate_weight_scales_e4m3, 1.0f, gate_weight_scale_2, cols, check_rows, xr.data());
  const std::vector<float> up = host_expected(up_packed_weights, up_weight_scales_e4m3, 1.0f, up_weight_scale_2, cols, check_rows, xr.data());
  max_abs_error = 0.0;
  for (int r = 0; r < check_rows; ++r) {
    const float g = gate[static_cast<size_t>(r)];
    const float expected = g / (1.0f + std::exp(-g)) * up[static_cast<size_t>(r)];
    max_abs_error = std::max(max_abs_error, static_cast<double>(std::fabs(bf16_bits_to_f32(yb[static_cast<size_t>(r)]) - expected)));
  }
  return true;
}

bool run_nvfp4_fp4_probe(const std::vector<std::uint8_t> & packed_weights, const std::vector<std::uint8_t> & weight_scales_e4m3,
                         float weight_scale_2, int rows, int cols, int sample_rows, double & max_abs_error,
                         double & elapsed_ms, double & max_abs_expected, double & max_abs_actual,
                         std::string & error_message) {
  if (rows <= 0 || cols <= 0 || (cols % 64) != 0) {
    error_message = "Invalid matrix dimensions for NVFP4 tensor-core probe (cols must be a multiple of 64).";
    return false;
  }
  const int used_rows = std::min(rows, std::max(1, sample_rows));
  const int packed_cols = cols / 2, scale_cols = cols / 16;
  if (packed_weights.size() < static_cast<size_t>(used_rows) * packed_cols ||
      weight_scales_e4m3.size() < static_cast<size_t>(used_rows) * scale_cols) {
    error_message = "NVFP4 tensor buffers are smaller than the requested probe shape.";
    return false;
  }
  const std::vector<float> x = fixed_input(cols);
  // host quantisation of the one input row with the engine's recipe (per-tensor g, decoded-scale divisor)
  float amax = 0.0f;
  for (float v : x) amax = std::max(amax, std::fabs(v));
  const float g = amax > 0.0f ? amax / (6.0f * 448.0f) : 1.0f;
  std::vector<float> xq(x.size());
  for (int b = 0; b < scale_cols; ++b) {
    float bmax = 0.0f;
    for (int i = 0; i < 16; ++i) bmax = std::max(bmax, std::fabs(x[static_cast<size_t>(b) * 16 + i]));
    std::uint8_t sb = encode_ue4m3(std::max(bmax / 6.0f / g, 1.0e-8f));
    if (sb > 0x7e) sb = 0x7e;
    const float dd = std::max(decode_e4m3(sb), 1.0e-8f) * g;
    for (int i = 0; i < 16; ++i) {
      const size_t c = static_cast<size_t>(b) * 16 + i;
      xq[c] = decode_e2m1(encode_e2m1(x[c] / dd)) * decode_e4m3(sb) * g;
    }
  }
  const std::vector<float> expected = host_expected(packed_weights, weight_scales_e4m3, 1.0f, weight_scale_2, cols, used_rows, xq.data());

  DeviceBuffers d;
  float * d_x = nullptr;
  std::uint16_t * d_y = nullptr;
  std::uint8_t * d_codes = nullptr;
  std::uint8_t * d_scales = nullptr;
  float * d_g = nullptr;
  void * d_ws = nullptr;
  const std::vector<std::uint8_t> w_rows(packed_weights.begin(), packed_weights.begin() + static_cast<size_t>(used_rows) * packed_cols);
  const std::vector<std::uint8_t> s_rows(weight_scales_e4m3.begin(), weight_scales_e4m3.begin() + static_cast<size_t>(used_rows) * scale_cols);
  if (!ok(q35b_weight_create(w_rows.data(), s_rows.data(), weight_scale_2, 1.0f, used_rows, cols, 0, 1, &d.weight), error_message) ||
      !d.alloc(&d_x, x.size() * sizeof(float), "cudaMalloc(probe input)", error_message) ||
      !d.alloc(&d_y, static_cast<size_t>(used_rows) * 2, "cudaMalloc(probe output)", error_message) ||
      !d.alloc(&d_codes, q35b_act_codes_bytes(1, cols), "cudaMalloc(probe activation)", error_message) ||
      !d.alloc(&d_scales, q35b_act_scales_bytes(1, cols), "cudaMalloc(probe activation scales)", error_message) ||
      !d.alloc(&d_g, sizeof(float), "cudaMalloc(probe input scale)", error_message) ||
      !d.alloc(&d_ws, q35b_quant_workspace_bytes(), "cudaMalloc(quantiser workspace)", error_message) ||
      !cuda_ok(cudaMemset(d_ws, 0, q35b_quant_workspace_bytes()), "cudaMemset(quantiser workspace)", error_message) ||
      !cuda_ok(cudaMemcpy(d_x, x.data(), x.size() * sizeof(float), cudaMemcpyHostToDevice), "cudaMemcpy(probe input)", error_message) ||
      !cuda_ok(cudaEventCreate(&d.start), "cudaEventCreate", error_message) ||
      !cuda_ok(cudaEventCreate(&d.stop), "cudaEventCreate", error_message)) {
    return false;
  }
  auto launch = [&]() -> bool {
    return ok(q35b_quantize_nvfp4_f32(d_x, 1, cols, 0.0f, d_codes, d_scales, d_g, d_ws, nullptr), error_message) &&
           ok(q35b_gemm_w4a4_bf16(d.weight, d_codes, d_scales, d_g, 1, d_y, used_rows, nullptr, nullptr), error_message);
  };
  if (!launch()) return false;  // first call: set-up costs stay out of the timing, as in the reference's probe
  float ms = 0.0f;
  if (!cuda_ok(cudaEventRecord(d.start), "cudaEventRecord", error_message) || !launch() ||
      !cuda_ok(cudaEventRecord(d.stop), "cudaEventRecord", error_message) ||
      !cuda_ok(cudaEventSynchronize(d.stop), "cudaEventSynchronize", error_message) ||
      !cuda_ok(cudaEventElapsedTime(&ms, d.start, d.stop), "cudaEventElapsedTime", error_message)) {
    return false;
  }
  elapsed_ms = ms;
  unsigned int wait_code = 0;
  if (!ok(q35b_gemm_default_status(&wait_code), error_message)) return false;
  if (wait_code != 0) {
    error_message = "A device-side wait of the NVFP4 tensor-core probe expired (code " + std::to_string(wait_code) + ").";
    return false;
  }
  std::vector<std::uint16_t> yb(static_cast<size_t>(used_rows));
  if (!cuda_ok(cudaMemcpy(yb.data(), d_y, yb.size() * 2, cudaMemcpyDeviceToHost), "cudaMemcpy(probe output)", error_message)) return false;
  max_abs_error = max_abs_expected = max_abs_actual = 0.0;
  for (int r = 0; r < used_rows; ++r) {
    const double a = bf16_bits_to_f32(yb[static_cast<size_t>(r)]), e = expected[static_cast<size_t>(r)];
    max_abs_error = std::max(max_abs_error, std::fabs(a - e));
    max_abs_expected = std::max(max_abs_expected, std::fabs(e));
    max_abs_actual = std::max(max_abs_actual, std::fabs(a));
  }
  return true;
}

bool make_synthetic_tensor(int rows, int cols, std::uint64_t seed, float std_dev, std::vector<std::uint8_t> & packed,
                           std::vector<std::uint8_t> & scales, float & weight_scale_2, std::string & error_message) {
  if (rows <= 0 || cols <= 0 || (cols % 16) != 0) {
    error_message = "Invalid dimensions for a synthetic NVFP4 tensor.";
    return false;
  }
  const size_t n = static_cast<size_t>(rows) * cols;
  std::vector<float> w(n);
  std::uint64_t state = seed * 0x9e3779b97f4a7c15ull + 0x632be59bd9b4e019ull;
  auto next = [&state]() {
    std::uint64_t z = (state += 0x9e3779b97f4a7c15ull);
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
  };
  for (size_t i = 0; i < n; i += 2) {
    const double u1 = (static_cast<double>(next() >> 11) + 1.0) * (1.0 / 9007199254740993.0);
    const double u2 = static_cast<double>(next() >> 11) * (1.0 / 9007199254740992.0);
    const double r = std::sqrt(-2.0 * std::log(u1));
    w[i] = static_cast<float>(r * std::cos(6.283185307179586 * u2) * std_dev);
    if (i + 1 < n) w[i + 1] = static_cast<float>(r * std::sin(6.283185307179586 * u2) * std_dev);
  }
  DeviceBuffers d;
  float * d_w = nullptr;
  std::uint8_t * d_codes = nullptr;
  std::uint8_t * d_scales = nullptr;
  float * d_s2 = nullptr;
  void * d_ws = nullptr;
  packed.resize(n / 2);
  scales.resize(n / 16);
  return d.alloc(&d_w, n * sizeof(float), "cudaMalloc(synthetic weights)", error_message) &&
         d.alloc(&d_codes, n / 2, "cudaMalloc(synthetic codes)", error_message) &&
         d.alloc(&d_scales, n / 16, "cudaMalloc(synthetic scales)", error_message) &&
         d.alloc(&d_s2, sizeof(float), "cudaMalloc(synthetic weight_scale_2)", error_message) &&
         d.alloc(&d_ws, q35b_quant_workspace_bytes(), "cudaMalloc(quantiser workspace)", error_message) &&
         cuda_ok(cudaMemset(d_ws, 0, q35b_quant_workspace_bytes()), "cudaMemset(quantiser workspace)", error_message) &&
         cuda_ok(cudaMemcpy(d_w, w.data(), n * sizeof(float), cudaMemcpyHostToDevice), "cudaMemcpy(synthetic weights)", error_message) &&
         ok(q35b_quantize_weight_f32(d_w, rows, cols, d_codes, d_scales, d_s2, d_ws, nullptr), error_message) &&
         cuda_ok(cudaMemcpy(packed.data(), d_codes, n / 2, cudaMemcpyDeviceToHost), "cudaMemcpy(synthetic codes)", error_message) &&
         cuda_ok(cudaMemcpy(scales.data(), d_scales, n / 16, cudaMemcpyDeviceToHost), "cudaMemcpy(synthetic scales)", error_message) &&
         cuda_ok(cudaMemcpy(&weight_scale_2, d_s2, sizeof(float), cudaMemcpyDeviceToHost), "cudaMemcpy(synthetic weight_scale_2)", error_message);
}

}  // namespace q35b::runtime
