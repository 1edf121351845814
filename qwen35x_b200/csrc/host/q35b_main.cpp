// q35b command line: the reference CLI's NVFP4 projection modes (src/main.cpp:361-403, 592-758) on the B200 engine.
//
//   q35b --check-nvfp4-tensor            [--nvfp4-sample-rows N]
//   q35b --bench-nvfp4-projection        [--nvfp4-projection-kernel row|warp|scale-group|blackwell-fp4|b200-simt|b200-stream]
//   q35b --bench-nvfp4-prefill-projection [--nvfp4-prefill-seq-len S]
//   q35b --probe-nvfp4-cublaslt          [--nvfp4-sample-rows N]      (the FP4 tensor-core probe; here tcgen05, not cuBLASLt)
//        [--bench-warmup W] [--bench-iters K] (--synthetic ROWS,COLS[,SEED] | --hf-model-dir DIR [--nvfp4-tensor BASE])
//   q35b --bench-nvfp4-gate-up [--bench-warmup W] [--bench-iters K]
//        (--synthetic ROWS,COLS[,SEED] | --hf-model-dir DIR [--nvfp4-gate-tensor BASE] [--nvfp4-up-tensor BASE])
//   q35b --validate-nvfp4-model --hf-model-dir DIR [--expect-layers N [--full-attention-interval I]]
//
// The tensor family comes from a ModelOpt NVFP4 checkpoint directory (--hf-model-dir/--nvfp4-tensor, as in the
// reference, src/main.cpp:350-385) or from --synthetic (fp32 N(0, 0.02) weights quantised with the engine's NVFP4
// recipe).  --validate-nvfp4-model applies the checkpoint rules without touching the GPU (src/main.cpp:560-591).
// Output is the reference's `key: value` block.  Exit codes: 0 ok, 2 usage, 10 failure.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <string>
#include <vector>

#include "nvfp4_checkpoint.h"
#include "nvfp4_runtime.h"

namespace rt = q35b::runtime;

static void usage() {
  std::cerr << "usage: q35b (--check-nvfp4-tensor | --probe-nvfp4-cublaslt | --bench-nvfp4-projection |\n"
               "             --bench-nvfp4-prefill-projection | --bench-nvfp4-gate-up)\n"
               "            (--synthetic ROWS,COLS[,SEED] | --hf-model-dir DIR [--nvfp4-tensor BASE])\n"
               "            [--nvfp4-projection-kernel NAME] [--nvfp4-sample-rows N]\n"
               "            [--nvfp4-prefill-seq-len S] [--bench-warmup W] [--bench-iters K] [--nvfp4-input-scale F]\n"
               "            [--nvfp4-gate-tensor BASE] [--nvfp4-up-tensor BASE]\n"
               "       q35b --validate-nvfp4-model --hf-model-dir DIR [--expect-layers N [--full-attention-interval I]]\n";
}

int main(int argc, char ** argv) {
  enum Mode { kNone, kCheck, kBench, kPrefill, kValidate, kGateUp, kProbe } mode = kNone;
  std::string model_dir, tensor_base;
  // defaults of the reference's gate/up benchmark (include/qwen35x/runtime/runtime.h)
  std::string gate_base = "model.language_model.layers.0.mlp.gate_proj", up_base = "model.language_model.layers.0.mlp.up_proj";
  int expect_layers = 0, full_interval = 4;
  bool input_scale_given = false;
  std::string kernel = "scale-group";
  int rows = 0, cols = 0, sample_rows = 16, seq_len = 256, warmup = 5, iters = 20;
  unsigned long long seed = 42;
  float input_scale = 1.0f;
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    auto value = [&](const char * flag) -> const char * {
      if (i + 1 >= argc) {
        std::cerr << flag << " needs a value\n";
        std::exit(2);
      }
      return argv[++i];
    };
    if (a == "--check-nvfp4-tensor") mode = kCheck;
    else if (a == "--bench-nvfp4-projection") mode = kBench;
    else if (a == "--bench-nvfp4-prefill-projection") mode = kPrefill;
    else if (a == "--bench-nvfp4-gate-up") mode = kGateUp;
    else if (a == "--probe-nvfp4-cublaslt") mode = kProbe;
    else if (a == "--nvfp4-gate-tensor") gate_base = value("--nvfp4-gate-tensor");
    else if (a == "--nvfp4-up-tensor") up_base = value("--nvfp4-up-tensor");
    else if (a == "--nvfp4-projection-kernel") kernel = value("--nvfp4-projection-kernel");
    else if (a == "--nvfp4-sample-rows") sample_rows = std::atoi(value("--nvfp4-sample-rows"));
    else if (a == "--nvfp4-prefill-seq-len") seq_len = std::atoi(value("--nvfp4-prefill-seq-len"));
    else if (a == "--bench-warmup") warmup = std::atoi(value("--bench-warmup"));
    else if (a == "--bench-iters") iters = std::atoi(value("--bench-iters"));
    else if (a == "--nvfp4-input-scale") {
      input_scale = static_cast<float>(std::atof(value("--nvfp4-input-scale")));
      input_scale_given = true;
    } else if (a == "--validate-nvfp4-model") mode = kValidate;
    else if (a == "--hf-model-dir") model_dir = value("--hf-model-dir");
    else if (a == "--nvfp4-tensor") tensor_base = value("--nvfp4-tensor");
    else if (a == "--expect-layers") expect_layers = std::atoi(value("--expect-layers"));
    else if (a == "--full-attention-interval") full_interval = std::atoi(value("--full-attention-interval"));
    else if (a == "--synthetic") {
      const std::string v = value("--synthetic");
      if (std::sscanf(v.c_str(), "%d,%d,%llu", &rows, &cols, &seed) < 2) {
        std::cerr << "--synthetic expects ROWS,COLS[,SEED]\n";
        return 2;
      }
    } else if (a == "--help" || a == "-h") {
      usage();
      return 0;
    } else {
      std::cerr << "unknown argument: " << a << "\n";
      usage();
      return 2;
    }
  }
  std::string error;
  if (mode == kValidate) {
    if (model_dir.empty()) {
      std::cerr << "NVFP4 model validation failed: --hf-model-dir is required\n";
      return 10;
    }
    namespace ck = q35b::checkpoint;
    ck::ValidationResult result;
    const std::vector<std::string> bases =
      expect_layers > 0 ? ck::expected_module_bases(expect_layers, full_interval) : std::vector<std::string>();
    if (!ck::validate_nvfp4_checkpoint(model_dir, bases, result, error)) {
      std::cerr << "NVFP4 model validation failed: " << error << "\n";
      return 10;
    }
    std::cout << "ModelOpt NVFP4 validation passed\n"
              << "  model_dir: " << model_dir << "\n"
              << "  group_size: " << result.group_size << "\n"
              << "  quantized_modules: " << result.quantized_tensors << "\n"
              << "  packed_u8_tensors: " << result.packed_u8_tensors << "\n"
              << "  fp8_scale_tensors: " << result.fp8_scale_tensors << "\n"
              << "  f32_input_scale_tensors: " << result.f32_input_scale_tensors << "\n"
              << "  f32_weight_scale2_tensors: " << result.f32_weight_scale2_tensors << "\n";
    return 0;
  }
  const bool from_checkpoint = !model_dir.empty();
  if (mode == kNone || (!from_checkpoint && (rows <= 0 || cols <= 0))) {
    usage();
    return 2;
  }

  if (mode == kGateUp) {
    // two tensor families: gate_proj and up_proj of one MLP (src/main.cpp:760-790, src/runtime/runtime.cpp:280-360)
    std::vector<std::uint8_t> g_packed, g_scales, u_packed, u_scales;
    float g_s2 = 1.0f, u_s2 = 1.0f;
    if (from_checkpoint) {
      q35b::checkpoint::Nvfp4Tensor g, u;
      if (!q35b::checkpoint::load_nvfp4_tensor(model_dir, gate_base, g, error) ||
          !q35b::checkpoint::load_nvfp4_tensor(model_dir, up_base, u, error)) {
        std::cerr << "NVFP4 gate/up benchmark failed: " << error << "\n";
        return 10;
      }
      if (g.rows != u.rows || g.cols != u.cols) {
        std::cerr << "NVFP4 gate/up benchmark failed: Gate and up packed weight shapes must match for benchmark.\n";
        return 10;
      }
      g_packed = std::move(g.packed_weights); g_scales = std::move(g.weight_scales); g_s2 = g.weight_scale_2;
      u_packed = std::move(u.packed_weights); u_scales = std::move(u.weight_scales); u_s2 = u.weight_scale_2;
      rows = g.rows;
      cols = g.cols;
    } else {
      if (!rt::make_synthetic_tensor(rows, cols, seed, 0.02f, g_packed, g_scales, g_s2, error) ||
          !rt::make_synthetic_tensor(rows, cols, seed + 1, 0.02f, u_packed, u_scales, u_s2, error)) {
        std::cerr << "NVFP4 synthetic tensor failed: " << error << "\n";
        return 10;
      }
      gate_base = "synthetic[" + std::to_string(rows) + "," + std::to_string(cols) + "] seed " + std::to_string(seed);
      up_base = "synthetic[" + std::to_string(rows) + "," + std::to_string(cols) + "] seed " + std::to_string(seed + 1);
    }
    double avg_ms = 0.0, max_abs_error = 0.0;
    if (!rt::run_nvfp4_gate_up_benchmark(g_packed, g_scales, g_s2, u_packed, u_scales, u_s2, rows, cols, warmup, iters, avg_ms,
                                         max_abs_error, error)) {
      std::cerr << "NVFP4 gate/up benchmark failed: " << error << "\n";
      return 10;
    }
    std::cout << "NVFP4 gate/up benchmark\n"
              << "  gate_tensor_base: " << gate_base << "\n"
              << "  up_tensor_base: " << up_base << "\n"
              << "  source_shape: " << rows << "x" << cols << "\n"
              << "  avg_iteration_ms: " << avg_ms << "\n"
              << "  iterations_per_second: " << 1000.0 / avg_ms << "\n"
              << "  max_abs_error: " << max_abs_error << "\n";
    return 0;
  }

  std::vector<std::uint8_t> packed, scales;
  float s2 = 1.0f;
  std::string tensor;
  if (from_checkpoint) {
    // default tensors of the reference's modes (include/qwen35x/runtime/runtime.h:31,56,76)
    if (tensor_base.empty()) {
      tensor_base = mode == kCheck ? "model.language_model.layers.0.linear_attn.in_proj_qkv" : "model.language_model.layers.0.mlp.gate_proj";
    }
    q35b::checkpoint::Nvfp4Tensor t;
    if (!q35b::checkpoint::load_nvfp4_tensor(model_dir, tensor_base, t, error)) {
      std::cerr << "NVFP4 tensor load failed: " << error << "\n";
      return 10;
    }
    packed = std::move(t.packed_weights);
    scales = std::move(t.weight_scales);
    s2 = t.weight_scale_2;
    rows = t.rows;
    cols = t.cols;
    if (!input_scale_given) input_scale = t.input_scale;
    tensor = tensor_base;
  } else {
    if (!rt::make_synthetic_tensor(rows, cols, seed, 0.02f, packed, scales, s2, error)) {
      std::cerr << "NVFP4 synthetic tensor failed: " << error << "\n";
      return 10;
    }
    tensor = "synthetic[" + std::to_string(rows) + "," + std::to_string(cols) + "] seed " + std::to_string(seed);
  }

  if (mode == kCheck) {
    double max_abs_error = 0.0;
    if (!rt::run_nvfp4_matvec_check(packed, scales, input_scale, s2, rows, cols, sample_rows, max_abs_error, error)) {
      std::cerr << "NVFP4 tensor check failed: " << error << "\n";
      return 10;
    }
    std::cout << "nvfp4_tensor_check:\n"
              << "  tensor: " << tensor << "\n"
              << "  source_shape: [" << rows << ", " << cols << "]\n"
              << "  packed_shape: [" << rows << ", " << cols / 2 << "]\n"
              << "  scale_shape: [" << rows << ", " << cols / 16 << "]\n"
              << "  sample_rows: " << sample_rows << "\n"
              << "  max_abs_error: " << max_abs_error << "\n";
    return 0;
  }
  if (mode == kProbe) {
    double max_abs_error = 0.0, elapsed_ms = 0.0, max_abs_expected = 0.0, max_abs_actual = 0.0;
    if (!rt::run_nvfp4_fp4_probe(packed, scales, s2, rows, cols, sample_rows, max_abs_error, elapsed_ms, max_abs_expected,
                                 max_abs_actual, error)) {
      std::cerr << "NVFP4 cuBLASLt probe failed: " << error << "\n";
      return 10;
    }
    std::cout << "NVFP4 cuBLASLt probe\n"
              << "  backend_note: sm_100a tcgen05 mxf4nvf4 block-scale path in place of cuBLASLt\n"
              << "  tensor_base: " << tensor << "\n"
              << "  source_shape: " << rows << "x" << cols << "\n"
              << "  packed_shape: " << rows << "x" << cols / 2 << "\n"
              << "  scale_shape: " << rows << "x" << cols / 16 << "\n"
              << "  sample_rows: " << std::min(rows, std::max(1, sample_rows)) << "\n"
              << "  elapsed_ms: " << elapsed_ms << "\n"
              << "  max_abs_expected: " << max_abs_expected << "\n"
              << "  max_abs_actual: " << max_abs_actual << "\n"
              << "  max_abs_error: " << max_abs_error << "\n";
    return 0;
  }
  if (mode == kBench) {
    int variant = 0;
    if (!rt::parse_projection_kernel(kernel, variant, error)) {
      std::cerr << "NVFP4 projection benchmark failed: " << error << "\n";
      return 10;
    }
    double avg_ms = 0.0, max_abs_error = 0.0;
    if (!rt::run_nvfp4_custom_projection_benchmark(packed, scales, input_scale, s2, rows, cols, variant, warmup, iters, avg_ms,
                                                   max_abs_error, error)) {
      std::cerr << "NVFP4 projection benchmark failed: " << error << "\n";
      return 10;
    }
    const double bytes = static_cast<double>(rows) * cols * (0.5 + 1.0 / 16.0);
    std::cout << "nvfp4_projection_benchmark:\n"
              << "  tensor: " << tensor << "\n"
              << "  kernel: " << kernel << "\n"
              << "  backend_note: " << rt::projection_kernel_note(variant) << "\n"
              << "  source_shape: [" << rows << ", " << cols << "]\n"
              << "  avg_iteration_ms: " << avg_ms << "\n"
              << "  iterations_per_second: " << 1000.0 / avg_ms << "\n"
              << "  weight_gbytes_per_second: " << bytes / (avg_ms * 1e-3) / 1e9 << "\n"
              << "  max_abs_error: " << max_abs_error << "\n";
    return 0;
  }
  // prefill: the reference's input sin((i % 251) * 0.03125) * 0.25 (src/runtime/runtime.cpp:498-501)
  std::vector<float> input(static_cast<size_t>(seq_len) * cols);
  for (size_t i = 0; i < input.size(); ++i) input[i] = std::sin(static_cast<float>(i % 251) * 0.03125f) * 0.25f;
  double avg_ms = 0.0, max_abs_error = 0.0;
  if (!rt::run_nvfp4_prefill_projection(input.data(), packed, scales, s2, seq_len, rows, cols, warmup, iters, avg_ms,
                                        max_abs_error, error)) {
    std::cerr << "NVFP4 prefill projection benchmark failed: " << error << "\n";
    return 10;
  }
  std::cout << "nvfp4_prefill_projection_benchmark:\n"
            << "  tensor: " << tensor << "\n"
            << "  source_shape: [" << rows << ", " << cols << "]\n"
            << "  sequence_length: " << seq_len << "\n"
            << "  avg_iteration_ms: " << avg_ms << "\n"
            << "  iterations_per_second: " << 1000.0 / avg_ms << "\n"
            << "  tflops: " << 2.0 * seq_len * rows * cols / (avg_ms * 1e-3) / 1e12 << "\n"
            << "  max_abs_error: " << max_abs_error << "\n";
  return 0;
}
