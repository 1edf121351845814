/*
 * Reference shim.  TEST INFRASTRUCTURE ONLY.
 *
 * Compiles the reference's own translation unit src/runtime/cuda_bench.cu
 * unmodified, from where it lies in the reference checkout (the include below
 * is resolved by a -D/-I given by oracle/build_oracle.py), and exposes a few
 * of its internal-linkage functions and kernels through extern "C" wrappers so
 * that tests can compare the oracle with the reference itself:
 *   - host codecs/encoders/layout helpers: callable without a GPU;
 *   - the reference's CUDA kernels and bridges: callable on a GPU box, used to
 *     check the oracle against reference outputs and to time the reference's
 *     kernels beside the engine's.
 * Nothing of the reference is copied here; the output goes to oracle/_ref/.
 */
#ifndef QWEN35X_HAS_CUDA
#define QWEN35X_HAS_CUDA 1
#endif
#include QWEN35X_REF_CUDA_BENCH_CU

#include <cstring>

#define REF_API extern "C" __attribute__((visibility("default")))

namespace qc = qwen35x::cuda;

static thread_local std::string g_ref_error;

REF_API const char * ref_last_error() { return g_ref_error.c_str(); }

/* ---- host functions (no GPU needed) ---- */
REF_API float ref_decode_e2m1(std::uint8_t nibble) { return qc::decode_nvfp4_e2m1_host(nibble); }
REF_API float ref_decode_e4m3(std::uint8_t bits) { return qc::decode_e4m3_host(bits); }
REF_API std::uint8_t ref_encode_ue4m3(float v) { return qc::encode_ue4m3_scale(v); }
REF_API std::uint8_t ref_encode_e2m1(float v) { return qc::encode_nvfp4_e2m1(v); }

REF_API long long ref_swizzle_scales(const std::uint8_t * scale, int rows, int cols, std::uint8_t * out, long long out_capacity) {
  std::vector<std::uint8_t> in(scale, scale + static_cast<std::size_t>(rows) * cols);
  const auto sw = qc::swizzle_nvfp4_block_scale(in, rows, cols);
  if (static_cast<long long>(sw.size()) > out_capacity) return -static_cast<long long>(sw.size());
  std::memcpy(out, sw.data(), sw.size());
  return static_cast<long long>(sw.size());
}

REF_API void ref_swap_nibbles(const std::uint8_t * data, long long bytes, std::uint8_t * out) {
  const auto sw = qc::swap_fp4_nibbles(data, static_cast<std::size_t>(bytes));
  std::memcpy(out, sw.data(), sw.size());
}

/* ---- GPU functions (device pointers; legacy default stream as the reference) ---- */

/* The reference's W4A16 kernels on caller-owned device buffers.
 * variant: 0 = row, 1 = warp, 2 = scale-group, 4 = thread-per-row check kernel
 * (launch shapes as cuda_bench.cu:2016-2019 and :2138-2147). Returns 0 on success. */
REF_API int ref_w4a16_projection(const std::uint8_t * d_codes, const std::uint8_t * d_scales, const float * d_input,
                                 float input_scale, float s2, float * d_output, int rows, int cols, int variant) {
  if (variant == 4) {
    const int threads = 128;
    const int blocks = (rows + threads - 1) / threads;
    qc::nvfp4_matvec_check_kernel<<<blocks, threads>>>(d_codes, d_scales, d_input, input_scale, s2, d_output, rows, cols, rows);
  } else if (variant == 1) {
    const int threads = 256;
    const int rows_per_block = threads / 32;
    qc::nvfp4_projection_warp_rows_kernel<<<(rows + rows_per_block - 1) / rows_per_block, threads>>>(
      d_codes, d_scales, d_input, input_scale, s2, d_output, rows, cols);
  } else if (variant == 2) {
    qc::nvfp4_projection_scale_group_kernel<<<rows, 256>>>(d_codes, d_scales, d_input, input_scale, s2, d_output, rows, cols);
  } else {
    qc::nvfp4_projection_row_parallel_kernel<<<rows, 256>>>(d_codes, d_scales, d_input, input_scale, s2, d_output, rows, cols);
  }
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { g_ref_error = cudaGetErrorString(e); return 1; }
  return 0;
}

/* run_nvfp4_custom_projection_benchmark (cuda_bench.h:42-54) on host tensors. */
REF_API int ref_custom_projection_benchmark(const std::uint8_t * codes, const std::uint8_t * scales, float input_scale,
                                            float s2, int rows, int cols, int variant, int warmup, int iters,
                                            double * avg_ms, double * max_abs_error) {
  std::vector<std::uint8_t> w(codes, codes + static_cast<std::size_t>(rows) * (cols / 2));
  std::vector<std::uint8_t> s(scales, scales + static_cast<std::size_t>(rows) * (cols / 16));
  g_ref_error.clear();
  const bool ok = qc::run_nvfp4_custom_projection_benchmark(w, s, input_scale, s2, rows, cols, variant, warmup, iters,
                                                           *avg_ms, *max_abs_error, g_ref_error);
  return ok ? 0 : 1;
}

/* The reference's BF16 activation quantiser kernel (cuda_bench.cu:178-213),
 * launched as cuda_bench.cu:2639. Output buffers must be zeroed by the caller. */
REF_API int ref_quantize_bf16_matrix(const void * d_input_bf16, std::uint8_t * d_codes, std::uint8_t * d_scales_tiled,
                                     int rows, int cols) {
  qc::nvfp4_quantize_bf16_matrix_for_cublaslt_kernel<<<dim3(cols / 16, rows), 16>>>(
    static_cast<const __nv_bfloat16 *>(d_input_bf16), d_codes, d_scales_tiled, rows, cols);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { g_ref_error = cudaGetErrorString(e); return 1; }
  return 0;
}

/* run_nvfp4_cublaslt_prefill_projection_device_bf16 (cuda_bench.h:70-83): the reference's
 * W4A4 prefill GEMM (activation quantise + cuBLASLt FP4 matmul), fp32 output [S, rows]. */
REF_API int ref_cublaslt_prefill_bf16(const void * d_input_bf16, const std::uint8_t * d_weights_swapped,
                                      const std::uint8_t * d_weight_scales_tiled, const float * d_s2, int seq, int rows,
                                      int cols, std::uint8_t * d_act_scratch, std::uint8_t * d_act_scale_scratch,
                                      float * d_output_f32, double * elapsed_ms) {
  g_ref_error.clear();
  const bool ok = qc::run_nvfp4_cublaslt_prefill_projection_device_bf16(
    d_input_bf16, d_weights_swapped, d_weight_scales_tiled, d_s2, seq, rows, cols, d_act_scratch, d_act_scale_scratch,
    d_output_f32, elapsed_ms, g_ref_error);
  return ok ? 0 : 1;
}
