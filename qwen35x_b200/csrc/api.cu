// C ABI of libq35b: argument checking, weight repack, dispatch.
#include <algorithm>
#include <cstring>
#include <mutex>
#include <vector>

#include "engine.h"
#include "nvfp4_codec.cuh"

namespace q35b {

static thread_local std::string t_error;
std::atomic<unsigned long long> g_launches{0};

void set_error(const std::string & message) { t_error = message; }

int fail(int status, const std::string & message) {
  t_error = message;
  return status;
}

int fail_cuda(cudaError_t e, const char * what) {
  t_error = std::string(what) + " failed: " + cudaGetErrorString(e);
  return Q35B_ERR_CUDA;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

int check_weight_device(const q35b_weight * w) {
  int dev = -1;
  Q35B_CUDA_TRY(cudaGetDevice(&dev), "cudaGetDevice");
  if (w != nullptr && dev != w->device) {
    return fail(Q35B_ERR_ARGUMENT, "NVFP4 weight lives on device " + std::to_string(w->device) + " but the current device is " +
                                     std::to_string(dev) + ".");
  }
  return Q35B_OK;
}

namespace {

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Host-only finishing touches of a new weight: tensor maps, and the library's default status word resolved on this
// device so that no projection call has to do it (possibly under stream capture).
int finish_weight(q35b_weight * w) {
  if (const int st = build_weight_maps(w)) return st;
  unsigned int * word = nullptr;
  return default_status_word(&word);
}

int validate_dims(int n, int k, int shard_index, int shard_count) {
  if (n <= 0 || k <= 0 || (k % 16) != 0) {
    return fail(Q35B_ERR_SHAPE, "Invalid matrix dimensions for NVFP4 weight (cols must be a positive multiple of 16).");
  }
  if (shard_count < 1 || shard_index < 0 || shard_index >= shard_count) {
    return fail(Q35B_ERR_ARGUMENT, "Invalid shard index/count for NVFP4 weight.");
  }
  return Q35B_OK;
}

int alloc_weight(int n, int k, int shard_index, int shard_count, float s2, float input_scale, q35b_weight ** out) {
  int begin = 0, count = 0;
  q35b_shard_range(n, shard_index, shard_count, &begin, &count);
  auto * w = new q35b_weight();
  w->n_total = n;
  w->k = k;
  w->row_begin = begin;
  w->rows = count;
  w->s2 = s2;
  w->input_scale = input_scale;
  if (cudaGetDevice(&w->device) != cudaSuccess) {
    delete w;
    return fail_cuda(cudaGetLastError(), "cudaGetDevice");
  }
  w->codes_bytes = static_cast<size_t>(count) * (k / 2);
  w->scales_bytes = static_cast<size_t>(count) * (k / 16);
  w->scales_tiled_bytes = static_cast<size_t>(round_up_int(std::max(count, 1), 128)) * round_up_int(k / 16, 4);
  const size_t o_scales = align_up(w->codes_bytes, 256);
  const size_t o_tiled = o_scales + align_up(w->scales_bytes, 256);
  const size_t total = o_tiled + align_up(w->scales_tiled_bytes, 256) + 256;  // + one control block
  const cudaError_t e = cudaMalloc(&w->base, total);
  if (e != cudaSuccess) {
    delete w;
    return fail_cuda(e, "cudaMalloc(nvfp4 weight)");
  }
  w->codes = static_cast<uint8_t *>(w->base);
  w->scales = w->codes + o_scales;
  w->scales_tiled = w->codes + o_tiled;
  *out = w;
  return Q35B_OK;
}

}  // namespace
}  // namespace q35b

using namespace q35b;

// Q35B_GEMV_AUTO sends a single projection to the streaming kernel from this many weight bytes on (measured
// crossover on B200: the SIMT launch wins at 13 MB, the streaming kernel at 47 MB).
static constexpr size_t kAutoStreamBytes = 24u << 20;

extern "C" {

const char * q35b_last_error(void) { return t_error.c_str(); }

const char * q35b_version(void) { return "q35b 0.1 (sm_100a)"; }

unsigned long long q35b_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int q35b_shard_range(int n, int shard_index, int shard_count, int * row_begin, int * row_count) {
  if (n <= 0 || shard_count < 1 || shard_index < 0 || shard_index >= shard_count) {
    if (row_begin) *row_begin = 0;
    if (row_count) *row_count = 0;
    return fail(Q35B_ERR_ARGUMENT, "Invalid shard index/count.");
  }
  // 128-row blocks (the scale tile height) dealt out as evenly as possible.
  const long long blocks = (n + 127) / 128;
  const long long b0 = blocks * shard_index / shard_count;
  const long long b1 = blocks * (shard_index + 1) / shard_count;
  const int begin = static_cast<int>(std::min<long long>(b0 * 128, n));
  const int end = static_cast<int>(std::min<long long>(b1 * 128, n));
  if (row_begin) *row_begin = begin;
  if (row_count) *row_count = end - begin;
  return Q35B_OK;
}

int q35b_weight_create(const uint8_t * codes_host, const uint8_t * scales_host, float weight_scale_2, float input_scale,
                       int n, int k, int shard_index, int shard_count, q35b_weight ** out) {
  if (codes_host == nullptr || scales_host == nullptr || out == nullptr) {
    return fail(Q35B_ERR_ARGUMENT, "NVFP4 weight creation received a null buffer.");
  }
  *out = nullptr;
  if (const int st = validate_dims(n, k, shard_index, shard_count)) return st;
  q35b_weight * w = nullptr;
  if (const int st = alloc_weight(n, k, shard_index, shard_count, weight_scale_2, input_scale, &w)) return st;
  const int scale_cols = k / 16;
  const uint8_t * src_codes = codes_host + static_cast<size_t>(w->row_begin) * (k / 2);
  const uint8_t * src_scales = scales_host + static_cast<size_t>(w->row_begin) * scale_cols;
  // Host-side repack of the block scales into 128x4 tiles (zero padded).
  std::vector<uint8_t> tiled(w->scales_tiled_bytes, 0);
  const int padded_cols = round_up_int(scale_cols, 4);
  for (int r = 0; r < w->rows; ++r) {
    for (int c = 0; c < scale_cols; ++c) {
      tiled[static_cast<size_t>(tiled_scale_offset(r, c, padded_cols))] = src_scales[static_cast<size_t>(r) * scale_cols + c];
    }
  }
  for (size_t i = 0; i < w->scales_bytes; ++i) {
    if (src_scales[i] & 0x80u) {
      w->negative_scales = true;
      break;
    }
  }
  cudaError_t e = cudaSuccess;
  if (w->rows > 0) {
    e = cudaMemcpy(w->codes, src_codes, w->codes_bytes, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(w->scales, src_scales, w->scales_bytes, cudaMemcpyHostToDevice);
  }
  if (e == cudaSuccess) e = cudaMemcpy(w->scales_tiled, tiled.data(), tiled.size(), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    q35b_weight_destroy(w);
    return fail_cuda(e, "cudaMemcpy(nvfp4 weight)");
  }
  if (const int st = finish_weight(w)) {
    q35b_weight_destroy(w);
    return st;
  }
  *out = w;
  return Q35B_OK;
}

int q35b_weight_create_from_device(const uint8_t * codes_dev, const uint8_t * scales_dev, float weight_scale_2,
                                   float input_scale, int n, int k, int shard_index, int shard_count,
                                   q35b_stream stream, q35b_weight ** out) {
  if (codes_dev == nullptr || scales_dev == nullptr || out == nullptr) {
    return fail(Q35B_ERR_ARGUMENT, "NVFP4 weight creation received a null buffer.");
  }
  *out = nullptr;
  if (const int st = validate_dims(n, k, shard_index, shard_count)) return st;
  q35b_weight * w = nullptr;
  if (const int st = alloc_weight(n, k, shard_index, shard_count, weight_scale_2, input_scale, &w)) return st;
  auto s = static_cast<cudaStream_t>(stream);
  const int scale_cols = k / 16;
  cudaError_t e = cudaSuccess;
  if (w->rows > 0) {
    e = cudaMemcpyAsync(w->codes, codes_dev + static_cast<size_t>(w->row_begin) * (k / 2), w->codes_bytes,
                        cudaMemcpyDeviceToDevice, s);
    if (e == cudaSuccess) {
      e = cudaMemcpyAsync(w->scales, scales_dev + static_cast<size_t>(w->row_begin) * scale_cols, w->scales_bytes,
                          cudaMemcpyDeviceToDevice, s);
    }
  }
  if (e != cudaSuccess) {
    q35b_weight_destroy(w);
    return fail_cuda(e, "cudaMemcpyAsync(nvfp4 weight)");
  }
  auto * sign_flag = reinterpret_cast<unsigned int *>(w->scales_tiled + align_up(w->scales_tiled_bytes, 256));
  e = cudaMemsetAsync(sign_flag, 0, sizeof(unsigned int), s);
  if (e != cudaSuccess) {
    q35b_weight_destroy(w);
    return fail_cuda(e, "cudaMemsetAsync(nvfp4 weight)");
  }
  if (const int st = launch_tile_scales(w->scales, w->rows, scale_cols, w->scales_tiled, sign_flag, s)) {
    q35b_weight_destroy(w);
    return st;
  }
  unsigned int flag = 0;
  e = cudaMemcpyAsync(&flag, sign_flag, sizeof(flag), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) {
    q35b_weight_destroy(w);
    return fail_cuda(e, "cudaStreamSynchronize(nvfp4 weight)");
  }
  w->negative_scales = flag != 0;
  if (const int st = finish_weight(w)) {
    q35b_weight_destroy(w);
    return st;
  }
  *out = w;
  return Q35B_OK;
}

int q35b_weight_create_gate_up(const uint8_t * gate_codes_host, const uint8_t * gate_scales_host, float gate_weight_scale_2,
                               const uint8_t * up_codes_host, const uint8_t * up_scales_host, float up_weight_scale_2,
                               int n_half, int k, q35b_weight ** out) {
  return q35b_weight_create_gate_up_shard(gate_codes_host, gate_scales_host, gate_weight_scale_2, up_codes_host,
                                          up_scales_host, up_weight_scale_2, n_half, k, 0, 1, out);
}

int q35b_weight_create_gate_up_shard(const uint8_t * gate_codes_host, const uint8_t * gate_scales_host,
                                     float gate_weight_scale_2, const uint8_t * up_codes_host,
                                     const uint8_t * up_scales_host, float up_weight_scale_2, int n_half, int k,
                                     int shard_index, int shard_count, q35b_weight ** out) {
  if (gate_codes_host == nullptr || gate_scales_host == nullptr || up_codes_host == nullptr || up_scales_host == nullptr ||
      out == nullptr) {
    return fail(Q35B_ERR_ARGUMENT, "NVFP4 weight creation received a null buffer.");
  }
  *out = nullptr;
  if (n_half <= 0 || (n_half % 8) != 0) return fail(Q35B_ERR_SHAPE, "A gate/up weight needs a row count that is a multiple of 8.");
  if (const int st = validate_dims(2 * n_half, k, shard_index, shard_count)) return st;
  // rows alternate in groups of eight: 8 gate rows, 8 up rows, ...
  const size_t code_row = static_cast<size_t>(k) / 2, scale_row = static_cast<size_t>(k) / 16;
  std::vector<uint8_t> codes(2 * static_cast<size_t>(n_half) * code_row), scales(2 * static_cast<size_t>(n_half) * scale_row);
  for (int grp = 0; grp < n_half / 8; ++grp) {
    std::memcpy(&codes[(2 * grp) * 8 * code_row], gate_codes_host + static_cast<size_t>(grp) * 8 * code_row, 8 * code_row);
    std::memcpy(&codes[(2 * grp + 1) * 8 * code_row], up_codes_host + static_cast<size_t>(grp) * 8 * code_row, 8 * code_row);
    std::memcpy(&scales[(2 * grp) * 8 * scale_row], gate_scales_host + static_cast<size_t>(grp) * 8 * scale_row, 8 * scale_row);
    std::memcpy(&scales[(2 * grp + 1) * 8 * scale_row], up_scales_host + static_cast<size_t>(grp) * 8 * scale_row, 8 * scale_row);
  }
  q35b_weight * w = nullptr;
  if (const int st = q35b_weight_create(codes.data(), scales.data(), gate_weight_scale_2, 1.0f, 2 * n_half, k, shard_index,
                                        shard_count, &w)) {
    return st;
  }
  w->gate_up = true;
  w->s2_up = up_weight_scale_2;
  *out = w;
  return Q35B_OK;
}

int q35b_weight_is_gate_up(const q35b_weight * w) { return (w != nullptr && w->gate_up) ? 1 : 0; }

int q35b_weight_dequant_bf16(const q35b_weight * w, void * w_bf16, q35b_stream stream) {
  return launch_dequant_bf16(w, w_bf16, static_cast<cudaStream_t>(stream));
}

void q35b_weight_destroy(q35b_weight * w) {
  if (w == nullptr) return;
  for (auto *& b : w->stream_batch) {
    gemv_batch_free(b);
    b = nullptr;
  }
  if (w->base != nullptr) cudaFree(w->base);
  delete w;
}

int q35b_weight_row_begin(const q35b_weight * w) { return w ? w->row_begin : 0; }
int q35b_weight_rows(const q35b_weight * w) { return w ? w->rows : 0; }
int q35b_weight_cols(const q35b_weight * w) { return w ? w->k : 0; }
size_t q35b_weight_stream_bytes(const q35b_weight * w) { return w ? w->codes_bytes + w->scales_bytes : 0; }

int q35b_gemv_w4a16_bf16(const q35b_weight * w, const void * x_bf16, int m, void * y_bf16, int kernel,
                         q35b_stream stream) {
  if (kernel == Q35B_GEMV_AUTO && w != nullptr && m >= 1 && m <= 8 && !w->gate_up &&
      w->codes_bytes + w->scales_bytes >= kAutoStreamBytes && x_bf16 != nullptr &&
      (reinterpret_cast<uintptr_t>(x_bf16) & 15u) == 0 && gemv_stream_eligible(w, m)) {
    // A weight this large keeps the persistent streaming kernel busy for longer than its set-up costs; below the
    // threshold the plain SIMT launch finishes first.  The streaming kernel's first use allocates its work list,
    // which a capturing stream must not do: stay on the SIMT kernel then.
    bool can_stream = w->stream_batch[m] != nullptr;
    if (!can_stream) {
      cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
      can_stream = cudaStreamIsCapturing(static_cast<cudaStream_t>(stream), &cs) == cudaSuccess && cs == cudaStreamCaptureStatusNone;
    }
    if (can_stream) kernel = Q35B_GEMV_STREAM;
  }
  if (kernel == Q35B_GEMV_STREAM) {
    if (w == nullptr || x_bf16 == nullptr || y_bf16 == nullptr) {
      return fail(Q35B_ERR_ARGUMENT, "NVFP4 projection received a null buffer.");
    }
    if (m < 1 || m > 8) return fail(Q35B_ERR_SHAPE, "NVFP4 decode projection supports 1..8 tokens.");
    if (w->rows == 0) return Q35B_OK;
    if (w->gate_up) return fail(Q35B_ERR_ARGUMENT, "A gate/up weight runs through the projection work list (q35b_gemv_batch_*).");
    if ((reinterpret_cast<uintptr_t>(x_bf16) & 15u) != 0) {
      return fail(Q35B_ERR_ARGUMENT, "Activations of the streaming NVFP4 projection must be 16-byte aligned.");
    }
    if (const int st = check_weight_device(w)) return st;
    auto * wm = const_cast<q35b_weight *>(w);
    q35b_gemv_batch * batch = nullptr;
    {
      std::lock_guard<std::mutex> lock(wm->batch_mutex);
      if (wm->stream_batch[m] == nullptr) {
        // first use with this token count: build (and upload) the single-projection work list
        q35b_gemv_item item{w, nullptr, nullptr, nullptr, 0};
        if (const int st = gemv_batch_build(&item, 1, m, &wm->stream_batch[m])) return st;
      }
      batch = wm->stream_batch[m];
    }
    return gemv_batch_launch(batch, x_bf16, y_bf16, static_cast<cudaStream_t>(stream));
  }
  return launch_gemv_bf16(w, x_bf16, m, y_bf16, kernel, static_cast<cudaStream_t>(stream));
}

size_t q35b_gemv_item_bytes(void) { return sizeof(q35b_gemv_item); }

int q35b_gemv_batch_create(const q35b_gemv_item * items, int count, int m, q35b_gemv_batch ** out) {
  return gemv_batch_build(items, count, m, out);
}

int q35b_gemv_batch_create_tensor(const q35b_gemv_item * items, int count, int m, int digits, q35b_gemv_batch ** out) {
  return gemv_batch_build_tensor(items, count, m, digits, out);
}

int q35b_gemv_batch_run(const q35b_gemv_batch * batch, q35b_stream stream) {
  return gemv_batch_launch(batch, nullptr, nullptr, static_cast<cudaStream_t>(stream));
}

void q35b_gemv_batch_destroy(q35b_gemv_batch * batch) { gemv_batch_free(batch); }

int q35b_gemv_batch_status(const q35b_gemv_batch * batch, unsigned int * status_out) {
  return gemv_batch_read_status(batch, status_out);
}

int q35b_debug_gemv_plan(int m, int max_k, int * ctas_per_sm, int * ring_stages, int * activation_buffers, int * smem_bytes) {
  return q35b::gemv_plan_debug(m, max_k, ctas_per_sm, ring_stages, activation_buffers, smem_bytes);
}

int q35b_debug_gemv_batch_wait(q35b_gemv_batch * batch, unsigned int wait_limit_polls, unsigned int extra_completions) {
  return gemv_batch_debug_wait(batch, wait_limit_polls, extra_completions);
}

size_t q35b_gemv_batch_stream_bytes(const q35b_gemv_batch * batch) { return gemv_batch_bytes(batch); }

int q35b_gemv_w4a16_f32(const q35b_weight * w, const float * x_f32, float input_scale, float * y_f32, int kernel,
                        q35b_stream stream) {
  return launch_gemv_f32(w, x_f32, input_scale, y_f32, kernel, static_cast<cudaStream_t>(stream));
}

size_t q35b_act_codes_bytes(int m, int k) { return (m > 0 && k > 0) ? static_cast<size_t>(m) * (k / 2) : 0; }

size_t q35b_act_scales_bytes(int m, int k) {
  return (m > 0 && k > 0) ? static_cast<size_t>(round_up_int(m, 128)) * round_up_int(k / 16, 4) : 0;
}

size_t q35b_quant_workspace_bytes(void) { return 256; }

int q35b_quantize_nvfp4_bf16(const void * x_bf16, int m, int k, float global_scale, uint8_t * codes,
                             uint8_t * scales_tiled, float * input_scale_dev, void * workspace, q35b_stream stream) {
  return launch_quantize_bf16(x_bf16, m, k, global_scale, codes, scales_tiled, input_scale_dev, workspace,
                              static_cast<cudaStream_t>(stream));
}

int q35b_quantize_nvfp4_f32(const float * x_f32, int m, int k, float global_scale, uint8_t * codes, uint8_t * scales_tiled,
                            float * input_scale_dev, void * workspace, q35b_stream stream) {
  return launch_quantize_f32(x_f32, m, k, global_scale, codes, scales_tiled, input_scale_dev, workspace,
                             static_cast<cudaStream_t>(stream));
}

int q35b_quantize_nvfp4_bf16_reference_recipe(const void * x_bf16, int m, int k, int swap_nibbles, uint8_t * codes,
                                              uint8_t * scales_tiled, q35b_stream stream) {
  return launch_quantize_reference_recipe(x_bf16, m, k, swap_nibbles, codes, scales_tiled,
                                          static_cast<cudaStream_t>(stream));
}

int q35b_quantize_weight_f32(const float * w_f32, int n, int k, uint8_t * codes, uint8_t * scales, float * s2_dev,
                             void * workspace, q35b_stream stream) {
  return launch_quantize_weight_f32(w_f32, n, k, codes, scales, s2_dev, workspace, static_cast<cudaStream_t>(stream));
}

int q35b_gemm_w4a4_bf16(const q35b_weight * w, const uint8_t * a_codes, const uint8_t * a_scales_tiled,
                        const float * input_scale_dev, int m, void * c_bf16, int ldc, unsigned int * status_dev,
                        q35b_stream stream) {
  return launch_gemm_w4a4(w, a_codes, a_scales_tiled, input_scale_dev, m, c_bf16, ldc, nullptr, 0,
                          status_dev, static_cast<cudaStream_t>(stream));
}

int q35b_gemm_w4a4_gate_up_nvfp4(const q35b_weight * w, const uint8_t * a_codes, const uint8_t * a_scales_tiled,
                                 const float * input_scale_dev, int m, uint8_t * out_codes, uint8_t * out_scales_tiled,
                                 const float * out_scale_dev, unsigned int * status_dev, q35b_stream stream) {
  const GemmQuantOut q{out_codes, out_scales_tiled, out_scale_dev, w != nullptr ? w->n_total / 2 : 0};
  return launch_gemm_w4a4(w, a_codes, a_scales_tiled, input_scale_dev, m, nullptr, 0, nullptr, 0,
                          status_dev, static_cast<cudaStream_t>(stream), &q);
}

int q35b_gemm_w4a4_bf16_residual(const q35b_weight * w, const uint8_t * a_codes, const uint8_t * a_scales_tiled,
                                 const float * input_scale_dev, int m, const void * residual_bf16, int ldr, void * c_bf16,
                                 int ldc, unsigned int * status_dev, q35b_stream stream) {
  if (residual_bf16 == nullptr) return fail(Q35B_ERR_ARGUMENT, "NVFP4 prefill projection received a null residual.");
  return launch_gemm_w4a4(w, a_codes, a_scales_tiled, input_scale_dev, m, c_bf16, ldc,
                          residual_bf16, ldr, status_dev, static_cast<cudaStream_t>(stream));
}

/* Host-callable twins of the device encoders/decoders, so that their
 * equivalence with the reference's scan can be tested without a GPU. */
uint8_t q35b_debug_encode_ue4m3(float v) { return encode_ue4m3(v); }
uint8_t q35b_debug_encode_e2m1(float v) { return encode_e2m1(v); }
float q35b_debug_decode_e4m3(uint8_t b) { return decode_e4m3(b); }
float q35b_debug_decode_e2m1(uint8_t c) { return decode_e2m1(c); }
long long q35b_debug_tiled_scale_offset(int row, int col, int padded_cols) {
  return tiled_scale_offset(row, col, padded_cols);
}

}  // extern "C"
