// Internal declarations shared by the translation units of libq35b.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <mutex>
#include <string>

#include "../../include/q35b_nvfp4.h"

namespace q35b {

// Thread-local message behind q35b_last_error().
void set_error(const std::string & message);
int fail(int status, const std::string & message);
int fail_cuda(cudaError_t e, const char * what);

#define Q35B_CUDA_TRY(call, what)                                 \
  do {                                                            \
    const cudaError_t q35b_e_ = (call);                           \
    if (q35b_e_ != cudaSuccess) return ::q35b::fail_cuda(q35b_e_, what); \
  } while (0)

extern std::atomic<unsigned long long> g_launches;
inline void count_launch(unsigned n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int sm_count();

// Launch with programmatic stream serialisation: the grid may be scheduled while the previous kernel of the stream is
// still finishing.  Every kernel launched this way executes griddepcontrol.wait before its first access to global
// memory, which returns only when everything earlier in the stream is complete and visible, so what overlaps is
// launch latency and the prologue (barrier set-up, TMEM allocation), never data.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args &&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Q35B_OK when the weight lives on the calling thread's current device, else Q35B_ERR_ARGUMENT: every launch goes
// to the current device, and a weight of another GPU would be read through a pointer that device cannot reach.
int check_weight_device(const struct ::q35b_weight * w);

}  // namespace q35b

// One projection weight on the device.  All three arrays live in a single
// allocation; codes and both scale layouts are 256-byte aligned.
struct q35b_weight {
  int n_total = 0;    // rows of the whole tensor
  int k = 0;          // columns
  int row_begin = 0;  // first global row of this shard
  int rows = 0;       // rows held
  float s2 = 1.0f;    // weight_scale_2
  float s2_up = 1.0f; // weight_scale_2 of the up half of a gate/up weight
  bool gate_up = false;  // rows alternate 8 gate / 8 up
  float input_scale = 1.0f;
  int device = 0;
  void * base = nullptr;            // the allocation
  uint8_t * codes = nullptr;        // [rows, k/2], checkpoint order (K-major: also the UMMA B operand)
  uint8_t * scales = nullptr;       // [rows, k/16] row-major (decode kernels)
  uint8_t * scales_tiled = nullptr; // [ceil128(rows), ceil4(k/16)] 128x4 tiles (UMMA scale factors)
  size_t codes_bytes = 0, scales_bytes = 0, scales_tiled_bytes = 0;
  bool negative_scales = false;      // some block scale has its sign bit set (only the SIMT decode kernel takes those)
  // Single-projection work lists of the streaming decode kernel, by token count: built on first use under
  // batch_mutex (the only state of a weight that changes after q35b_weight_create*).
  struct q35b_gemv_batch * stream_batch[9] = {nullptr};
  std::mutex batch_mutex;
  // Tensor maps of the GEMMs, encoded once at creation (build_weight_maps): B tiles of the 1-CTA kernel in its two
  // widths, and the 2-CTA kernel's 96-row code boxes and 4-chunk scale boxes.
  bool has_maps = false;
  alignas(64) CUtensorMap tmap_codes_128;
  alignas(64) CUtensorMap tmap_codes_256;
  alignas(64) CUtensorMap tmap2_codes;
  alignas(64) CUtensorMap tmap2_sf;
};

namespace q35b {

// gemv_w4a16.cu
int launch_dequant_bf16(const q35b_weight * w, void * w_bf16, cudaStream_t s);
int launch_gemv_bf16(const q35b_weight * w, const void * x_bf16, int m, void * y_bf16, int kernel, cudaStream_t s);
int launch_gemv_f32(const q35b_weight * w, const float * x, float input_scale, float * y, int kernel, cudaStream_t s);

// act_quant.cu
int launch_quantize_bf16(const void * x, int m, int k, float global_scale, uint8_t * codes, uint8_t * scales_tiled,
                         float * g_dev, void * workspace, cudaStream_t s);
int launch_quantize_f32(const float * x, int m, int k, float global_scale, uint8_t * codes, uint8_t * scales_tiled,
                        float * g_dev, void * workspace, cudaStream_t s);
int launch_quantize_reference_recipe(const void * x, int m, int k, int swap, uint8_t * codes, uint8_t * scales_tiled,
                                     cudaStream_t s);
int launch_quantize_weight_f32(const float * w, int n, int k, uint8_t * codes, uint8_t * scales_rowmajor,
                               float * s2_dev, void * workspace, cudaStream_t s);
int launch_tile_scales(const uint8_t * scales_rowmajor, int rows, int scale_cols, uint8_t * tiled,
                       unsigned int * sign_flag, cudaStream_t s);

// gemv_stream.cu
bool gemv_stream_eligible(const q35b_weight * w, int m);
int gemv_batch_build(const q35b_gemv_item * items, int count, int m, struct q35b_gemv_batch ** out);
int gemv_batch_build_tensor(const q35b_gemv_item * items, int count, int m, int digits, struct q35b_gemv_batch ** out);
int gemv_batch_launch(const struct q35b_gemv_batch * b, const void * x_override, void * y_override, cudaStream_t s);
void gemv_batch_free(struct q35b_gemv_batch * b);
int gemv_batch_read_status(const struct q35b_gemv_batch * b, unsigned int * out);
size_t gemv_batch_bytes(const struct q35b_gemv_batch * b);
int gemv_plan_debug(int m, int max_k, int * ctas_per_sm, int * ring_stages, int * activation_buffers, int * smem_bytes);
int gemv_batch_debug_wait(struct q35b_gemv_batch * b, unsigned int wait_limit, unsigned int extra_completions);

// gemm_w4a4_tcgen05.cu
int make_code_map(CUtensorMap * map, const void * base, int rows, int k_bytes, int box_rows);
// Where a gate/up GEMM writes silu(gate) * up as an NVFP4 activation instead of BF16 (see gemm_epilogue.cuh).
struct GemmQuantOut {
  uint8_t * codes;          // [m, total_cols / 2] bytes: the whole activation, of which this weight writes its columns
  uint8_t * scales_tiled;   // tiled block scales of the [m, total_cols] activation
  const float * g_dev;      // its per-tensor scale, known in advance
  int total_cols;           // width of the whole activation (= rows / 2 for an unsharded gate/up weight)
};
// Where a gathering GEMM repeats its stores on the other ranks and signals completion (see gemm_epilogue.cuh,
// peer_gather.cu).  Pointers are this process's mappings of the other ranks' buffers, already moved to the shard's
// first column.
struct GemmGather {
  int n_peers = 0;
  void * peer_c[7] = {};
  unsigned int * peer_flag[7] = {};
  unsigned int * done_counter = nullptr;
  unsigned int epoch = 0;
  unsigned int * send_seq = nullptr;   // used when epoch == 0 (see GemmEpilogue)
};
// Encodes the weight's tensor maps (host only, no device work); called by q35b_weight_create*.
int build_weight_maps(q35b_weight * w);
// The library's own status word of the current device (a file-scope device variable): what the GEMM entry points
// use when the caller passes no status word.  Resolved once per device; q35b_weight_create* calls it so that the
// first projection does not have to.
int default_status_word(unsigned int ** out);
int launch_gemm_w4a4(const q35b_weight * w, const uint8_t * a_codes, const uint8_t * a_scales_tiled, const float * g_dev,
                     int m, void * c_bf16, int ldc, const void * residual_bf16, int ldr, unsigned int * status_dev,
                     cudaStream_t s, const GemmQuantOut * qout = nullptr, const GemmGather * gather = nullptr);


// gemm_wstream.cu: weight-streaming projection for 1..128 operand rows (small-M prefill, tensor-core decode)
bool gemm_wstream_eligible(const q35b_weight * w, int m);
int launch_gemm_wstream(const q35b_weight * w, const uint8_t * a_codes, const uint8_t * a_scales_tiled, const float * g_dev,
                        int m, void * c_bf16, int ldc, const void * residual_bf16, int ldr, unsigned int * status_dev,
                        cudaStream_t s);

struct WBatch;  // decode work list on the tensor path (digit-expanded activations)
int wbatch_build(const q35b_gemv_item * items, int count, int m, int digits, WBatch ** out);
int wbatch_launch(const WBatch * b, cudaStream_t s);
void wbatch_free(WBatch * b);
int wbatch_status(const WBatch * b, unsigned int * out);
size_t wbatch_bytes(const WBatch * b);

// gemm_w4a4_2cta.cu
bool gemm_2cta_eligible(const q35b_weight * w, int m);
struct GemmEpilogue;
int make_sf_map(CUtensorMap * map, const void * base, long long chunks);
int launch_gemm_w4a4_2cta(const q35b_weight * w, const uint8_t * a_codes, const uint8_t * a_scales_tiled, const float * g_dev,
                          int m, void * c_bf16, int ldc, const GemmEpilogue & ep, unsigned int * status_dev,
                          cudaStream_t s);

}  // namespace q35b
