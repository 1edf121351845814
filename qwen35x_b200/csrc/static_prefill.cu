// Prefill projection for callers that cannot allocate device memory.
//
// q35b_project_prefill_bf16 needs scratch beyond its input and output: the
// quantised activation (E2M1 codes, tiled E4M3 scales), the per-tensor scale
// word, the quantiser's reduction workspace and a status word.  Normally the
// caller allocates those.  Some hosts cannot: a runtime that carved the whole
// device into its own arena at start-up and has no spare block of the right
// size, a plug-in that runs inside a stream-ordered region where cudaMalloc
// would synchronise the device, or a process whose memory budget is fixed by
// its launcher.  For them the scratch lives here, in one file-scope device
// array that every GPU loading this library holds until the process exits.
#include "engine.h"
#include "nvfp4_codec.cuh"

#include <mutex>

namespace q35b {
namespace {

// Capacity of the built-in scratch: enough for the largest prefill chunk the
// reference runs (4096 tokens x 9216 columns): 18 MiB of codes + 2.25 MiB of
// scales, plus one 256-byte control block.
constexpr size_t kControlBytes = 256;
constexpr size_t kStaticScratchBytes = static_cast<size_t>(24) << 20;

static __device__ __align__(256) unsigned char g_prefill_scratch[kStaticScratchBytes];

// Device address of g_prefill_scratch on each device, resolved on first use.
// (In host code the symbol's own name is only a handle for the runtime, not a
// device address: it must go through cudaGetSymbolAddress.)
std::mutex g_mutex;
unsigned char * g_scratch_ptr[64] = {nullptr};

int scratch_for_current_device(unsigned char ** out) {
  int dev = 0;
  Q35B_CUDA_TRY(cudaGetDevice(&dev), "cudaGetDevice");
  if (dev < 0 || dev >= 64) return fail(Q35B_ERR_ARGUMENT, "Device ordinal out of range for the built-in prefill scratch.");
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void * p = nullptr;
    Q35B_CUDA_TRY(cudaGetSymbolAddress(&p, g_prefill_scratch), "cudaGetSymbolAddress(prefill scratch)");
    g_scratch_ptr[dev] = static_cast<unsigned char *>(p);
  }
  *out = g_scratch_ptr[dev];
  return Q35B_OK;
}

}  // namespace
}  // namespace q35b

using namespace q35b;

extern "C" {

size_t q35b_static_prefill_capacity_bytes(void) { return kStaticScratchBytes - kControlBytes; }

int q35b_project_prefill_bf16_static(const q35b_weight * w, const void * x_bf16, int m, float global_scale,
                                     void * c_bf16, int ldc, q35b_stream stream) {
  if (w == nullptr || x_bf16 == nullptr || c_bf16 == nullptr) {
    return fail(Q35B_ERR_ARGUMENT, "NVFP4 prefill projection received a null device buffer.");
  }
  if (m <= 0) return fail(Q35B_ERR_SHAPE, "Invalid dimensions for NVFP4 prefill projection.");
  const size_t codes_bytes = (q35b_act_codes_bytes(m, w->k) + 255) / 256 * 256;
  const size_t scales_bytes = q35b_act_scales_bytes(m, w->k);
  if (codes_bytes + scales_bytes > kStaticScratchBytes - kControlBytes) {
    return fail(Q35B_ERR_SHAPE,
                "Activation of " + std::to_string(m) + " x " + std::to_string(w->k) + " needs " +
                  std::to_string(codes_bytes + scales_bytes) + " bytes of scratch; the built-in scratch holds " +
                  std::to_string(kStaticScratchBytes - kControlBytes) +
                  ". Split the tokens into smaller chunks or use q35b_quantize_nvfp4_bf16 + q35b_gemm_w4a4_bf16 with "
                  "caller-owned scratch.");
  }
  if (const int st = check_weight_device(w)) return st;
  unsigned char * base = nullptr;
  if (const int st = scratch_for_current_device(&base)) return st;
  auto s = static_cast<cudaStream_t>(stream);
  // Control block: [0,8) quantiser workspace, [16,20) per-tensor scale, [32,36) GEMM status.  The array keeps
  // whatever the previous call left, so everything that must start at zero is cleared here.
  Q35B_CUDA_TRY(cudaMemsetAsync(base, 0, kControlBytes, s), "cudaMemsetAsync(prefill scratch control block)");
  auto * workspace = base;
  auto * g_dev = reinterpret_cast<float *>(base + 16);
  auto * status = reinterpret_cast<unsigned int *>(base + 32);
  uint8_t * codes = base + kControlBytes;
  uint8_t * scales = codes + codes_bytes;
  if (const int st = launch_quantize_bf16(x_bf16, m, w->k, global_scale, codes, scales, g_dev, workspace, s)) return st;
  return launch_gemm_w4a4(w, codes, scales, g_dev, m, c_bf16, ldc, nullptr, 0, status, s);
}

int q35b_static_prefill_status(unsigned int * status_out) {
  if (status_out == nullptr) return fail(Q35B_ERR_ARGUMENT, "Null status pointer.");
  unsigned char * base = nullptr;
  if (const int st = scratch_for_current_device(&base)) return st;
  Q35B_CUDA_TRY(cudaMemcpy(status_out, base + 32, sizeof(unsigned int), cudaMemcpyDeviceToHost), "cudaMemcpy(prefill scratch status)");
  return Q35B_OK;
}

}  // extern "C"
