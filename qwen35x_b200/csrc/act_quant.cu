// NVFP4 quantisation on the GPU: BF16 (activations) or fp32 (weights) ->
// E2M1 codes, E4M3 block scales, fp32 per-tensor scale.
//
// Replaces nvfp4_quantize_{single_row,matrix,bf16_matrix}_for_cublaslt_kernel
// (src/runtime/cuda_bench.cu:98-213) and the cudaMemset pair that precedes
// them in every bridge (:2621-2624): padding scale bytes are written here.
//
// Recipe (bit-exact contract, all fp32, IEEE division, no fused contraction
// that could change a rounding):
//   g  = amax(X) / (6 * 448)   (1 if the tensor is all zero), or a given g
//   per 16-block: t  = amax_blk / 6
//                 sb = min(UE4M3(max(t / g, 1e-8)), 0x7e)
//                 d  = max(decode(sb), 1e-8) * g
//                 code_i = E2M1(x_i / d), element 2j in the low nibble
// UE4M3()/E2M1() are the reference's nearest-with-ties-down encoders
// (src/runtime/cuda_bench.cu:58-96).  0x7f is never emitted because the
// tensor-core UE4M3 format reads it as NaN.
//
// HBM traffic per [M,K] BF16 call: 2*M*K read by the amax pass, 2*M*K read
// again (L2-resident for prefill sizes) + M*K/2 + M*K/16 written by the
// quantise pass.
#include <cuda_bf16.h>

#include "engine.h"
#include "nvfp4_codec.cuh"
#include "nvfp4_quant_block.cuh"

namespace q35b {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float abs_max8(const uint4 q) {
  // 8 bf16 values: |v| as fp32 bit patterns compare like unsigned integers.
  const uint32_t r[4] = {q.x, q.y, q.z, q.w};
  uint32_t m = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t lo = (r[j] << 16) & 0x7fffffffu;
    const uint32_t hi = r[j] & 0x7fff0000u;
    // NaN payloads are skipped like fmaxf does.
    if (lo <= 0x7f800000u) m = max(m, lo);
    if (hi <= 0x7f800000u) m = max(m, hi);
  }
  return __uint_as_float(m);
}

// Pass 1: per-tensor amax -> g.  ws[0] holds the running maximum (fp32 bits),
// ws[1] counts finished blocks; the last block publishes g and leaves both
// words zero for the next call.
template <typename T>
__global__ void __launch_bounds__(kThreads)
amax_to_global_scale_kernel(const T * __restrict__ x, size_t n, unsigned int * __restrict__ ws,
                            float * __restrict__ g_out) {
  // no early griddepcontrol.launch_dependents here: a dependent grid that became resident early would take the
  // registers this kernel's remaining blocks need; the implicit trigger at block exit overlaps the tail only
  asm volatile("griddepcontrol.wait;" ::: "memory");  // x may come from the kernel before
  float local = 0.0f;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  if constexpr (sizeof(T) == 2) {
    const uint4 * v = reinterpret_cast<const uint4 *>(x);
    const size_t nv = n >> 3;
    size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    // four independent 16-byte loads in flight per thread
    for (; i + 3 * stride < nv; i += 4 * stride) {
      const uint4 a = __ldg(v + i), b = __ldg(v + i + stride), c = __ldg(v + i + 2 * stride), d = __ldg(v + i + 3 * stride);
      local = fmaxf(fmaxf(local, fmaxf(abs_max8(a), abs_max8(b))), fmaxf(abs_max8(c), abs_max8(d)));
    }
    for (; i < nv; i += stride) local = fmaxf(local, abs_max8(__ldg(v + i)));
  } else {
    const float4 * v = reinterpret_cast<const float4 *>(x);
    const size_t nv = n >> 2;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nv; i += stride) {
      const float4 q = __ldg(v + i);
      local = fmaxf(local, fmaxf(fmaxf(fabsf(q.x), fabsf(q.y)), fmaxf(fabsf(q.z), fabsf(q.w))));
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) local = fmaxf(local, __shfl_xor_sync(0xffffffffu, local, off));
  __shared__ float red[kThreads / 32];
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = local;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = red[0];
#pragma unroll
    for (int i = 1; i < kThreads / 32; ++i) m = fmaxf(m, red[i]);
    atomicMax(ws, __float_as_uint(m));
    __threadfence();
    const unsigned int ticket = atomicAdd(ws + 1, 1u);
    if (ticket == gridDim.x - 1) {
      __threadfence();
      const float amax = __uint_as_float(atomicExch(ws, 0u));
      *g_out = (amax > 0.0f) ? __fdiv_rn(amax, 6.0f * 448.0f) : 1.0f;
      ws[1] = 0u;
    }
  }
}

template <typename T>
__device__ __forceinline__ void load16(const T * p, float (&v)[16]);

template <>
__device__ __forceinline__ void load16<__nv_bfloat16>(const __nv_bfloat16 * p, float (&v)[16]) {
  const uint4 * q = reinterpret_cast<const uint4 *>(p);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const uint4 a = __ldg(q + i);
    const uint32_t r[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[i * 8 + j * 2] = __uint_as_float(r[j] << 16);
      v[i * 8 + j * 2 + 1] = __uint_as_float(r[j] & 0xffff0000u);
    }
  }
}

template <>
__device__ __forceinline__ void load16<float>(const float * p, float (&v)[16]) {
  const float4 * q = reinterpret_cast<const float4 *>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 a = __ldg(q + i);
    v[i * 4] = a.x;
    v[i * 4 + 1] = a.y;
    v[i * 4 + 2] = a.z;
    v[i * 4 + 3] = a.w;
  }
}

// Pass 2: one thread per 16-element block, so a warp reads 1 KB of contiguous activations and writes 256 bytes of
// contiguous codes; the four scale bytes of a 64-element group are gathered into lane 0 of each quad with
// shuffles and stored as one 32-bit word of the tiled layout (or four bytes of the row-major layout).
// The grid covers roundup(K/16, 4) block slots per row and rows_padded rows: slots past K and rows past `rows`
// only produce zero scale bytes (TILED layout).
template <typename T, int RECIPE, bool TILED>
__global__ void __launch_bounds__(kThreads, 6)  // 39 registers, six CTAs per SM: measured 4-5 % faster than five CTAs of 45
quantize_nvfp4_kernel(const T * __restrict__ x, int rows, int rows_padded, int k, const float * __restrict__ g_dev,
                      float g_fixed, float * __restrict__ g_out, int swap, uint8_t * __restrict__ codes,
                      uint8_t * __restrict__ scales) {
  asm volatile("griddepcontrol.wait;" ::: "memory");  // the per-tensor scale, and x itself, may come from the kernel before
  const int scale_cols = k >> 4;
  const int slots = ((scale_cols + 3) >> 2) << 2;  // block slots per row, a multiple of 4
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t total = static_cast<size_t>(rows_padded) * slots;
  // whole quads run or exit together (slots % 4 == 0 and kThreads % 4 == 0), so the shuffles below are safe
  const bool live = idx < total;
  const int row = live ? static_cast<int>(idx / slots) : 0;
  const int b = live ? static_cast<int>(idx % slots) : 0;
  float g = 1.0f;
  if (RECIPE == kEngine) {
    // one load of the per-tensor scale per CTA, handed round in shared memory: every warp of a large grid loading
    // the same word would queue up on one L2 slice (measured: the kernel took 1.7x as long)
    __shared__ float g_shared;
    if (threadIdx.x == 0) g_shared = (g_dev != nullptr) ? __ldcg(g_dev) : g_fixed;
    __syncthreads();
    g = g_shared;
    if (g_out != nullptr && idx == 0) *g_out = g;
  }
  uint32_t sb = 0;
  if (live && row < rows && b < scale_cols) {
    float v[16];
    load16<T>(x + static_cast<size_t>(row) * k + static_cast<size_t>(b) * 16, v);
    uint2 packed;
    sb = quantize_block<RECIPE>(v, g, swap != 0, packed);
    *reinterpret_cast<uint2 *>(codes + (static_cast<size_t>(row) * k + static_cast<size_t>(b) * 16) / 2) = packed;
  }
  // gather the quad's four scale bytes
  const int lane = threadIdx.x & 31;
  uint32_t word = sb;
  word |= __shfl_sync(0xffffffffu, sb, (lane & ~3) + 1) << 8;
  word |= __shfl_sync(0xffffffffu, sb, (lane & ~3) + 2) << 16;
  word |= __shfl_sync(0xffffffffu, sb, (lane & ~3) + 3) << 24;
  if (!live || (lane & 3) != 0) return;
  if (TILED) {
    *reinterpret_cast<uint32_t *>(scales + tiled_scale_offset(row, b, slots)) = word;
  } else if (row < rows) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (b + j < scale_cols) scales[static_cast<size_t>(row) * scale_cols + b + j] = static_cast<uint8_t>(word >> (8 * j));
    }
  }
}

__global__ void __launch_bounds__(kThreads)
tile_scales_kernel(const uint8_t * __restrict__ src, int rows, int rows_padded, int scale_cols,
                   uint8_t * __restrict__ tiled, unsigned int * __restrict__ sign_flag) {
  const int groups = (scale_cols + 3) >> 2;
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<size_t>(rows_padded) * groups) return;
  const int row = static_cast<int>(idx / groups);
  const int grp = static_cast<int>(idx % groups);
  uint32_t sbytes = 0;
  if (row < rows) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int b = grp * 4 + j;
      if (b < scale_cols) sbytes |= static_cast<uint32_t>(src[static_cast<size_t>(row) * scale_cols + b]) << (8 * j);
    }
  }
  *reinterpret_cast<uint32_t *>(tiled + tiled_scale_offset(row, grp * 4, groups * 4)) = sbytes;
  if (sign_flag != nullptr && (sbytes & 0x80808080u) != 0u) atomicOr(sign_flag, 1u);
}

int check_quant_args(const void * x, int m, int k, const void * codes, const void * scales) {
  if (x == nullptr || codes == nullptr || scales == nullptr) {
    return fail(Q35B_ERR_ARGUMENT, "NVFP4 quantisation received a null buffer.");
  }
  if (m <= 0 || k <= 0 || (k % 16) != 0) return fail(Q35B_ERR_SHAPE, "Invalid dimensions for NVFP4 quantisation.");
  if ((reinterpret_cast<uintptr_t>(x) & 15u) != 0 || (reinterpret_cast<uintptr_t>(codes) & 7u) != 0 ||
      (reinterpret_cast<uintptr_t>(scales) & 3u) != 0) {
    return fail(Q35B_ERR_ARGUMENT, "NVFP4 quantisation buffers must be 16-byte aligned.");
  }
  return Q35B_OK;
}

template <typename T>
int launch_amax(const T * x, size_t n, unsigned int * ws, float * g_out, cudaStream_t s) {
  // few blocks (every one ends with two atomics on the same pair of words), each with plenty of loads in flight
  const size_t per_block = static_cast<size_t>(kThreads) * 8 * 4;
  int blocks = static_cast<int>(std::min<size_t>((n + per_block - 1) / per_block, static_cast<size_t>(sm_count()) * 4));
  if (blocks < 1) blocks = 1;
  const cudaError_t le = launch_pdl(amax_to_global_scale_kernel<T>, dim3(blocks), dim3(kThreads), 0, s, x, n, ws, g_out);
  count_launch();
  Q35B_CUDA_TRY(le, "amax_to_global_scale_kernel launch");
  return Q35B_OK;
}

}  // namespace

namespace {

template <typename T>
int launch_quantize_activations(const T * x, int m, int k, float global_scale, uint8_t * codes, uint8_t * scales_tiled,
                                float * g_dev, void * workspace, cudaStream_t s) {
  if (const int st = check_quant_args(x, m, k, codes, scales_tiled)) return st;
  if (g_dev == nullptr) return fail(Q35B_ERR_ARGUMENT, "NVFP4 quantisation needs a device word for the input scale.");
  const bool dynamic = !(global_scale > 0.0f);
  if (dynamic) {
    if (workspace == nullptr) return fail(Q35B_ERR_ARGUMENT, "Dynamic NVFP4 quantisation needs its workspace.");
    if (const int st = launch_amax(x, static_cast<size_t>(m) * k, static_cast<unsigned int *>(workspace), g_dev, s)) return st;
  }
  const int rows_padded = round_up_int(m, 128);
  const size_t threads = static_cast<size_t>(rows_padded) * ((((k >> 4) + 3) >> 2) << 2);
  const unsigned blocks = static_cast<unsigned>((threads + kThreads - 1) / kThreads);
  const cudaError_t le = launch_pdl(quantize_nvfp4_kernel<T, kEngine, true>, dim3(blocks), dim3(kThreads), 0, s, x, m, rows_padded, k,
                                    dynamic ? g_dev : nullptr, global_scale, dynamic ? nullptr : g_dev, 0, codes, scales_tiled);
  count_launch();
  Q35B_CUDA_TRY(le, "quantize_nvfp4_kernel launch");
  return Q35B_OK;
}

}  // namespace

int launch_quantize_bf16(const void * x, int m, int k, float global_scale, uint8_t * codes, uint8_t * scales_tiled,
                         float * g_dev, void * workspace, cudaStream_t s) {
  return launch_quantize_activations(static_cast<const __nv_bfloat16 *>(x), m, k, global_scale, codes, scales_tiled, g_dev,
                                     workspace, s);
}

int launch_quantize_f32(const float * x, int m, int k, float global_scale, uint8_t * codes, uint8_t * scales_tiled,
                        float * g_dev, void * workspace, cudaStream_t s) {
  return launch_quantize_activations(x, m, k, global_scale, codes, scales_tiled, g_dev, workspace, s);
}

int launch_quantize_reference_recipe(const void * x, int m, int k, int swap, uint8_t * codes, uint8_t * scales_tiled,
                                     cudaStream_t s) {
  if (const int st = check_quant_args(x, m, k, codes, scales_tiled)) return st;
  const int rows_padded = round_up_int(m, 128);
  const size_t threads = static_cast<size_t>(rows_padded) * ((((k >> 4) + 3) >> 2) << 2);
  const unsigned blocks = static_cast<unsigned>((threads + kThreads - 1) / kThreads);
  quantize_nvfp4_kernel<__nv_bfloat16, kReference, true><<<blocks, kThreads, 0, s>>>(
    static_cast<const __nv_bfloat16 *>(x), m, rows_padded, k, nullptr, 1.0f, nullptr, swap, codes, scales_tiled);
  count_launch();
  Q35B_CUDA_TRY(cudaGetLastError(), "quantize_nvfp4_kernel(reference recipe) launch");
  return Q35B_OK;
}

int launch_quantize_weight_f32(const float * w, int n, int k, uint8_t * codes, uint8_t * scales_rowmajor,
                               float * s2_dev, void * workspace, cudaStream_t s) {
  if (w == nullptr || codes == nullptr || scales_rowmajor == nullptr || s2_dev == nullptr || workspace == nullptr) {
    return fail(Q35B_ERR_ARGUMENT, "NVFP4 weight quantisation received a null buffer.");
  }
  if (n <= 0 || k <= 0 || (k % 16) != 0) return fail(Q35B_ERR_SHAPE, "Invalid dimensions for NVFP4 weight quantisation.");
  if (const int st = launch_amax(w, static_cast<size_t>(n) * k, static_cast<unsigned int *>(workspace), s2_dev, s)) return st;
  const size_t threads = static_cast<size_t>(n) * ((((k >> 4) + 3) >> 2) << 2);
  const unsigned blocks = static_cast<unsigned>((threads + kThreads - 1) / kThreads);
  quantize_nvfp4_kernel<float, kEngine, false><<<blocks, kThreads, 0, s>>>(w, n, n, k, s2_dev, 1.0f, nullptr, 0, codes,
                                                                          scales_rowmajor);
  count_launch();
  Q35B_CUDA_TRY(cudaGetLastError(), "quantize_nvfp4_kernel(weights) launch");
  return Q35B_OK;
}

int launch_tile_scales(const uint8_t * scales_rowmajor, int rows, int scale_cols, uint8_t * tiled,
                       unsigned int * sign_flag, cudaStream_t s) {
  const int rows_padded = round_up_int(rows, 128);
  const size_t threads = static_cast<size_t>(rows_padded) * ((scale_cols + 3) >> 2);
  const unsigned blocks = static_cast<unsigned>((threads + kThreads - 1) / kThreads);
  tile_scales_kernel<<<blocks, kThreads, 0, s>>>(scales_rowmajor, rows, rows_padded, scale_cols, tiled, sign_flag);
  count_launch();
  Q35B_CUDA_TRY(cudaGetLastError(), "tile_scales_kernel launch");
  return Q35B_OK;
}

}  // namespace q35b
