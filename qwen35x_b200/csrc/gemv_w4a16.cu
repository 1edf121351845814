// W4A16 decode projection (M = 1..8 tokens) for sm_100a.
//
// y[m, r] = sum_c e2m1(w[r,c]) * e4m3(s[r,c/16]) * s2 * x[m,c], fp32 accumulation.
// Replaces the reference's scalar projection kernels
// (src/runtime/cuda_bench.cu:283-429) and the in-megakernel nvfp4_row_dot
// (src/kernels/cuda/decode_layers.cuh:200-261).
//
// HBM layout read here: codes [rows, K/2] and scales [rows, K/16], both
// row-major as in the checkpoint, so a warp that walks a row issues fully
// coalesced 16-byte loads (32 codes per lane) and 2-byte scale loads.
//
// Dequantisation: an E2M1 nibble s|eem placed at fp16 bits 15|11:9 is the
// value scaled by 2^-14 (exact, fp16 subnormals included); the 2^14 is folded
// into the per-block scale, which is decoded once per 16 weights.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "engine.h"
#include "nvfp4_codec.cuh"

namespace q35b {
namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kThreads = kWarpsPerBlock * 32;

// Two E2M1 codes (nibbles j and j+4 of `w`, j = shift/4) -> float2 scaled by 2^-14.
__device__ __forceinline__ float2 e2m1_pair_to_f32(uint32_t w, int shift) {
  const uint32_t q = (w >> shift);
  const uint32_t bits = ((q & 0x00070007u) << 9) | ((q & 0x00080008u) << 12);
  const __half2 h = *reinterpret_cast<const __half2 *>(&bits);
  return __half22float2(h);
}

// E4M3 byte -> fp32 (the reference's decode, sign honoured, 0x7f = 480).
__device__ __forceinline__ float e4m3_to_f32(uint32_t b) {
  const float mag = __uint_as_float((b & 0x7fu) << 20) * 0x1p120f;
  return (b & 0x80u) ? -mag : mag;
}

template <typename XT>
struct XLoad;

// 32 consecutive activations -> fp32 registers.
template <>
struct XLoad<__nv_bfloat16> {
  static __device__ __forceinline__ void load32(const __nv_bfloat16 * p, float scale, float (&x)[32]) {
    const uint4 * v = reinterpret_cast<const uint4 *>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 q = __ldg(v + i);
      const uint32_t r[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        x[i * 8 + j * 2 + 0] = __uint_as_float(r[j] << 16) * scale;
        x[i * 8 + j * 2 + 1] = __uint_as_float(r[j] & 0xffff0000u) * scale;
      }
    }
  }
};

template <>
struct XLoad<float> {
  static __device__ __forceinline__ void load32(const float * p, float scale, float (&x)[32]) {
    const float4 * v = reinterpret_cast<const float4 *>(p);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float4 q = __ldg(v + i);
      x[i * 4 + 0] = q.x * scale;
      x[i * 4 + 1] = q.y * scale;
      x[i * 4 + 2] = q.z * scale;
      x[i * 4 + 3] = q.w * scale;
    }
  }
};

__device__ __forceinline__ void store_out(__nv_bfloat16 * p, float v) { *p = __float2bfloat16_rn(v); }
__device__ __forceinline__ void store_out(float * p, float v) { *p = v; }

// Dot product of 16 weights (two 32-bit code words) with 16 activations.
// Code j of the block sits in nibble j%8 of word j/8.
__device__ __forceinline__ float block_dot(uint32_t w0, uint32_t w1, const float * x) {
  float acc = 0.0f;
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const float2 a = e2m1_pair_to_f32(w0, 4 * p);  // codes p and p+4
    acc = fmaf(a.x, x[p], acc);
    acc = fmaf(a.y, x[p + 4], acc);
  }
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const float2 a = e2m1_pair_to_f32(w1, 4 * p);
    acc = fmaf(a.x, x[8 + p], acc);
    acc = fmaf(a.y, x[8 + p + 4], acc);
  }
  return acc;
}

// One warp owns RW consecutive rows; lanes stride over K in 32-code (16-byte)
// pieces; a warp-shuffle tree finishes each (row, token) sum.
// Requires K % 32 == 0.
template <int M, int RW, typename XT, typename OT>
__global__ void __launch_bounds__(kThreads)
gemv_w4a16_simt_kernel(const uint8_t * __restrict__ codes, const uint8_t * __restrict__ scales,
                       const XT * __restrict__ x, OT * __restrict__ y, int rows, int k, float s2_scaled,
                       float x_scale) {
  // Launched with programmatic stream serialisation: the grid may be scheduled while the previous kernel of the
  // stream drains (a 2 MB projection is shorter than a launch), but reads and writes nothing before that kernel is
  // complete and visible.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int lane = threadIdx.x & 31;
  const int warp = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int row0 = warp * RW;
  if (row0 >= rows) return;
  const int packed_cols = k >> 1;
  const int scale_cols = k >> 4;

  float acc[RW][M];
#pragma unroll
  for (int r = 0; r < RW; ++r)
#pragma unroll
    for (int m = 0; m < M; ++m) acc[r][m] = 0.0f;

  for (int k0 = lane * 32; k0 < k; k0 += 32 * 32) {
    uint4 cw[RW];
    uint32_t sc[RW];
#pragma unroll
    for (int r = 0; r < RW; ++r) {
      const int row = min(row0 + r, rows - 1);
      cw[r] = __ldcs(reinterpret_cast<const uint4 *>(codes + static_cast<size_t>(row) * packed_cols + (k0 >> 1)));
      sc[r] = __ldcs(reinterpret_cast<const unsigned short *>(scales + static_cast<size_t>(row) * scale_cols + (k0 >> 4)));
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float xv[32];
      XLoad<XT>::load32(x + static_cast<size_t>(m) * k + k0, x_scale, xv);
#pragma unroll
      for (int r = 0; r < RW; ++r) {
        const float d0 = block_dot(cw[r].x, cw[r].y, xv);
        const float d1 = block_dot(cw[r].z, cw[r].w, xv + 16);
        acc[r][m] = fmaf(d0, e4m3_to_f32(sc[r] & 0xffu), acc[r][m]);
        acc[r][m] = fmaf(d1, e4m3_to_f32(sc[r] >> 8), acc[r][m]);
      }
    }
  }

#pragma unroll
  for (int r = 0; r < RW; ++r) {
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float v = acc[r][m];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
      if (lane == 0 && row0 + r < rows) {
        store_out(y + static_cast<size_t>(m) * rows + row0 + r, v * s2_scaled);
      }
    }
  }
}

// Any K % 16 == 0: one warp per row, one 16-weight block per lane step, byte
// loads.  Only shapes the vector kernel cannot take end up here.
template <typename XT, typename OT>
__global__ void __launch_bounds__(kThreads)
gemv_w4a16_generic_kernel(const uint8_t * __restrict__ codes, const uint8_t * __restrict__ scales,
                          const XT * __restrict__ x, OT * __restrict__ y, int rows, int k, int m_tokens,
                          float s2_scaled, float x_scale) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int packed_cols = k >> 1;
  const int scale_cols = k >> 4;
  for (int m = 0; m < m_tokens; ++m) {
    float acc = 0.0f;
    for (int b = lane; b < scale_cols; b += 32) {
      const uint2 cw = *reinterpret_cast<const uint2 *>(codes + static_cast<size_t>(row) * packed_cols + b * 8);
      float xv[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) xv[i] = static_cast<float>(x[static_cast<size_t>(m) * k + b * 16 + i]) * x_scale;
      acc = fmaf(block_dot(cw.x, cw.y, xv), e4m3_to_f32(scales[static_cast<size_t>(row) * scale_cols + b]), acc);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) store_out(y + static_cast<size_t>(m) * rows + row, acc * s2_scaled);
  }
}

// One thread per 16-weight block: bf16(e2m1 * (e4m3 * s2)), the reference's load-time dequantisation
// (src/runtime/qwen35x_cuda_backend.cpp:742-755).  Rows of a gate/up weight take the scale of their half.
__global__ void __launch_bounds__(kThreads)
dequant_bf16_kernel(const uint8_t * __restrict__ codes, const uint8_t * __restrict__ scales, __nv_bfloat16 * __restrict__ out,
                    int rows, int k, float s2, float s2_up, int gate_up) {
  const int scale_cols = k >> 4;
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<size_t>(rows) * scale_cols) return;
  const int row = static_cast<int>(idx / scale_cols);
  const float row_s2 = (gate_up && ((row >> 3) & 1)) ? s2_up : s2;
  const float scale = e4m3_to_f32(scales[idx]) * row_s2;
  const uint2 cw = *reinterpret_cast<const uint2 *>(codes + idx * 8);
  const uint32_t w[2] = {cw.x, cw.y};
  uint32_t packed[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t c0 = (w[j >> 2] >> ((j & 3) * 8)) & 0xfu;
    const uint32_t c1 = (w[j >> 2] >> ((j & 3) * 8 + 4)) & 0xfu;
    const float v0 = __uint_as_float(((c0 & 7u) << 22) | ((c0 & 8u) << 28)) * 0x1p126f * scale;
    const float v1 = __uint_as_float(((c1 & 7u) << 22) | ((c1 & 8u) << 28)) * 0x1p126f * scale;
    const __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
    packed[j] = *reinterpret_cast<const uint32_t *>(&h);
  }
  uint4 * dst = reinterpret_cast<uint4 *>(out + idx * 16);
  dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
}

template <int M, typename XT, typename OT>
int launch_simt(const q35b_weight * w, const XT * x, OT * y, float x_scale, cudaStream_t s) {
  constexpr int RW = (M <= 2) ? 2 : 1;
  const int warps = (w->rows + RW - 1) / RW;
  const int blocks = (warps + kWarpsPerBlock - 1) / kWarpsPerBlock;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(blocks));
  cfg.blockDim = dim3(kThreads);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const uint8_t * codes = w->codes;
  const uint8_t * scales = w->scales;
  const cudaError_t le = cudaLaunchKernelEx(&cfg, gemv_w4a16_simt_kernel<M, RW, XT, OT>, codes, scales, x, y, w->rows, w->k,
                                            w->s2 * 16384.0f, x_scale);
  count_launch();
  Q35B_CUDA_TRY(le, "gemv_w4a16_simt_kernel launch");
  return Q35B_OK;
}

template <typename XT, typename OT>
int launch_any(const q35b_weight * w, const XT * x, int m, OT * y, float x_scale, int kernel, cudaStream_t s) {
  if (w == nullptr || x == nullptr || y == nullptr) return fail(Q35B_ERR_ARGUMENT, "NVFP4 projection received a null buffer.");
  if (m < 1 || m > 8) return fail(Q35B_ERR_SHAPE, "NVFP4 decode projection supports 1..8 tokens.");
  if (w->rows == 0) return Q35B_OK;
  if (w->gate_up) return fail(Q35B_ERR_ARGUMENT, "A gate/up weight runs through the projection work list (q35b_gemv_batch_*).");
  if (kernel != Q35B_GEMV_AUTO && kernel != Q35B_GEMV_SIMT && kernel != Q35B_GEMV_STREAM) {
    return fail(Q35B_ERR_ARGUMENT, "Unknown NVFP4 projection kernel id " + std::to_string(kernel) + ".");
  }
  if (const int st = check_weight_device(w)) return st;
  if ((w->k % 32) == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) != 0) {
    // the vector kernel reads activations with 16-byte loads
    return fail(Q35B_ERR_ARGUMENT, "Activations of the NVFP4 projection must be 16-byte aligned.");
  }
  if ((w->k % 32) != 0) {
    const int blocks = (w->rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
    gemv_w4a16_generic_kernel<XT, OT><<<blocks, kThreads, 0, s>>>(w->codes, w->scales, x, y, w->rows, w->k, m,
                                                                 w->s2 * 16384.0f, x_scale);
    count_launch();
    Q35B_CUDA_TRY(cudaGetLastError(), "gemv_w4a16_generic_kernel launch");
    return Q35B_OK;
  }
  switch (m) {
    case 1: return launch_simt<1>(w, x, y, x_scale, s);
    case 2: return launch_simt<2>(w, x, y, x_scale, s);
    case 3: return launch_simt<3>(w, x, y, x_scale, s);
    case 4: return launch_simt<4>(w, x, y, x_scale, s);
    case 5: return launch_simt<5>(w, x, y, x_scale, s);
    case 6: return launch_simt<6>(w, x, y, x_scale, s);
    case 7: return launch_simt<7>(w, x, y, x_scale, s);
    default: return launch_simt<8>(w, x, y, x_scale, s);
  }
}

}  // namespace

int launch_dequant_bf16(const q35b_weight * w, void * w_bf16, cudaStream_t s) {
  if (w == nullptr || w_bf16 == nullptr) return fail(Q35B_ERR_ARGUMENT, "NVFP4 dequantisation received a null buffer.");
  if ((reinterpret_cast<uintptr_t>(w_bf16) & 15u) != 0) return fail(Q35B_ERR_ARGUMENT, "NVFP4 dequantisation output must be 16-byte aligned.");
  if (const int st = check_weight_device(w)) return st;
  if (w->rows == 0) return Q35B_OK;
  const size_t blocks16 = static_cast<size_t>(w->rows) * (w->k / 16);
  dequant_bf16_kernel<<<static_cast<unsigned>((blocks16 + kThreads - 1) / kThreads), kThreads, 0, s>>>(
    w->codes, w->scales, static_cast<__nv_bfloat16 *>(w_bf16), w->rows, w->k, w->s2, w->s2_up, w->gate_up ? 1 : 0);
  count_launch();
  Q35B_CUDA_TRY(cudaGetLastError(), "dequant_bf16_kernel launch");
  return Q35B_OK;
}

int launch_gemv_bf16(const q35b_weight * w, const void * x_bf16, int m, void * y_bf16, int kernel, cudaStream_t s) {
  return launch_any(w, static_cast<const __nv_bfloat16 *>(x_bf16), m, static_cast<__nv_bfloat16 *>(y_bf16), 1.0f,
                    kernel, s);
}

int launch_gemv_f32(const q35b_weight * w, const float * x, float input_scale, float * y, int kernel, cudaStream_t s) {
  return launch_any(w, x, 1, y, input_scale, kernel, s);
}

}  // namespace q35b
