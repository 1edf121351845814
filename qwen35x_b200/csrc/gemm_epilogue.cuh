// Epilogue shared by the tcgen05 GEMM kernels: one thread holds 32 consecutive fp32 accumulator columns of one
// output row and turns them into BF16 in global memory.
//
//   plain      c[row, col0 + i] = bf16(acc_i * alpha (+ residual[row, col0 + i]))
//   gate/up    the weight's rows (= accumulator columns) alternate 8 gate / 8 up, so each 16-column group yields 8
//              outputs c[row, (col0 + 16 j) / 2 + i] = bf16(silu(gate_i * alpha) * (up_i * alpha_up)),
//              silu(g) = g / (1 + exp(-g)): the SiLU-multiply the reference runs as a separate pass after its
//              gate and up GEMMs (src/kernels/cuda/prefill.cu:674-678, pf_silu_mul_bf16), and half the bytes written.
//   residual   replaces pf_add_residual_bf16 after the down / o projections (src/kernels/cuda/prefill.cu:679).
//   gate/up -> NVFP4   the same SiLU-multiply, rounded to BF16 exactly as above, then quantised in place of being
//              stored: the 16 outputs a thread holds per 32 accumulator columns are one NVFP4 block, so it writes
//              8 code bytes and one scale byte of the tiled layout, ready to be the A operand of the down
//              projection.  Replaces the reference's quantise pass between its gate/up and down GEMMs
//              (src/runtime/cuda_bench.cu:2621-2660) and needs the activation's per-tensor scale in advance (the
//              checkpoint's input_scale of the down projection, or a calibrated value).
#pragma once

#include <cuda_bf16.h>

#include <cstdint>

#include "nvfp4_quant_block.cuh"

namespace q35b {

struct GemmEpilogue {
  float s2 = 1.0f;        // weight_scale_2 (gate half for a gate/up weight)
  float s2_up = 1.0f;     // weight_scale_2 of the up half
  int gate_up = 0;
  const __nv_bfloat16 * residual = nullptr;  // [m, n], row stride ldr
  int ldr = 0;
  // gate/up -> NVFP4 (all three set, or none): codes [m, n/4] bytes, tiled scales of the [m, n/2] activation with
  // q_slots = roundup(n/32, 4) scale columns per row, and that activation's per-tensor scale (device scalar)
  uint8_t * q_codes = nullptr;
  uint8_t * q_scales = nullptr;
  const float * q_g = nullptr;
  int q_slots = 0;
};

__device__ __forceinline__ void st_global_v8(void * p, const uint32_t (&v)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]),
               "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}

// silu(g) * u with the hardware exponential and reciprocal (a few fp32 ulp, far inside the BF16 rounding that follows)
__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t *>(&h);
}

// r: 32 accumulator columns starting at global column col0 (a multiple of 32) of row `row`; n = accumulator columns
// of the whole problem (weight rows); g = the activation tensor's scale.
__device__ __forceinline__ void gemm_store_chunk32(const uint32_t (&r)[32], int row, int col0, int n, float g,
                                                   const GemmEpilogue & ep, __nv_bfloat16 * __restrict__ c, int ldc) {
  const float alpha = g * ep.s2;
  if (ep.gate_up) {
    const float alpha_up = g * ep.s2_up;
    if (ep.q_codes != nullptr) {
      // n % 32 == 0 is checked on the host, so the chunk is whole
      float v[16];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float gv = __uint_as_float(r[16 * j + i]) * alpha;
          const float uv = __uint_as_float(r[16 * j + 8 + i]) * alpha_up;
          v[8 * j + i] = __bfloat162float(__float2bfloat16_rn(silu_mul(gv, uv)));
        }
      }
      uint2 packed;
      const uint32_t sb = quantize_block<kEngine>(v, __ldg(ep.q_g), false, packed);
      *reinterpret_cast<uint2 *>(ep.q_codes + static_cast<size_t>(row) * (n >> 2) + (col0 >> 2)) = packed;
      ep.q_scales[tiled_scale_offset(row, col0 >> 5, ep.q_slots)] = static_cast<uint8_t>(sb);
      return;
    }
    __nv_bfloat16 * dst = c + static_cast<size_t>(row) * ldc + (col0 >> 1);
    if (col0 + 32 <= n && ((reinterpret_cast<uintptr_t>(dst) & 31u) == 0)) {
      uint32_t p[8];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
          const float g0 = __uint_as_float(r[16 * j + i]) * alpha, g1 = __uint_as_float(r[16 * j + i + 1]) * alpha;
          const float u0 = __uint_as_float(r[16 * j + 8 + i]) * alpha_up, u1 = __uint_as_float(r[16 * j + 8 + i + 1]) * alpha_up;
          p[4 * j + (i >> 1)] = pack_bf16(silu_mul(g0, u0), silu_mul(g1, u1));
        }
      }
      st_global_v8(dst, p);
    } else {
      for (int j = 0; j < 2; ++j) {
        for (int i = 0; i < 8; ++i) {
          if (col0 + 16 * j + 8 + i < n) {
            const float gv = __uint_as_float(r[16 * j + i]) * alpha;
            const float uv = __uint_as_float(r[16 * j + 8 + i]) * alpha_up;
            dst[8 * j + i] = __float2bfloat16_rn(silu_mul(gv, uv));
          }
        }
      }
    }
    return;
  }
  __nv_bfloat16 * dst = c + static_cast<size_t>(row) * ldc + col0;
  const __nv_bfloat16 * res = ep.residual != nullptr ? ep.residual + static_cast<size_t>(row) * ep.ldr + col0 : nullptr;
  if (col0 + 32 <= n && ((reinterpret_cast<uintptr_t>(dst) & 31u) == 0) &&
      (res == nullptr || (reinterpret_cast<uintptr_t>(res) & 15u) == 0)) {
#pragma unroll
    for (int v = 0; v < 2; ++v) {
      uint32_t p[8];
      uint32_t rr[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
      if (res != nullptr) {
        const uint4 a = __ldg(reinterpret_cast<const uint4 *>(res + v * 16));
        const uint4 b = __ldg(reinterpret_cast<const uint4 *>(res + v * 16 + 8));
        rr[0] = a.x; rr[1] = a.y; rr[2] = a.z; rr[3] = a.w;
        rr[4] = b.x; rr[5] = b.y; rr[6] = b.z; rr[7] = b.w;
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float r0 = __uint_as_float(rr[e] << 16), r1 = __uint_as_float(rr[e] & 0xffff0000u);
        p[e] = pack_bf16(fmaf(__uint_as_float(r[v * 16 + e * 2]), alpha, r0),
                         fmaf(__uint_as_float(r[v * 16 + e * 2 + 1]), alpha, r1));
      }
      st_global_v8(dst + v * 16, p);
    }
  } else {
    for (int e = 0; e < 32; ++e) {
      if (col0 + e < n) {
        const float rv = res != nullptr ? __bfloat162float(res[e]) : 0.0f;
        dst[e] = __float2bfloat16_rn(fmaf(__uint_as_float(r[e]), alpha, rv));
      }
    }
  }
}

}  // namespace q35b
