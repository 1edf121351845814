// One 16-element NVFP4 block: amax -> UE4M3 scale byte -> sixteen E2M1 codes.  Shared by the stand-alone
// quantiser (act_quant.cu) and the GEMM epilogue that emits quantised activations (gemm_epilogue.cuh), so that
// both produce the same bits from the same values.
//
// Recipes (all fp32, IEEE division, no fused contraction that could change a rounding):
//   engine     t = amax_blk / 6; sb = min(UE4M3(max(t / g, 1e-8)), 0x7e); d = max(decode(sb), 1e-8) * g
//   reference  d = max(amax_blk / 6, 1e-8); sb = UE4M3(d)      (src/runtime/cuda_bench.cu:98-213)
//   code_i = E2M1(x_i / d), element 2j in the low nibble (or swapped for the reference's cuBLASLt order)
#pragma once

#include <cstdint>

#include "nvfp4_codec.cuh"

namespace q35b {

enum Recipe { kEngine = 0, kReference = 1 };

// x / d rounded to nearest, for a divisor whose refined reciprocal r is at hand: quotient estimate, then two
// residual corrections, the last one delivering the rounded result.  The block's sixteen quotients share one
// divisor, so this replaces sixteen full divisions (each with its own reciprocal and range check) by one
// reciprocal and five dependent-free FMA-pipe instructions per element.  Used only when the block's divisor and
// amax are far from the exponent limits (see quantize_block); tests/test_quant_gpu.py feeds it values placed
// ulp by ulp around every rounding boundary of the E2M1 encoder and compares with IEEE division on the host.
__device__ __forceinline__ float div_by_shared(float x, float d, float r) {
  float q = __fmul_rn(x, r);
  float e = __fmaf_rn(-d, q, x);
  q = __fmaf_rn(e, r, q);
  e = __fmaf_rn(-d, q, x);
  return __fmaf_rn(e, r, q);
}

// encode_e2m1_bounded (nvfp4_codec.cuh) on 32-bit values throughout: no narrowing to a byte and back per element.
__device__ __forceinline__ uint32_t e2m1_code_bounded(float q) {
  const uint32_t au = __float_as_uint(q) & 0x7fffffffu;
  const float a = __uint_as_float(au);
  const uint32_t high = min((au + (0x1fffffu - 0x3f800000u + 0x800000u)) >> 22, 7u);  // 2 + half-exponent steps above 1.0
  const uint32_t low = (a > 0.25f ? 1u : 0u) + (a > 0.75f ? 1u : 0u);
  return ((a >= 1.0f) ? high : low) | ((q < 0.0f) ? 8u : 0u);
}

// Quantise one 16-block; returns the scale byte, writes 8 code bytes.
template <int RECIPE>
__device__ __forceinline__ uint32_t quantize_block(const float (&v)[16], float g, bool swap, uint2 & out) {
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  uint32_t sb;
  float d;
  if (RECIPE == kEngine) {
    const float t = __fdiv_rn(amax, 6.0f);
    sb = encode_ue4m3(fmaxf(__fdiv_rn(t, g), 1.0e-8f));
    sb = sb > 0x7eu ? 0x7eu : sb;
    d = __fmul_rn(fmaxf(decode_e4m3(static_cast<uint8_t>(sb)), 1.0e-8f), g);
  } else {
    d = fmaxf(__fdiv_rn(amax, 6.0f), 1.0e-8f);
    sb = encode_ue4m3(d);
  }
  uint32_t code[16];
  // exponents of d and amax inside [2^-60, 2^60]: no intermediate of div_by_shared can overflow, and a quotient
  // small enough to lose bits is far below the first rounding boundary (0.25); amax < 2^19 d keeps every quotient
  // inside the range of the branch-free encoder
  const uint32_t de = (__float_as_uint(d) >> 23) & 0xffu, ae = (__float_as_uint(amax) >> 23) & 0xffu;
  if (de >= 67u && de <= 187u && ae <= 187u && amax < d * 524288.0f) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(d));
    r = __fmaf_rn(r, __fmaf_rn(-d, r, 1.0f), r);
#pragma unroll
    for (int i = 0; i < 16; ++i) code[i] = e2m1_code_bounded(div_by_shared(v[i], d, r));
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) code[i] = encode_e2m1(__fdiv_rn(v[i], d));
  }
  // element 2j in the low nibble of byte j: eight codes per word, built as word * 16 + code from the top down
  // (multiply-adds, which leave the comparison pipe to the encoders); the reference's cuBLASLt order swaps the two
  // nibbles of every byte afterwards
  uint32_t word[2] = {0u, 0u};
#pragma unroll
  for (int h = 0; h < 2; ++h) {
#pragma unroll
    for (int i = 7; i >= 0; --i) word[h] = word[h] * 16u + code[8 * h + i];
    if (swap) word[h] = ((word[h] & 0x0f0f0f0fu) << 4) | ((word[h] >> 4) & 0x0f0f0f0fu);
  }
  out = make_uint2(word[0], word[1]);
  return sb;
}

}  // namespace q35b
