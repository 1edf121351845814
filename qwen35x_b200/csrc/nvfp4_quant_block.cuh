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

// Eight quotients -> one word of eight E2M1 codes with the hardware converter (nearest on the E2M1 grid, saturating
// at 6, sign kept): byte j holds element 2j in its low nibble and 2j + 1 in its high nibble.
__device__ __forceinline__ uint32_t cvt_e2m1x8(const float (&q)[8]) {
  uint32_t w;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
      : "=r"(w)
      : "f"(q[0]), "f"(q[1]), "f"(q[2]), "f"(q[3]), "f"(q[4]), "f"(q[5]), "f"(q[6]), "f"(q[7]));
  return w;
}

// Quantise one 16-block; returns the scale byte, writes 8 code bytes.
template <int RECIPE>
__device__ __forceinline__ uint32_t quantize_block(const float (&v)[16], float g, bool swap, uint2 & out) {
  // block amax that turns NaN if any element is NaN (max.NaN), so that such a block is recognised below; the
  // reference's fmaxf chain, which skips NaNs, is recomputed for those blocks only
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) asm("max.NaN.f32 %0, %0, %1;" : "+f"(amax) : "f"(fabsf(v[i])));
  const bool has_nan = amax != amax;
  if (has_nan) {
    amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  }
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
  // exponents of d and amax inside [2^-60, 2^60]: no intermediate of the shared-reciprocal quotients can overflow,
  // and a quotient small enough to lose bits is far below the first rounding boundary (0.25); amax < 2^19 d keeps
  // every quotient finite and far inside the converter's range
  const uint32_t de = (__float_as_uint(d) >> 23) & 0xffu, ae = (__float_as_uint(amax) >> 23) & 0xffu;
  uint32_t word[2] = {0u, 0u};
  if (!has_nan && de >= 67u && de <= 187u && ae <= 187u && amax < d * 524288.0f) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(d));
    r = __fmaf_rn(r, __fmaf_rn(-d, r, 1.0f), r);
    // Bracket every quotient: x * r lies within 2^-23 (relative) of x / d, so lo = x * r (1 - 2^-20) and
    // hi = x * r (1 + 2^-20) enclose the correctly rounded quotient strictly.  The code is a monotone function of
    // the quotient and the hardware converter agrees with the reference's nearest-with-ties-down encoder
    // everywhere except exactly on a rounding boundary, so where lo and hi convert to the same code the
    // reference's code is that code; a boundary inside the bracket shows up as two different codes, and only that
    // pair of elements is redone with correctly rounded quotients and the ties-down encoder.  A negative value that
    // rounds to zero keeps its sign bit in both encoders; the + 0.0f turns x = -0 into +0, as (value < 0) does.
    const float r_lo = __fmul_rn(r, 1.0f - 0x1p-20f), r_hi = __fmul_rn(r, 1.0f + 0x1p-20f);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float lo[8], hi[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        lo[i] = __fmaf_rn(v[8 * h + i], r_lo, 0.0f);
        hi[i] = __fmaf_rn(v[8 * h + i], r_hi, 0.0f);
      }
      const uint32_t w_lo = cvt_e2m1x8(lo), w_hi = cvt_e2m1x8(hi);
      uint32_t w = w_lo;
      const uint32_t diff = w_lo ^ w_hi;
      if (diff != 0u) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if ((diff >> (8 * j)) & 0xffu) {
            const uint32_t c0 = e2m1_code_bounded(div_by_shared(v[8 * h + 2 * j], d, r));
            const uint32_t c1 = e2m1_code_bounded(div_by_shared(v[8 * h + 2 * j + 1], d, r));
            w = (w & ~(0xffu << (8 * j))) | ((c0 | (c1 << 4)) << (8 * j));
          }
        }
      }
      word[h] = w;
    }
  } else {
    uint32_t code[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) code[i] = encode_e2m1(__fdiv_rn(v[i], d));
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
      for (int i = 7; i >= 0; --i) word[h] = word[h] * 16u + code[8 * h + i];
    }
  }
  // element 2j sits in the low nibble of byte j; the reference's cuBLASLt order swaps the two nibbles of every byte
  if (swap) {
#pragma unroll
    for (int h = 0; h < 2; ++h) word[h] = ((word[h] & 0x0f0f0f0fu) << 4) | ((word[h] >> 4) & 0x0f0f0f0fu);
  }
  out = make_uint2(word[0], word[1]);
  return sb;
}

}  // namespace q35b
