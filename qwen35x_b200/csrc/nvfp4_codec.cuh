// NVFP4 codecs shared by host and device code.
//
// Semantics are those of the reference's exhaustive-scan encoders and
// arithmetic decoders (src/runtime/cuda_bench.cu:36-96 device, :902-940 and
// :1929-1949 host); the encoders here reach the same bytes with a handful of
// integer/compare operations instead of a 128- or 8-iteration scan.  The
// equivalence is proved per threshold by tests/test_codec_fast.py through
// q35b_debug_encode_* (every switch point of the scan, +-1 ulp).
#pragma once

#include <cstdint>
#include <cstring>

#if defined(__CUDACC__)
#define Q35B_HD __host__ __device__ __forceinline__
#else
#define Q35B_HD inline
#endif

namespace q35b {

Q35B_HD uint32_t f32_bits(float f) {
#if defined(__CUDA_ARCH__)
  return __float_as_uint(f);
#else
  uint32_t u;
  std::memcpy(&u, &f, 4);
  return u;
#endif
}

Q35B_HD float bits_f32(uint32_t u) {
#if defined(__CUDA_ARCH__)
  return __uint_as_float(u);
#else
  float f;
  std::memcpy(&f, &u, 4);
  return f;
#endif
}

// E4M3 byte -> fp32 exactly as the reference: 0 -> 0, exponent 0 is
// subnormal (m * 2^-9), 0x7f decodes to 480, the sign bit is honoured.
// (b & 0x7f) << 20 is the value scaled by 2^-120 (also right for subnormals).
Q35B_HD float decode_e4m3(uint8_t b) {
  const float mag = bits_f32(static_cast<uint32_t>(b & 0x7fu) << 20) * 0x1p120f;
  return (b & 0x80u) ? -mag : mag;
}

// E2M1 nibble -> fp32: (c & 7) << 22 is the magnitude scaled by 2^-126.
Q35B_HD float decode_e2m1(uint8_t c) {
  const float mag = bits_f32(static_cast<uint32_t>(c & 7u) << 22) * 0x1p126f;
  return (c & 8u) ? -mag : mag;
}

// The reference's scan, kept for the ranges where fp32 rounding of
// |decoded - value| makes the scan's answer differ from "nearest".
Q35B_HD uint8_t encode_ue4m3_scan(float value) {
  if (!(value > 0.0f)) return 0;
  int best_bits = 0;
  float best_error = bits_f32(0x7f800000u);
  for (int bits = 0; bits < 128; ++bits) {
    const float decoded = decode_e4m3(static_cast<uint8_t>(bits));
    float error = decoded - value;
    error = error < 0.0f ? -error : error;
    if (error < best_error) {
      best_error = error;
      best_bits = bits;
    }
  }
  return static_cast<uint8_t>(best_bits);
}

// fp32 -> nearest non-negative E4M3 byte, ties to the lower byte
// (src/runtime/cuda_bench.cu:902-924).
Q35B_HD uint8_t encode_ue4m3(float value) {
  if (!(value > 0.0f)) return 0;  // also NaN
  const uint32_t u = f32_bits(value);
  if (u >= 0x4b800000u) {  // >= 2^24 (and +inf): outside the exact range, rare
    return encode_ue4m3_scan(value);
  }
  if (u < 0x3c800000u) {  // < 2^-6: subnormal target, levels k * 2^-9
    const float t = value * 512.0f - 0.5f;
    int k = static_cast<int>(t);
    if (static_cast<float>(k) < t) ++k;  // ceil for positive t; t <= 0 gives 0
    return static_cast<uint8_t>(k < 0 ? 0 : k);
  }
  const int e = static_cast<int>(u >> 23) - 127;
  const uint32_t m3 = ((u & 0x7fffffu) + 0x7ffffu) >> 20;  // round half down
  const int code = ((e + 7) << 3) + static_cast<int>(m3);
  return static_cast<uint8_t>(code > 127 ? 127 : code);
}

Q35B_HD uint8_t encode_e2m1_scan(float value) {
  const bool negative = value < 0.0f;
  const float a = value < 0.0f ? -value : value;
  const float levels[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
  int best = 0;
  float best_error = bits_f32(0x7f800000u);
  for (int i = 0; i < 8; ++i) {
    float error = levels[i] - a;
    error = error < 0.0f ? -error : error;
    if (error < best_error) {
      best_error = error;
      best = i;
    }
  }
  return static_cast<uint8_t>((negative ? 8u : 0u) | static_cast<unsigned>(best));
}

// fp32 -> E2M1 nibble, nearest magnitude with ties to the smaller one, sign
// bit = (value < 0) (src/runtime/cuda_bench.cu:926-940).
// The same for |value| < 2^20 or NaN (the scan also gives 0 for NaN): no range check, no branch.
// From 1.0 up the levels are 2^e and 1.5 * 2^e, i.e. the magnitude rounded to one mantissa bit with ties going down:
// adding just under half a step to the bit pattern and dropping 22 bits counts half-exponent steps above 1.0
// (a mantissa carry moves on to the next exponent by itself); level index = 2 + steps, at most 7.  Below 1.0 the
// levels 0, 0.5, 1.0 are told apart by two comparisons.
Q35B_HD uint8_t encode_e2m1_bounded(float value) {
  const uint32_t au = f32_bits(value) & 0x7fffffffu;
  const float a = bits_f32(au);
  const unsigned steps = (au + 0x1fffffu - 0x3f800000u) >> 22;
  const unsigned high = steps + 2u < 7u ? steps + 2u : 7u;
  const unsigned low = (a > 0.25f) + (a > 0.75f);
  const unsigned code = (a >= 1.0f) ? high : low;  // NaN takes the low branch and gets 0, like the scan
  return static_cast<uint8_t>(((value < 0.0f) ? 8u : 0u) | code);
}

Q35B_HD uint8_t encode_e2m1(float value) {
  const uint32_t au = f32_bits(value) & 0x7fffffffu;
  if (au >= 0x49800000u && au <= 0x7f800000u) {  // 2^20 <= |v| <= inf: rare, follow the scan
    return encode_e2m1_scan(value);
  }
  return encode_e2m1_bounded(value);
}

// Round-to-nearest-even fp32 -> bf16 bits (NaN kept quiet), the reference's
// float_to_bf16 (src/runtime/qwen35x_cuda_backend.cpp:622-629).
Q35B_HD uint16_t f32_to_bf16_bits(float f) {
  uint32_t u = f32_bits(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}

Q35B_HD float bf16_bits_to_f32(uint16_t h) { return bits_f32(static_cast<uint32_t>(h) << 16); }

// Byte offset of block scale (row, col) in the 128-row x 4-column tiled
// layout (512-byte tiles, row-block major), the layout of
// nvfp4_tiled_scale_offset_device (src/runtime/cuda_bench.cu:132-142); it is
// also the shared-memory image tcgen05.cp 32x128b.warpx4 expects for the
// scale factors of a 128-row operand tile.
Q35B_HD int64_t tiled_scale_offset(int row, int col, int padded_cols) {
  const int row_block = row >> 7;
  const int row_in_block = row & 127;
  return ((((static_cast<int64_t>(row_block) * (padded_cols >> 2) + (col >> 2)) * 32 + (row_in_block & 31)) * 4 +
           (row_in_block >> 5)) * 4) + (col & 3);
}

Q35B_HD int round_up_int(int v, int m) { return ((v + m - 1) / m) * m; }

}  // namespace q35b
