/*
 * CPU oracle for the NVFP4 projection path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the host-side arithmetic the reference
 * (Danmoreng/qwen35x) embeds in its CUDA benchmark functions.  It is the
 * checker that the parity tests, the smoke test and the benchmark's
 * cpu_baseline leg compare the CUDA path against; the product library never
 * links or calls it.
 *
 * Each function names the reference lines it follows (paths are relative to
 * the reference project root).
 *
 * Parity status: the codecs, encoders, the tiled scale layout and the
 * cuBLASLt-style activation quantiser are pinned against the reference's own
 * host functions (compiled unmodified from the reference tree into
 * oracle/_ref by oracle/build_oracle.py, see tests/test_oracle_vs_reference.py)
 * and against committed golden vectors generated from them.  The W4A4 GEMM
 * expected value has no asserting counterpart in the reference (its cuBLASLt
 * call is only reported, never checked); it is pinned to an OUTPUT of the
 * reference instead: run_nvfp4_cublaslt_prefill_projection_device_bf16
 * (cuda_bench.cu:1056-1167) run on the GPU box agrees with the engine's GEMM,
 * which tests/test_gemm_gpu.py holds to this function, to relative L2 1e-3
 * (tests/test_reference_gpu.py); the formula followed is cuda_bench.cu:872-884.
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (no fused
 * multiply-add contraction: results must be bit-identical to IEEE fp32 code
 * on the GPU compiled without fast-math).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define Q35O_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ */
/* bf16 helpers                                                        */
/* ------------------------------------------------------------------ */

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* Round-to-nearest-even fp32 -> bf16, as src/runtime/qwen35x_cuda_backend.cpp:622-629
 * (NaN kept quiet). */
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) {
    return (uint16_t)((u >> 16) | 0x0040u);
  }
  const uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}

Q35O_API float q35o_bf16_to_f32(uint16_t h) { return bf16_to_f32(h); }
Q35O_API uint16_t q35o_f32_to_bf16(float f) { return f32_to_bf16(f); }

/* ------------------------------------------------------------------ */
/* codecs                                                              */
/* ------------------------------------------------------------------ */

static const float kE2M1Levels[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

/* src/runtime/cuda_bench.cu:1929-1933 (host) and :36-40 (device). */
Q35O_API float q35o_decode_e2m1(uint8_t nibble) {
  const float v = kE2M1Levels[nibble & 0x7u];
  return (nibble & 0x8u) ? -v : v;
}

/* src/runtime/cuda_bench.cu:1935-1949.  Note: 0x7f decodes to 480, the sign
 * bit is honoured, there is no NaN. */
Q35O_API float q35o_decode_e4m3(uint8_t bits) {
  if (bits == 0) {
    return 0.0f;
  }
  const int sign = (bits >> 7) & 1;
  const int exponent = (bits >> 3) & 0xf;
  const int mantissa = bits & 0x7;
  float value;
  if (exponent == 0) {
    value = ldexpf((float)mantissa / 8.0f, -6);
  } else {
    value = ldexpf(1.0f + (float)mantissa / 8.0f, exponent - 7);
  }
  return sign ? -value : value;
}

/* src/runtime/cuda_bench.cu:902-924: exhaustive scan over the 128
 * non-negative E4M3 bit patterns, strict '<' so ties go to the lower bits;
 * non-positive and NaN inputs give 0. */
Q35O_API uint8_t q35o_encode_ue4m3(float value) {
  if (!(value > 0.0f)) {
    return 0;
  }
  int best_bits = 0;
  float best_error = INFINITY;
  for (int exponent = 0; exponent < 16; ++exponent) {
    for (int mantissa = 0; mantissa < 8; ++mantissa) {
      float decoded;
      if (exponent == 0) {
        decoded = ldexpf((float)mantissa / 8.0f, -6);
      } else {
        decoded = ldexpf(1.0f + (float)mantissa / 8.0f, exponent - 7);
      }
      const float error = fabsf(decoded - value);
      if (error < best_error) {
        best_error = error;
        best_bits = (exponent << 3) | mantissa;
      }
    }
  }
  return (uint8_t)best_bits;
}

/* src/runtime/cuda_bench.cu:926-940: nearest of the 8 magnitudes, strict '<'
 * so ties go to the smaller magnitude; sign bit = (value < 0). */
Q35O_API uint8_t q35o_encode_e2m1(float value) {
  const int negative = value < 0.0f;
  const float abs_value = fabsf(value);
  int best = 0;
  float best_error = INFINITY;
  for (int i = 0; i < 8; ++i) {
    const float error = fabsf(kE2M1Levels[i] - abs_value);
    if (error < best_error) {
      best_error = error;
      best = i;
    }
  }
  return (uint8_t)((negative ? 0x8u : 0u) | (unsigned)best);
}

/* ------------------------------------------------------------------ */
/* tiled block-scale layout                                            */
/* ------------------------------------------------------------------ */

static inline int round_up(int v, int m) { return ((v + m - 1) / m) * m; }

/* src/runtime/cuda_bench.cu:132-142: byte offset of scale (row, col) in the
 * 128-row x 4-column tiled layout; cols = number of scale columns (K/16). */
Q35O_API int64_t q35o_tiled_scale_offset(int row, int col, int cols) {
  const int padded_cols = round_up(cols, 4);
  const int row_block = row / 128;
  const int row_in_block = row & 127;
  const int row_group = row_in_block / 32;
  const int row_in_group = row_in_block & 31;
  const int col_block = col / 4;
  const int col_in_group = col & 3;
  return ((((int64_t)row_block * (padded_cols / 4) + col_block) * 32 + row_in_group) * 4 + row_group) * 4 +
         col_in_group;
}

Q35O_API int64_t q35o_tiled_scale_bytes(int rows, int cols) {
  return (int64_t)round_up(rows, 128) * round_up(cols, 4);
}

/* src/runtime/cuda_bench.cu:1173-1203: pad to 128 x 4 multiples and reorder
 * into 512-byte tiles.  out must hold q35o_tiled_scale_bytes(rows, cols). */
Q35O_API void q35o_swizzle_scales(const uint8_t *scale, int rows, int cols, uint8_t *out) {
  const int padded_rows = round_up(rows, 128);
  const int padded_cols = round_up(cols, 4);
  size_t o = 0;
  for (int rb = 0; rb < padded_rows / 128; ++rb) {
    for (int cb = 0; cb < padded_cols / 4; ++cb) {
      for (int rig = 0; rig < 32; ++rig) {
        for (int rg = 0; rg < 4; ++rg) {
          for (int cig = 0; cig < 4; ++cig) {
            const int row = rb * 128 + rg * 32 + rig;
            const int col = cb * 4 + cig;
            out[o++] = (row < rows && col < cols) ? scale[(size_t)row * cols + col] : 0;
          }
        }
      }
    }
  }
}

/* ------------------------------------------------------------------ */
/* W4A16 projection                                                    */
/* ------------------------------------------------------------------ */

/* src/runtime/cuda_bench.cu:2091-2100 (and :1978-1986 with input_scale = 1):
 * y[r] = sum_c e2m1(w) * (e4m3(s) * s2) * (x[c] * input_scale), fp32,
 * accumulated in column order.  x is fp32 here, exactly as the reference's
 * benchmark.  Rows [row_begin, row_end) only. */
Q35O_API void q35o_matvec_f32(const uint8_t *codes, const uint8_t *scales, float input_scale, float s2,
                              int rows, int cols, const float *x, int row_begin, int row_end, float *y) {
  const int packed_cols = cols / 2;
  const int scale_cols = cols / 16;
  (void)rows;
  for (int row = row_begin; row < row_end; ++row) {
    float acc = 0.0f;
    for (int c = 0; c < cols; ++c) {
      const uint8_t packed = codes[(size_t)row * packed_cols + c / 2];
      const uint8_t nibble = (c & 1) == 0 ? (packed & 0x0fu) : (uint8_t)(packed >> 4u);
      const float scale = q35o_decode_e4m3(scales[(size_t)row * scale_cols + c / 16]) * s2;
      acc += q35o_decode_e2m1(nibble) * scale * (x[c] * input_scale);
    }
    y[row - row_begin] = acc;
  }
}

/* Decode one weight row into fp32 values e2m1 * (e4m3 * s2), the per-element
 * weight of cuda_bench.cu:2096-2098. */
static void dequant_row(const uint8_t *codes, const uint8_t *scales, float s2, int cols, float *w) {
  for (int c = 0; c < cols; ++c) {
    const uint8_t packed = codes[c / 2];
    const uint8_t nibble = (c & 1) == 0 ? (packed & 0x0fu) : (uint8_t)(packed >> 4u);
    const float scale = q35o_decode_e4m3(scales[c / 16]) * s2;
    w[c] = q35o_decode_e2m1(nibble) * scale;
  }
}

/* The engine's decode contract: BF16 activations [m, cols] (rounded before
 * use, src/kernels/cuda/decode_layers.cuh:202,223), the reference matvec loop
 * in fp32 with input_scale = 1 (src/runtime/qwen35x_cuda_backend.cpp:2320),
 * BF16 round-to-nearest-even output [m, rows]
 * (decode_layers.cuh:425).  Also writes the unrounded fp32 result when
 * y_f32 != NULL.  threads <= 1 runs the scalar loop as the reference does;
 * threads > 1 splits output rows over OpenMP threads (same arithmetic). */
Q35O_API void q35o_gemv_bf16(const uint8_t *codes, const uint8_t *scales, float s2, int rows, int cols,
                             const uint16_t *x_bf16, int m, uint16_t *y_bf16, float *y_f32, int threads) {
  const int packed_cols = cols / 2;
  const int scale_cols = cols / 16;
#ifdef _OPENMP
#pragma omp parallel for schedule(static) num_threads(threads > 1 ? threads : 1)
#endif
  for (int row = 0; row < rows; ++row) {
    for (int t = 0; t < m; ++t) {
      float acc = 0.0f;
      const uint16_t *x = x_bf16 + (size_t)t * cols;
      for (int c = 0; c < cols; ++c) {
        const uint8_t packed = codes[(size_t)row * packed_cols + c / 2];
        const uint8_t nibble = (c & 1) == 0 ? (packed & 0x0fu) : (uint8_t)(packed >> 4u);
        const float scale = q35o_decode_e4m3(scales[(size_t)row * scale_cols + c / 16]) * s2;
        acc += q35o_decode_e2m1(nibble) * scale * (bf16_to_f32(x[c]) * 1.0f);
      }
      if (y_f32) y_f32[(size_t)t * rows + row] = acc;
      if (y_bf16) y_bf16[(size_t)t * rows + row] = f32_to_bf16(acc);
    }
  }
}

/* src/runtime/qwen35x_cuda_backend.cpp:742-755: weight -> BF16 (RNE) of
 * e2m1 * (e4m3 * s2). */
Q35O_API void q35o_dequant_weights_bf16(const uint8_t *codes, const uint8_t *scales, float s2, int rows,
                                        int cols, uint16_t *w_bf16) {
  const int packed_cols = cols / 2;
  const int scale_cols = cols / 16;
  for (int row = 0; row < rows; ++row) {
    for (int c = 0; c < cols; ++c) {
      const uint8_t packed = codes[(size_t)row * packed_cols + c / 2];
      const uint8_t nibble = (c & 1) == 0 ? (packed & 0x0fu) : (uint8_t)(packed >> 4u);
      const float scale = q35o_decode_e4m3(scales[(size_t)row * scale_cols + c / 16]) * s2;
      w_bf16[(size_t)row * cols + c] = f32_to_bf16(q35o_decode_e2m1(nibble) * scale);
    }
  }
}

/* ------------------------------------------------------------------ */
/* NVFP4 quantisation                                                  */
/* ------------------------------------------------------------------ */

/* The reference's cuBLASLt activation quantiser, host form
 * (src/runtime/cuda_bench.cu:2221-2235; GPU twins :98-213): per 16-block
 * scale = max(amax/6, 1e-8); scale byte = UE4M3(scale); code = E2M1(x / scale)
 * with the UNROUNDED scale as divisor; even element in the low nibble.
 * Scales are written row-major [rows, cols/16] (swizzle separately).
 * swap_nibbles != 0 applies the reference's swap_fp4_nibbles (:1205-1211), the
 * byte order its GPU kernels emit (:128,:174,:211). */
Q35O_API void q35o_act_quant_reference(const float *x, int rows, int cols, int swap_nibbles, uint8_t *codes,
                                       uint8_t *scales) {
  const int scale_cols = cols / 16;
  for (int r = 0; r < rows; ++r) {
    for (int g = 0; g < scale_cols; ++g) {
      const float *blk = x + (size_t)r * cols + (size_t)g * 16;
      float max_abs = 0.0f;
      for (int i = 0; i < 16; ++i) max_abs = fmaxf(max_abs, fabsf(blk[i]));
      const float scale = fmaxf(max_abs / 6.0f, 1.0e-8f);
      scales[(size_t)r * scale_cols + g] = q35o_encode_ue4m3(scale);
      for (int i = 0; i < 16; i += 2) {
        const uint8_t n0 = q35o_encode_e2m1(blk[i] / scale);
        const uint8_t n1 = q35o_encode_e2m1(blk[i + 1] / scale);
        const uint8_t byte = swap_nibbles ? (uint8_t)((n0 << 4) | n1) : (uint8_t)(n0 | (n1 << 4));
        codes[((size_t)r * cols + (size_t)g * 16 + i) / 2] = byte;
      }
    }
  }
}

/* Largest scale byte the engine emits.  The reference's encoder can return
 * 0x7f (which its decoder reads as 480, cuda_bench.cu:1935-1949); the
 * tensor-core UE4M3 format reads 0x7f as NaN, so the engine's recipe
 * saturates at 0x7e = 448. */
#define Q35O_MAX_SCALE_BYTE 0x7e

/* Per-tensor scale of the engine's NVFP4 recipe: amax / (6 * 448), 1 when the
 * tensor is all zero. */
Q35O_API float q35o_global_scale_from_amax(float amax) {
  if (!(amax > 0.0f)) return 1.0f;
  return amax / (6.0f * 448.0f);
}

/* The engine's NVFP4 recipe (same codecs as the reference, two-level scale
 * as in the ModelOpt weight format, src/weights/modelopt_nvfp4.cpp:105-136;
 * divisor = decoded block scale as the reference's SM120 packer,
 * src/runtime/cuda_bench.cu:518-541):
 *   g  = global_scale (> 0), or amax(X)/(6*448) when global_scale <= 0
 *   per 16-block: t = amax_blk / 6
 *                 sb = min(UE4M3(max(t / g, 1e-8)), 0x7e)
 *                 d  = max(decode(sb), 1e-8) * g
 *                 code_i = E2M1(x_i / d), element 2j in the low nibble
 * x is BF16 when x_is_bf16 != 0, else fp32.  Scales are written row-major
 * [rows, cols/16]; returns g through *g_out. */
Q35O_API void q35o_quantize_nvfp4(const void *x, int x_is_bf16, int rows, int cols, float global_scale,
                                  uint8_t *codes, uint8_t *scales, float *g_out) {
  const int scale_cols = cols / 16;
  const float *xf = (const float *)x;
  const uint16_t *xh = (const uint16_t *)x;
  float g = global_scale;
  if (!(g > 0.0f)) {
    float amax = 0.0f;
    const size_t n = (size_t)rows * cols;
    for (size_t i = 0; i < n; ++i) {
      const float v = x_is_bf16 ? bf16_to_f32(xh[i]) : xf[i];
      amax = fmaxf(amax, fabsf(v));
    }
    g = q35o_global_scale_from_amax(amax);
  }
  *g_out = g;
  for (int r = 0; r < rows; ++r) {
    for (int b = 0; b < scale_cols; ++b) {
      float blk[16];
      float max_abs = 0.0f;
      for (int i = 0; i < 16; ++i) {
        const size_t idx = (size_t)r * cols + (size_t)b * 16 + i;
        blk[i] = x_is_bf16 ? bf16_to_f32(xh[idx]) : xf[idx];
        max_abs = fmaxf(max_abs, fabsf(blk[i]));
      }
      const float t = max_abs / 6.0f;
      uint8_t sb = q35o_encode_ue4m3(fmaxf(t / g, 1.0e-8f));
      if (sb > Q35O_MAX_SCALE_BYTE) sb = Q35O_MAX_SCALE_BYTE;
      scales[(size_t)r * scale_cols + b] = sb;
      const float d = fmaxf(q35o_decode_e4m3(sb), 1.0e-8f) * g;
      for (int i = 0; i < 16; i += 2) {
        const uint8_t n0 = q35o_encode_e2m1(blk[i] / d);
        const uint8_t n1 = q35o_encode_e2m1(blk[i + 1] / d);
        codes[((size_t)r * cols + (size_t)b * 16 + i) / 2] = (uint8_t)(n0 | (n1 << 4));
      }
    }
  }
}

/* ------------------------------------------------------------------ */
/* W4A4 projection                                                     */
/* ------------------------------------------------------------------ */

/* src/runtime/cuda_bench.cu:872-884: expected value of a W4A4 projection,
 *   sum_k (double)( e2m1(w) * e4m3(ws) * (e2m1(a) * e4m3(as)) * input_scale * s2 )
 * with each term evaluated in fp32 in that order and accumulated in double.
 * a_codes [m, cols/2], a_scales row-major [m, cols/16], input_scale = the
 * activation tensor's global scale g.  Output rows [n_begin, n_end) of every
 * token: c_f32 / c_bf16 are [m, n_end - n_begin].  The reference asserts
 * nothing at this boundary; pinned through its cuBLASLt bridge's output on the
 * GPU box (see the file header). */
Q35O_API void q35o_gemm_w4a4(const uint8_t *w_codes, const uint8_t *w_scales, float s2, int rows, int cols,
                             const uint8_t *a_codes, const uint8_t *a_scales, float input_scale, int m,
                             int n_begin, int n_end, float *c_f32, uint16_t *c_bf16, int threads) {
  const int packed_cols = cols / 2;
  const int scale_cols = cols / 16;
  const int n_out = n_end - n_begin;
  (void)rows;
#ifdef _OPENMP
#pragma omp parallel for schedule(static) num_threads(threads > 1 ? threads : 1)
#endif
  for (int row = n_begin; row < n_end; ++row) {
    for (int t = 0; t < m; ++t) {
      double expected = 0.0;
      for (int k = 0; k < cols; ++k) {
        const uint8_t wp = w_codes[(size_t)row * packed_cols + k / 2];
        const uint8_t wn = (k & 1) == 0 ? (wp & 0x0fu) : (uint8_t)(wp >> 4u);
        const uint8_t ap = a_codes[(size_t)t * packed_cols + k / 2];
        const uint8_t an = (k & 1) == 0 ? (ap & 0x0fu) : (uint8_t)(ap >> 4u);
        const int grp = k / 16;
        const float input_quantized = q35o_decode_e2m1(an) * q35o_decode_e4m3(a_scales[(size_t)t * scale_cols + grp]);
        const float weight_scale = q35o_decode_e4m3(w_scales[(size_t)row * scale_cols + grp]);
        expected += (double)(q35o_decode_e2m1(wn) * weight_scale * input_quantized * input_scale * s2);
      }
      const float out = (float)expected;
      if (c_f32) c_f32[(size_t)t * n_out + (row - n_begin)] = out;
      if (c_bf16) c_bf16[(size_t)t * n_out + (row - n_begin)] = f32_to_bf16(out);
    }
  }
}

/* W4A16 reference of a full [m, rows] projection with fp32 activations,
 * used to time the reference's CPU path (cuda_bench.cu:2091-2100 per row)
 * over all host cores: rows are split over OpenMP threads, arithmetic as
 * q35o_matvec_f32. */
Q35O_API void q35o_matvec_f32_omp(const uint8_t *codes, const uint8_t *scales, float input_scale, float s2,
                                  int rows, int cols, const float *x, float *y, int threads) {
#ifdef _OPENMP
#pragma omp parallel for schedule(static) num_threads(threads > 1 ? threads : 1)
#endif
  for (int row = 0; row < rows; ++row) {
    q35o_matvec_f32(codes, scales, input_scale, s2, rows, cols, x, row, row + 1, y + row);
  }
}

Q35O_API int q35o_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Dequantise a whole row (exposed for tests of the codecs on real tensors). */
Q35O_API void q35o_dequant_row_f32(const uint8_t *codes, const uint8_t *scales, float s2, int cols, float *w) {
  dequant_row(codes, scales, s2, cols, w);
}
