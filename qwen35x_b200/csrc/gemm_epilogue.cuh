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
  // The NVFP4 output may be a column range of a wider activation (a row shard of the gate/up weight writing its
  // part of [m, intermediate]): q_codes already points at the range's first code byte, q_ld is the byte stride
  // between rows, q_slot0 the first scale column of the range and q_slots the scale columns of the whole width.
  int q_ld = 0;
  int q_slot0 = 0;
  // Gather fused into the stores (multi-GPU, rows sharded): every BF16 store is repeated into the same place of
  // the full output matrix on each other rank (peer_c[i], plain peer-memory stores over NVLink), and when the whole
  // grid has stored, its last CTA writes `epoch` into this rank's flag slot on every rank (peer_flag[i]).
  static constexpr int kMaxPeers = 7;
  int n_peers = 0;
  int forward_rows = 0;  // host-checked: ldc, the column count and every matrix base allow 32-byte row pieces
  __nv_bfloat16 * peer_c[kMaxPeers] = {};
  unsigned int * peer_flag[kMaxPeers] = {};
  unsigned int * done_counter = nullptr;   // this rank's, zero between launches
  unsigned int epoch = 0;
  // epoch == 0: the epoch is this rank's own send count, kept in device memory (send_seq) and advanced by the
  // launch itself, so that a captured launch can be replayed: replay k signals k where the receivers' k-th wait
  // expects it.
  unsigned int * send_seq = nullptr;
};

__device__ __forceinline__ void st_global_v8(void * p, const uint32_t (&v)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]),
               "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}

// A warp that has just stored 32 rows x COLS BF16 columns of the local matrix (one row per lane) sends them to the
// other ranks as whole lines: it reads its rows back from L2 with four lanes per 128 bytes and repeats them with the
// same lane mapping, so every store instruction covers whole 128-byte lines of a few rows, the unit NVLink moves
// well, instead of thirty-two 32-byte pieces of thirty-two rows.  Only taken when the host found ldc, n and the
// matrix bases to be multiples of 16 elements (GemmEpilogue::forward_rows); otherwise every lane repeats its own
// stores on the peers.  Pieces past column n or row m are skipped.
template <int COLS>
__device__ __forceinline__ void gemm_forward_rows_to_peers(const GemmEpilogue & ep, const __nv_bfloat16 * c, int ldc,
                                                           int row0, int m, int col0, int n, int lane) {
  constexpr int kPieces = COLS / 16;  // 32-byte pieces per row
  __threadfence_block();              // the lanes' own stores, before other lanes read them
  __syncwarp();
  // all loads first, then all stores: a warp issues in order, so a store waiting for its load would hold back the
  // loads behind it
  uint32_t v[kPieces][8];
#pragma unroll
  for (int it = 0; it < kPieces; ++it) {
    const int idx = it * 32 + lane;
    const int row = row0 + idx / kPieces;
    const int col = col0 + (idx % kPieces) * 16;
#pragma unroll
    for (int j = 0; j < 8; ++j) v[it][j] = 0u;
    if (row < m && col + 16 <= n) {
      const __nv_bfloat16 * src = c + static_cast<size_t>(row) * ldc + col;
      asm volatile("ld.global.cg.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                   : "=r"(v[it][0]), "=r"(v[it][1]), "=r"(v[it][2]), "=r"(v[it][3]), "=r"(v[it][4]), "=r"(v[it][5]),
                     "=r"(v[it][6]), "=r"(v[it][7])
                   : "l"(src));
    }
  }
#pragma unroll
  for (int it = 0; it < kPieces; ++it) {
    const int idx = it * 32 + lane;
    const int row = row0 + idx / kPieces;
    const int col = col0 + (idx % kPieces) * 16;
    if (row < m && col + 16 <= n) {
      const size_t off = static_cast<size_t>(row) * ldc + col;
      _Pragma("unroll") for (int i = 0; i < GemmEpilogue::kMaxPeers; ++i) if (i < ep.n_peers) st_global_v8(ep.peer_c[i] + off, v[it]);
    }
  }
}

// End of a gathering GEMM kernel; every thread of the CTA calls it after its last output store.
// A CTA that ran no tiles because an earlier error is recorded (`ran` false) counts itself but the flags are not
// written then: the other ranks' bounded waits expire and record the failure on their side too.
__device__ __forceinline__ void gemm_signal_peers(const GemmEpilogue & ep, bool ran) {
  if (ep.done_counter == nullptr) return;
  __threadfence_system();  // this thread's stores, local and remote, before anything that follows
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(ep.done_counter, 1u);
    if (prev == gridDim.x * gridDim.y * gridDim.z - 1) {  // every other CTA fenced its stores before it counted itself
      *ep.done_counter = 0u;
      __threadfence_system();
      unsigned int epoch = ep.epoch;
      if (epoch == 0u && ep.send_seq != nullptr) {
        epoch = *ep.send_seq + 1u;  // only this thread of the whole grid gets here
        *ep.send_seq = epoch;
      }
      if (ran) {
        _Pragma("unroll") for (int i = 0; i < GemmEpilogue::kMaxPeers; ++i) if (i < ep.n_peers) *reinterpret_cast<volatile unsigned int *>(ep.peer_flag[i]) = epoch;
      }
    }
  }
}


// silu(g) * u with the hardware exponential and reciprocal (a few fp32 ulp, far inside the BF16 rounding that follows)
__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t *>(&h);
}

// r: 32 accumulator columns starting at global column col0 (a multiple of 32) of row `row`; n = accumulator columns
// of the whole problem (weight rows); g = the activation tensor's scale.
// to_peers: also repeat every store on the other ranks (one 32-byte piece per lane); a caller that forwards whole
// rows afterwards (gemm_forward_rows_to_peers) passes false.
// q_g: value of *ep.q_g (the NVFP4 output's per-tensor scale), read once per warp by the caller: thousands of warps
// loading that one word per chunk would queue up on a single L2 slice.
__device__ __forceinline__ void gemm_store_chunk32(const uint32_t (&r)[32], int row, int col0, int n, float g,
                                                   const GemmEpilogue & ep, __nv_bfloat16 * __restrict__ c, int ldc,
                                                   bool to_peers = true, float q_g = 1.0f) {
  if (col0 >= n) return;  // a chunk wholly past the last column of a partial tile
  const int n_peers = to_peers ? ep.n_peers : 0;
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
      const uint32_t sb = quantize_block<kEngine>(v, q_g, false, packed);
      *reinterpret_cast<uint2 *>(ep.q_codes + static_cast<size_t>(row) * ep.q_ld + (col0 >> 2)) = packed;
      ep.q_scales[tiled_scale_offset(row, ep.q_slot0 + (col0 >> 5), ep.q_slots)] = static_cast<uint8_t>(sb);
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
      _Pragma("unroll") for (int i = 0; i < GemmEpilogue::kMaxPeers; ++i) if (i < n_peers) st_global_v8(ep.peer_c[i] + static_cast<size_t>(row) * ldc + (col0 >> 1), p);
    } else {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (col0 + 16 * j + 8 + i < n) {
            const float gv = __uint_as_float(r[16 * j + i]) * alpha;
            const float uv = __uint_as_float(r[16 * j + 8 + i]) * alpha_up;
            const __nv_bfloat16 o = __float2bfloat16_rn(silu_mul(gv, uv));
            dst[8 * j + i] = o;
            _Pragma("unroll") for (int pi = 0; pi < GemmEpilogue::kMaxPeers; ++pi) if (pi < n_peers) ep.peer_c[pi][static_cast<size_t>(row) * ldc + (col0 >> 1) + 8 * j + i] = o;
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
      _Pragma("unroll") for (int i = 0; i < GemmEpilogue::kMaxPeers; ++i) if (i < n_peers) st_global_v8(ep.peer_c[i] + static_cast<size_t>(row) * ldc + col0 + v * 16, p);
    }
  } else {
#pragma unroll
    for (int e = 0; e < 32; ++e) {
      if (col0 + e < n) {
        const float rv = res != nullptr ? __bfloat162float(res[e]) : 0.0f;
        const __nv_bfloat16 o = __float2bfloat16_rn(fmaf(__uint_as_float(r[e]), alpha, rv));
        dst[e] = o;
        _Pragma("unroll") for (int pi = 0; pi < GemmEpilogue::kMaxPeers; ++pi) if (pi < n_peers) ep.peer_c[pi][static_cast<size_t>(row) * ldc + col0 + e] = o;
      }
    }
  }
}

}  // namespace q35b
