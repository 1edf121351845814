// Streaming W4A16 decode projection for sm_100a: one persistent launch walks a
// work list of (projection, 128-row block) tiles; M = 1..8 tokens.
//
// Replaces the per-phase matvec loops of the reference's persistent decode
// kernel (src/kernels/cuda/decode_kernel.cuh:58-84 calling nvfp4_row_dot,
// src/kernels/cuda/decode_layers.cuh:200-261) for the projections of a step.
//
// Data movement (what bounds the kernel): per 256-column K step a tile moves
//   16 KB of codes   128 rows x 128 B, cp.async.bulk.tensor.2d, 128B swizzle,
//                    straight from the checkpoint-order [rows, K/2] matrix
//    2 KB of scales  four 512-byte 128x4 tiles, cp.async.bulk
// into a shared-memory ring (mbarrier full/empty pairs), so each CTA keeps
// (stages x 18 KB) in flight regardless of how its consumer warps are doing.
//
// Arithmetic (kept off the critical path): one consumer warp per 16 rows of the tile.  Two shapes of CTA: eight
// consumer warps and half of an SM's shared memory, two CTAs per SM, so that one CTA's stalls (change of
// projection, tile hand-over, epilogue) run under the other's arithmetic; or, when the activations need more room,
// sixteen consumer warps in one CTA per SM, two per row group splitting every K step (their partial sums
// meet in shared memory at the end of the tile).  ldmatrix pulls 8 E2M1 codes per lane per register,
// cvt.rn.f16x2.e2m1x2 (the sm_100a FP4 converter) turns every byte into two
// exact fp16 values, and mma.sync m16n8k16 forms the 16-element block dot
// products against fp16 activations; the eight MMA columns are (half h of the
// 32-code chunk, token m<4), so one MMA pair yields, in each lane, the dot
// product of exactly the block that lane loaded: no cross-lane data movement.
// The E4M3 block scale multiplies that block dot in fp32 and accumulates.
// Five to eight tokens use a dense mapping instead: the eight MMA columns are the tokens, every k-slot is used,
// and the block scales are folded exactly into the fp16 weight operand, so the MMAs accumulate straight over K.
// Activations are converted BF16 -> fp16 per token with an exact power-of-two scale taken from the token's amax:
// a dedicated warp bulk-copies the raw rows of the next projection into one of two buffers (under the tiles of the
// projection before), and the consumer warps convert them in place when they get there, each a slice of
// one token, meeting twice on bounded mbarriers (amax known, conversion done).
//
// All waits are bounded; on expiry a code is written to the batch's status word.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <vector>

#include "engine.h"
#include "nvfp4_codec.cuh"

namespace q35b {
namespace {

constexpr int kTileRows = 128;
constexpr int kStepBytes = 128;                 // 256 codes per row per K step
constexpr int kCodesBytes = kTileRows * kStepBytes;
constexpr int kScaleBytes = 4 * 512;
constexpr int kStageBytes = kCodesBytes + kScaleBytes;
constexpr int kRowGroups = 8;                   // 16-row groups per tile
// Two shapes of CTA.  KS = 1: eight consumer warps, one per 16-row group, each taking the whole K step; 112 KB of
// shared memory, so that two CTAs share an SM and each one's stalls (change of projection, tile hand-over, epilogue)
// run under the other's arithmetic.  KS = 2: sixteen consumer warps, two per row group splitting every K step (their
// partial sums meet in shared memory at the end of a tile); one CTA per SM with all of its shared memory, for
// activations too large for the first shape.
__host__ __device__ constexpr int consumer_warps(int ks) { return kRowGroups * ks; }
__host__ __device__ constexpr int cta_threads(int ks) { return (2 + consumer_warps(ks)) * 32; }  // warp 0 producer, warp 1 activation copies
__host__ __device__ constexpr int ctas_per_sm(int ks) { return ks == 1 ? 2 : 1; }
__host__ __device__ constexpr int smem_budget(int ks) { return ks == 1 ? 112 * 1024 : 227 * 1024; }
// floats of the buffer in which the two warps of a row group meet (none when a warp takes the whole K step)
__host__ __device__ constexpr int red_floats(int ks, int mt) { return ks == 2 ? 2 * kRowGroups * 32 * 4 * mt : 0; }
constexpr int kMaxTilesInSmem = 64;             // tile descriptors staged per CTA
constexpr int kMaxStages = 8;
constexpr int kZeroHalfs = 320;                 // covers the 8 chunk offsets (32 halfs apart) of a K step + a bank shift
constexpr uint32_t kWaitLimit = 1u << 22;
// fp16 elements of padding between tokens.  Up to four tokens: consecutive tokens sit 32 bytes apart modulo the
// 128-byte bank window; five to eight tokens (the dense mapping below): 64 bytes apart, because there the eight lanes
// served together by a 128-bit load read 64 contiguous bytes of each of two tokens.
constexpr int kDenseFrom = 5;  // token count from which the dense MMA mapping (template MT = 2) is used; measured: with
                               // two to four tokens the (block, token) mapping is 4-7 % faster
__host__ __device__ constexpr int x_pad(int m_tokens) { return m_tokens >= kDenseFrom ? 32 : 16; }

enum Epilogue : int { kEpiPlain = 0, kEpiGateUp = 1 };

enum StatusCode : unsigned { kProducerWait = 11, kPrepWait = 12, kConsumerWait = 13, kConsumerXWait = 14, kDependencyWait = 15 };

struct alignas(128) GemvItem {
  CUtensorMap tmap;              // codes [rows, K/2], box 128 rows x 128 bytes, 128B swizzle
  const uint8_t * scales_tiled;
  const __nv_bfloat16 * x;       // [m, K]
  __nv_bfloat16 * y;             // [m, rows]
  int rows;
  int k;
  int k_steps;                   // K / 256
  float s2;
};

// Everything a CTA needs to know about one tile, staged in shared memory at kernel start so that no role chases
// pointers through global memory at a tile boundary.
struct alignas(16) GemvTile {
  int item;
  int row_block;
  int k;
  int k_steps;
  int rows;
  float s2;
  const uint8_t * scales;        // tiled scales of this row block
  const uint8_t * codes;         // first code byte of this row block
  const __nv_bfloat16 * x;
  __nv_bfloat16 * y;
  const __nv_bfloat16 * residual;  // NULL or [m, rows]: added before the BF16 rounding
  float s2_up;                     // gate/up weight: weight_scale_2 of the up rows
  int epilogue;                    // kEpiPlain | kEpiGateUp
  int wait_item;                   // -1, or the item whose output this item's activations are
  unsigned int wait_count;         // completions that item reports per run (its tiles x 8 storing warps)
  int signal;                      // nonzero: another item waits for this one, count every stored tile part
};

__device__ __forceinline__ uint32_t smem_u32(const void * p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t limit) {
  for (uint32_t i = 0; i < limit; ++i) {
    uint32_t ok;
    asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap * map, uint32_t bar, int x, int y) {
  asm volatile(
    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
    "l"(map), "r"(bar), "r"(x), "r"(y)
    : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void * src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t & r0, uint32_t & r1, uint32_t & r2, uint32_t & r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}

// Four bytes of E2M1 pairs -> four fp16x2 registers (low nibble in the low half): exact.
__device__ __forceinline__ void e2m1x8_to_f16(uint32_t w, uint32_t (&h)[4]) {
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
      : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
      : "r"(w));
}

// d = a * b (+ c): fp16 operands, fp32 accumulate.
__device__ __forceinline__ void mma_f16_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
  asm volatile(
    "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
    : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
    : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}
__device__ __forceinline__ void mma_f16_acc(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                            uint32_t b1) {
  asm volatile(
    "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
    : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
    : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Product of two fp16x2 registers.
__device__ __forceinline__ uint32_t hmul2_bits(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// Unsigned E4M3 byte (bit 7 clear) -> fp32 (0x7f = 480, subnormals exact): the byte placed at bit 20 is the
// value scaled by 2^-120.  The shift is written as a multiply so that it issues on the FMA pipe.
__device__ __forceinline__ float ue4m3_to_f32(uint32_t byte) {
  return __uint_as_float(byte * 0x100000u) * 0x1p120f;
}

// MT = number of 4-token groups (1 for M <= 4, 2 for M <= 8).
template <int MT, int KS>
__global__ void __launch_bounds__(cta_threads(KS), ctas_per_sm(KS))
gemv_w4a16_stream_kernel(const GemvItem * __restrict__ items, const GemvTile * __restrict__ tiles,
                         const int * __restrict__ cta_begin, int m_tokens, const __nv_bfloat16 * x_override,
                         __nv_bfloat16 * y_override, int stages, int x_buf_halfs, int xs_buf_floats,
                         int x_bufs, unsigned long long * item_done,
                         int counted_items, unsigned int * status, uint32_t wait_limit, unsigned int wait_extra) {
  constexpr bool kDense = (MT == 2);  // five to eight tokens: dense MMA mapping
  constexpr int kConsumerWarps = consumer_warps(KS);
  constexpr int kConsumerShift = KS == 2 ? 4 : 3;  // log2(kConsumerWarps)
  constexpr int kThreads = cta_threads(KS);
  constexpr int kKSplit = KS;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment for the swizzled code tiles; pointer arithmetic on the __shared__ array (rather than an
  // integer round trip) keeps every later access a shared-memory access for the compiler.
  uint8_t * ring = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  __half * xbuf = reinterpret_cast<__half *>(ring + stages * kStageBytes);        // x_bufs (1 or 2) buffers of x_buf_halfs
  __half * zeros = xbuf + x_bufs * x_buf_halfs;                                   // kZeroHalfs of 0.0, 128-byte aligned
  float * xsbuf = reinterpret_cast<float *>(zeros + kZeroHalfs);                   // 2 buffers of xs_buf_floats (1/scale)
  float * red = xsbuf + 2 * xs_buf_floats;                                         // 2 x [8 row groups][32 lanes][4*MT]
  GemvTile * stile = reinterpret_cast<GemvTile *>(red + red_floats(KS, MT));
  uint64_t * bars = reinterpret_cast<uint64_t *>(stile + kMaxTilesInSmem);
  // bars: full[kMaxStages], empty[kMaxStages], xfull[2], xempty[2], red_full[2], red_free[2], conv[2]
  uint64_t * full = bars;
  uint64_t * empty = bars + kMaxStages;
  uint64_t * xfull = bars + 2 * kMaxStages;
  uint64_t * xempty = xfull + 2;
  uint64_t * red_full = xempty + 2;
  uint64_t * red_free = red_full + 2;
  uint64_t * conv = red_free + 2;                                                  // consumers: amax known, conversion done
  uint32_t * amax_s = reinterpret_cast<uint32_t *>(conv + 2);                      // [2][8] per-token amax bits, by item parity

  // Programmatic dependent launch: the next kernel of the stream may start on an SM as soon as this kernel's CTA has
  // left it, and this kernel may start under the tail of the previous one.  Weights, tile descriptors and tensor
  // maps are constant for the life of the work list, so the producer streams them at once; whatever an earlier
  // kernel may have written (activations, residuals, completion counts) and every output store comes after
  // griddepcontrol.wait, which returns when all earlier work of the stream is complete and visible.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tile_begin = cta_begin[blockIdx.x];
  const int n_tiles = cta_begin[blockIdx.x + 1] - tile_begin;

  if (threadIdx.x == 0) {
    for (int i = 0; i < stages; ++i) {
      mbar_init(smem_u32(full + i), 1);
      mbar_init(smem_u32(empty + i), kConsumerWarps);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(xfull + i), 1);
      mbar_init(smem_u32(xempty + i), kConsumerWarps);
      mbar_init(smem_u32(red_full + i), kRowGroups);
      mbar_init(smem_u32(red_free + i), kRowGroups);
    }
    for (int i = 0; i < 2; ++i) mbar_init(smem_u32(conv + i), kConsumerWarps);
    for (int i = 0; i < 16; ++i) amax_s[i] = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // stage this CTA's tile descriptors; clear the zero region
  for (int i = threadIdx.x; i < kZeroHalfs / 2; i += kThreads) reinterpret_cast<uint32_t *>(zeros)[i] = 0u;
  {
    const int n_stage = min(n_tiles, kMaxTilesInSmem);
    constexpr int kWords = sizeof(GemvTile) / 16;
    const uint4 * src = reinterpret_cast<const uint4 *>(tiles + tile_begin);
    uint4 * dst = reinterpret_cast<uint4 *>(stile);
    for (int i = threadIdx.x; i < n_stage * kWords; i += kThreads) dst[i] = __ldg(src + i);
  }
  __syncthreads();
  auto tile_at = [&](int i) -> const GemvTile * { return i < kMaxTilesInSmem ? stile + i : tiles + tile_begin + i; };

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int ti = 0; ti < n_tiles && ok; ++ti) {
        const GemvTile * tile = tile_at(ti);
        const CUtensorMap * tmap = &items[tile->item].tmap;
        const int k_steps = tile->k_steps;
        const uint8_t * sc = tile->scales;
        const int row0 = tile->row_block * kTileRows;
        for (int ks = 0; ks < k_steps; ++ks) {
          if (!mbar_wait(smem_u32(empty + stage), phase ^ 1, wait_limit)) {
            atomicCAS(status, 0u, kProducerWait);
            ok = false;
            break;
          }
          const uint32_t bar = smem_u32(full + stage);
          uint8_t * dst = ring + stage * kStageBytes;
          mbar_expect_tx(bar, kStageBytes);
          tma_load_2d(smem_u32(dst), tmap, bar, ks * kStepBytes, row0);
          bulk_load(smem_u32(dst + kCodesBytes), sc + static_cast<size_t>(ks) * kScaleBytes, kScaleBytes, bar);
          if (++stage == stages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ activation copies
    // Bulk-copies the raw BF16 activations of the next projection into one of the (one or two) activation buffers,
    // token rows padded apart; the consumers convert them to scaled fp16 in place.
    auto next_run = [&](int ti, int prev) {  // first tile index >= ti whose projection differs from `prev`
      while (ti < n_tiles && tile_at(ti)->item == prev) ++ti;
      return ti;
    };
    // An item that runs after another one may read its activations only when every storing warp of every tile of
    // that item has counted itself in item_done (stores fenced before the count).
    auto dependency_met = [&](const GemvTile * tl, bool block) -> bool {
      if (tl->wait_item < 0) return true;
      int met = 0;
      if (lane == 0) {
        const volatile unsigned long long * cnt = item_done + tl->wait_item;
        // a sixteenth of the budget of the barrier waits: when a dependency cannot be met this poll gives up first and
        // its code (the first one recorded stays) names the cause; the roles waiting on this warp follow
        for (uint32_t i = 0; i < max(wait_limit >> 4, 1u); ++i) {
          if (*cnt >= tl->wait_count + wait_extra) {
            met = 1;
            break;
          }
          if (!block) break;
          __nanosleep(32);
        }
      }
      met = __shfl_sync(0xffffffffu, met, 0);
      if (met) {
        __threadfence();
        asm volatile("fence.proxy.async;" ::: "memory");  // the bulk copy that follows reads what other SMs stored
      }
      return met != 0;
    };
    asm volatile("griddepcontrol.wait;" ::: "memory");
    int proc_ti = next_run(0, -1);
    uint32_t xi = 0;
    while (proc_ti < n_tiles) {
      // The raw BF16 rows of the next projection go straight into the (padded) buffer the consumers will read; the
      // sixteen consumer warps convert them in place when they reach the item.  (One warp converting eight tokens
      // takes several microseconds per item, and a CTA changes item at almost every tile of a 4B-class step.)
      // With two buffers the copy runs under the tiles of the item before.
      const GemvTile * tile = tile_at(proc_ti);
      if (!dependency_met(tile, true)) {
        if (lane == 0) atomicCAS(status, 0u, kDependencyWait);
        break;
      }
      const int buf = (x_bufs == 2) ? (xi & 1) : 0;
      const uint32_t xphase = (x_bufs == 2) ? ((xi >> 1) & 1) : (xi & 1);
      if (!mbar_wait(smem_u32(xempty + buf), xphase ^ 1, wait_limit)) {
        if (lane == 0) atomicCAS(status, 0u, kPrepWait);
        break;
      }
      if (lane == 0) {
        const int k = tile->k;
        const uint32_t bar = smem_u32(xfull + buf);
        const __nv_bfloat16 * x = x_override != nullptr ? x_override : tile->x;
        __half * xb = xbuf + buf * x_buf_halfs;
        mbar_expect_tx(bar, static_cast<uint32_t>(m_tokens) * k * 2u);
        for (int token = 0; token < m_tokens; ++token) {
          bulk_load(smem_u32(xb + static_cast<size_t>(token) * (k + x_pad(m_tokens))), x + static_cast<size_t>(token) * k,
                    static_cast<uint32_t>(k) * 2u, bar);
        }
      }
      ++xi;
      proc_ti = next_run(proc_ti + 1, tile->item);
    }
  } else {
    // ------------------------------------------------------------ consumers
    const int cw = warp - 2;           // 0..15
    const int rg = cw & 7;             // row group: tile rows 16*rg .. 16*rg+15
    const int kh = cw >> 3;            // which half of every K step (chunk pairs 2*kh, 2*kh+1)
    const int g = lane >> 2;
    const int t = lane & 3;
    // B-operand role of this lane: MMA column g = (half hB, token mB); it feeds k-slots owned by quad thread t.
    const int hB = g >> 2;
    const int mB = g & 3;
    const bool b_owner = (t >> 1) == hB;
    // D role: this lane receives block half hD = t >> 1, tokens 2*(t&1), 2*(t&1)+1 for rows g and g+8.
    const int hD = t >> 1;
    // Dense mapping (five to eight tokens): byte selectors that pull the scale of this lane's block (block
    // 2*cq + hD of a 4-block scale word) into both halves of a register.
    const uint32_t dense_sel[2] = {0x4040u | (static_cast<uint32_t>(hD) * 0x0101u),
                                   0x4040u | (static_cast<uint32_t>(2 + hD) * 0x0101u)};
    // ldmatrix row address of this lane: matrix mi = lane >> 3 -> rows 8*(mi&1).., chunk offset mi >> 1
    const int lm_row = 16 * rg + 8 * ((lane >> 3) & 1) + (lane & 7);
    const int lm_chunk = lane >> 4;
    const uint32_t lm_row_off = lm_row * kStepBytes;
    const int lm_xor = lm_row & 7;
    // scale word address pieces: row r -> (r % 32) * 16 + (r / 32) * 4 inside a 512-byte tile
    const int r0 = 16 * rg + g;
    const int sc_off0 = (r0 & 31) * 16 + (r0 >> 5) * 4;
    const int x_lane_off = 16 * hB + 8 * (t & 1);
    // The eight lanes served together by a 128-bit load hold two tokens of one block half: their activations fill a
    // 64-byte window of the 128-byte bank span (buffers are 128-byte aligned, tokens 32 bytes apart modulo 128).
    // Lanes that must feed zeros read them from the other 64 bytes of the span.
    const __half * zsrc = zeros + (m_tokens == 1 ? 48 : ((64 * (mB >> 1) + 32 * hB + 64) & 127) >> 1);

    int stage = 0;
    uint32_t phase = 0;
    uint32_t xi = 0;
    int prev_item = -1;
    int buf = 0;
    bool ok = true;
    for (int ti = 0; ti < n_tiles && ok; ++ti) {
      const GemvTile * tile = tile_at(ti);
      if (tile->item != prev_item) {
        if (prev_item >= 0) {
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // a bulk copy overwrites what this warp converted
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(xempty + buf));
        }
        prev_item = tile->item;
        buf = (x_bufs == 2) ? (xi & 1) : 0;
        if (!mbar_wait(smem_u32(xfull + buf), (x_bufs == 2) ? ((xi >> 1) & 1) : (xi & 1), wait_limit)) {
          if (lane == 0) atomicCAS(status, 0u, kConsumerXWait);
          ok = false;
          break;
        }
        if (xi == 0) asm volatile("griddepcontrol.wait;" ::: "memory");  // returns at once: the activation warp has waited
        {
          // The raw BF16 rows of this item have landed in the buffer: the sixteen consumer warps turn them into
          // scaled fp16 in place.  With T = 1, 2, 4 or 8 token slots (the power of two that holds the tokens), warp
          // cw takes token cw % T and slice cw / T of its columns; the warps of a token agree on its amax through
          // shared memory.  Both meeting points are bounded mbarrier waits.
          const int tshift = m_tokens > 4 ? 3 : (m_tokens > 2 ? 2 : (m_tokens > 1 ? 1 : 0));
          const int ctoken = cw & ((1 << tshift) - 1);
          const int khalf = tile->k >> (kConsumerShift - tshift);  // columns per slice
          const bool live = ctoken < m_tokens;
          __half * crow = xbuf + buf * x_buf_halfs + static_cast<size_t>(ctoken) * (tile->k + x_pad(m_tokens)) + (cw >> tshift) * khalf;
          const uint32_t par = xi & 1;
          uint32_t amax_bits = 0;
          if (live) {
            for (int i = lane * 8; i < khalf; i += 256) {
              const uint4 q = *reinterpret_cast<const uint4 *>(crow + i);
              const uint32_t r[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                amax_bits = max(amax_bits, (r[j] << 16) & 0x7fffffffu);
                amax_bits = max(amax_bits, r[j] & 0x7fff0000u);
              }
            }
          }
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) amax_bits = max(amax_bits, __shfl_xor_sync(0xffffffffu, amax_bits, off));
          if (lane == 0) {
            if (live) atomicMax(amax_s + par * 8 + ctoken, amax_bits);
            mbar_arrive(smem_u32(conv + 0));
          }
          if (!mbar_wait(smem_u32(conv + 0), par, wait_limit)) {
            if (lane == 0) atomicCAS(status, 0u, kConsumerXWait);
            ok = false;
            break;
          }
          if (live) {
            // exact power-of-two scale putting the token's amax in [2^14, 2^15) (exponent field clamped to stay normal):
            // fp16 then holds every BF16 significand exactly down to 2^-28 of the amax
            int e = static_cast<int>(amax_s[par * 8 + ctoken] >> 23);
            e = min(max(e, 16), 254);
            const float scale = __uint_as_float(static_cast<uint32_t>(268 - e) << 23);
            for (int i = lane * 8; i < khalf; i += 256) {
              const uint4 q = *reinterpret_cast<const uint4 *>(crow + i);
              const uint32_t r[4] = {q.x, q.y, q.z, q.w};
              uint32_t out[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const __half2 h = __floats2half2_rn(__uint_as_float(r[j] << 16) * scale, __uint_as_float(r[j] & 0xffff0000u) * scale);
                out[j] = *reinterpret_cast<const uint32_t *>(&h);
              }
              *reinterpret_cast<uint4 *>(crow + i) = make_uint4(out[0], out[1], out[2], out[3]);
            }
            if ((cw >> tshift) == 0 && lane == 0) (xsbuf + buf * xs_buf_floats)[ctoken] = __uint_as_float(static_cast<uint32_t>(e - 14) << 23);
          }
          // the words of the other parity serve the next item: nobody reads them any more, nobody adds to them yet
          if (cw == 0 && lane < 8) amax_s[(par ^ 1) * 8 + lane] = 0u;
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(conv + 1));
          if (!mbar_wait(smem_u32(conv + 1), par, wait_limit)) {
            if (lane == 0) atomicCAS(status, 0u, kConsumerXWait);
            ok = false;
            break;
          }
        }
        ++xi;
      }
      const int k_steps = tile->k_steps;
      const int xstride = tile->k + x_pad(m_tokens);
      const __half * xb = xbuf + buf * x_buf_halfs;
      const float * xs = xsbuf + buf * xs_buf_floats;

      float acc[MT][4];
#pragma unroll
      for (int ts = 0; ts < MT; ++ts)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[ts][i] = 0.0f;

      // B-fragment source of this lane per token group: its slice of the fp16 activations if it owns k-slots of
      // that MMA column, else a zeroed region (same offsets work in both, so the inner loop has no predicates).
      const __half * bsrc[MT];
      int bstep[MT];
      if constexpr (kDense) {
        // dense mapping: MMA column g is token g; this lane feeds the k-slots of its own eight codes of a chunk
        const bool owner = g < m_tokens;
        bsrc[0] = owner ? xb + static_cast<size_t>(g) * xstride + 8 * t : zeros;
        bstep[0] = owner ? 256 : 0;
        bsrc[1] = bsrc[0];
        bstep[1] = 0;
      } else {
#pragma unroll
        for (int ts = 0; ts < MT; ++ts) {
          const int token = 4 * ts + mB;
          const bool owner = b_owner && token < m_tokens;
          bsrc[ts] = owner ? xb + static_cast<size_t>(token) * xstride + x_lane_off : zsrc;
          bstep[ts] = owner ? 256 : 0;
        }
      }
      for (int ks = 0; ks < k_steps; ++ks) {
        if (!mbar_wait(smem_u32(full + stage), phase, wait_limit)) {
          if (lane == 0) atomicCAS(status, 0u, kConsumerWait);
          ok = false;
          break;
        }
        const uint8_t * codes = ring + stage * kStageBytes;
        const uint8_t * sc = codes + kCodesBytes;
        const uint32_t codes_addr = smem_u32(codes) + lm_row_off;

#pragma unroll
        for (int pp = 0; pp < 4 / kKSplit; ++pp) {
          const int pair = (4 / kKSplit) * kh + pp;
          uint32_t r[4];
          ldmatrix_x4(codes_addr + (((2 * pair + lm_chunk) ^ lm_xor) << 4), r[0], r[1], r[2], r[3]);
          if constexpr (kDense) {
            // Five to eight tokens: the eight MMA columns are the tokens, every k-slot is used, and the chunk's two
            // blocks (quad threads 0,1 and 2,3) share one MMA.  Their block scales therefore go into the A operand:
            // E2M1 x E4M3 is exact in fp16 (the scale byte at bit 7 of an fp16 is the scale times 2^-8, 0x7f = 480
            // included; products down to 2^-18 are fp16 subnormals, which multiply and MMA handle exactly), and
            // the MMAs accumulate straight over K in fp32.  The 2^8 is undone in the epilogue.
            const uint32_t sw0 = *reinterpret_cast<const uint32_t *>(sc + pair * 512 + sc_off0);        // row r0, 4 blocks
            const uint32_t sw1 = *reinterpret_cast<const uint32_t *>(sc + pair * 512 + sc_off0 + 128);  // row r0 + 8
#pragma unroll
            for (int cq = 0; cq < 2; ++cq) {
              const int q = 2 * pair + cq;
              uint32_t a_lo[4], a_hi[4];
              e2m1x8_to_f16(r[2 * cq], a_lo);
              e2m1x8_to_f16(r[2 * cq + 1], a_hi);
              const uint32_t s0 = __byte_perm(sw0, 0u, dense_sel[cq]) << 7;  // (scale, scale) as fp16x2, times 2^-8
              const uint32_t s1 = __byte_perm(sw1, 0u, dense_sel[cq]) << 7;
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                a_lo[i] = hmul2_bits(a_lo[i], s0);
                a_hi[i] = hmul2_bits(a_hi[i], s1);
              }
              const uint4 b = *reinterpret_cast<const uint4 *>(bsrc[0] + 32 * q);
              mma_f16_acc(acc[cq], a_lo[0], a_hi[0], a_lo[1], a_hi[1], b.x, b.y);
              mma_f16_acc(acc[cq], a_lo[2], a_hi[2], a_lo[3], a_hi[3], b.z, b.w);
            }
          } else {
          // scale bytes of this pair's 4-block tile (blocks 4*pair .. 4*pair+3 of rows r0 and r0+8): plain byte
          // loads keep the integer pipe free for the FP4 conversions
          const uint8_t * sc0 = sc + pair * 512 + sc_off0 + hD;
#pragma unroll
          for (int cq = 0; cq < 2; ++cq) {
            const int q = 2 * pair + cq;  // 32-code chunk index inside the K step
            uint32_t a_lo[4], a_hi[4];
            e2m1x8_to_f16(r[2 * cq], a_lo);      // rows 0..7 of the warp's 16
            e2m1x8_to_f16(r[2 * cq + 1], a_hi);  // rows 8..15
            // block 2*cq + hD of the 4-block tile; rows r0 and r0 + 8 (128 bytes further)
            const float s0 = ue4m3_to_f32(sc0[2 * cq]);
            const float s1 = ue4m3_to_f32(sc0[2 * cq + 128]);
#pragma unroll
            for (int ts = 0; ts < MT; ++ts) {
              const uint4 b = *reinterpret_cast<const uint4 *>(bsrc[ts] + 32 * q);
              float c[4];
              mma_f16_zero(c, a_lo[0], a_hi[0], a_lo[1], a_hi[1], b.x, b.y);
              mma_f16_acc(c, a_lo[2], a_hi[2], a_lo[3], a_hi[3], b.z, b.w);
              acc[ts][0] = fmaf(c[0], s0, acc[ts][0]);
              acc[ts][1] = fmaf(c[1], s0, acc[ts][1]);
              acc[ts][2] = fmaf(c[2], s1, acc[ts][2]);
              acc[ts][3] = fmaf(c[3], s1, acc[ts][3]);
            }
          }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(empty + stage));
        if (++stage == stages) {
          stage = 0;
          phase ^= 1;
        }
#pragma unroll
        for (int ts = 0; ts < MT; ++ts) bsrc[ts] += bstep[ts];
      }
      if (!ok) break;
      if constexpr (kDense) {
        // the two MMA chains (even and odd chunks) hold partial sums of the same outputs
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[0][i] += acc[1][i];
      }
      constexpr int kGroups = kDense ? 1 : MT;  // float4 groups of sums a lane carries into the epilogue

      // Meet the partner warp's half-K sums in shared memory (double-buffered by tile parity): the kh = 1 warp
      // writes, the kh = 0 warp adds, combines the two block halves (lanes t and t^2) and stores.
      const int rb = ti & 1;
      const uint32_t rphase = (ti >> 1) & 1;
      float * slot = red + ((rb * kRowGroups + rg) * 32 + lane) * 4 * MT;
      if (kKSplit == 2 && kh == 1) {
        if (!mbar_wait(smem_u32(red_free + rb), rphase ^ 1, wait_limit)) {
          if (lane == 0) atomicCAS(status, 0u, kConsumerWait);
          ok = false;
          break;
        }
#pragma unroll
        for (int ts = 0; ts < kGroups; ++ts)
          *reinterpret_cast<float4 *>(slot + 4 * ts) = make_float4(acc[ts][0], acc[ts][1], acc[ts][2], acc[ts][3]);
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(red_full + rb));
      } else {
        if constexpr (kKSplit == 2) {
          if (!mbar_wait(smem_u32(red_full + rb), rphase, wait_limit)) {
            if (lane == 0) atomicCAS(status, 0u, kConsumerWait);
            ok = false;
            break;
          }
#pragma unroll
          for (int ts = 0; ts < kGroups; ++ts) {
            const float4 o = *reinterpret_cast<const float4 *>(slot + 4 * ts);
            acc[ts][0] += o.x;
            acc[ts][1] += o.y;
            acc[ts][2] += o.z;
            acc[ts][3] += o.w;
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(red_free + rb));
        }
        __nv_bfloat16 * y = y_override != nullptr ? y_override : tile->y;
        const int rows = tile->rows;
        const float s2 = tile->s2;
        const int row_a = tile->row_block * kTileRows + r0;
        const __nv_bfloat16 * residual = tile->residual;
        const bool gate_up = tile->epilogue == kEpiGateUp;
        const float s2_up = tile->s2_up;
#pragma unroll
        for (int ts = 0; ts < kGroups; ++ts) {
          if constexpr (!kDense) {
            // the two block halves of a chunk sit in lanes t and t ^ 2
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[ts][i] += __shfl_xor_sync(0xffffffffu, acc[ts][i], 2);
          }
          if (kDense || t < 2) {
            // dense: this lane holds tokens 2t, 2t+1 of rows r0 and r0 + 8, with the block scales' 2^-8 still in
            const int tok0 = kDense ? 2 * t : 4 * ts + 2 * t;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              if (tok0 + e < m_tokens) {
                const float unscale = xs[tok0 + e] * (kDense ? 256.0f : 1.0f);  // undoes the token's fp16 scaling
                if (gate_up) {
                  // rows alternate 8 gate / 8 up: this lane's row r0 is gate row j, its row r0 + 8 the matching up row
                  const int j = (row_a >> 4) * 8 + (row_a & 7);
                  if (row_a + 8 < rows) {
                    const float gate = acc[ts][e] * (unscale * s2);
                    const float up = acc[ts][2 + e] * (unscale * s2_up);
                    y[static_cast<size_t>(tok0 + e) * (rows >> 1) + j] = __float2bfloat16_rn(gate / (1.0f + expf(-gate)) * up);
                  }
                } else {
                  const float f = unscale * s2;
                  if (row_a < rows) {
                    const size_t o = static_cast<size_t>(tok0 + e) * rows + row_a;
                    const float r = residual != nullptr ? __bfloat162float(residual[o]) : 0.0f;
                    y[o] = __float2bfloat16_rn(acc[ts][e] * f + r);
                  }
                  if (row_a + 8 < rows) {
                    const size_t o = static_cast<size_t>(tok0 + e) * rows + row_a + 8;
                    const float r = residual != nullptr ? __bfloat162float(residual[o]) : 0.0f;
                    y[o] = __float2bfloat16_rn(acc[ts][2 + e] * f + r);
                  }
                }
              }
            }
          }
        }
        if (tile->signal) {
          // another item of this run reads these outputs: make the stores visible, then count this warp's part
          __threadfence();
          __syncwarp();
          if (lane == 0) atomicAdd(item_done + tile->item, 1ULL);
        }
      }
    }
    if (ok && prev_item >= 0) {
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(xempty + buf));
    }
  }
  if (counted_items > 0) {
    // A run with dependencies leaves its completion counts at zero for the next one: the last CTA to get here clears
    // them (every wait of the run has ended by then, since every CTA is past its last tile).
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned int * ctas_done = reinterpret_cast<unsigned int *>(item_done + counted_items);
      __threadfence();
      if (atomicAdd(ctas_done, 1u) == gridDim.x - 1) {
        for (int i = 0; i < counted_items; ++i) item_done[i] = 0ULL;
        *ctas_done = 0u;
      }
    }
  }
}

constexpr int kBarrierBytes = (2 * kMaxStages + 8 + 2) * 8 + 2 * 8 * 4;

struct Plan {
  int stages = 0;
  int x_buf_halfs = 0;
  int xs_buf_floats = 0;
  int x_bufs = 0;
  int smem_bytes = 0;
  int ksplit = 2;  // shape of the CTA (template KS)
};

// Shared-memory plan for a batch with at most max_k columns: activation buffers (raw BF16 rows land in them and are
// converted in place, so there is no separate raw ring), then as many ring stages as fit.  Two buffers (the next
// item's copy runs under the current item's tiles) when at least five stages remain, else one.
bool make_plan(int m, int max_k, Plan * p, int min_ks = 1) {
  const int mt = m < kDenseFrom ? 1 : 2;
  const int x_halfs = ((m * (max_k + x_pad(m)) + 63) / 64) * 64;  // whole 128-byte bank spans
  const int xs_floats = 8;
  // The two-CTAs-per-SM shape first (measured: 0.8B-class step at one token 51 -> 45 us); it needs four ring stages
  // per CTA beside two activation buffers, or three beside one.  Else the one-CTA shape with all of the SM's memory.
  for (int ks = min_ks; ks <= 2; ++ks) {
    const int base = 1024 + 2 * xs_floats * 4 + red_floats(ks, mt) * 4 + kZeroHalfs * 2 +
                     kMaxTilesInSmem * static_cast<int>(sizeof(GemvTile)) + kBarrierBytes;
    for (int bufs = 2; bufs >= 1; --bufs) {
      const int fixed = base + bufs * x_halfs * 2;
      const int stages = std::min(kMaxStages, (smem_budget(ks) - fixed) / kStageBytes);
      if (stages >= (bufs == 2 ? (ks == 1 ? 4 : 5) : 3)) {
        p->stages = stages;
        p->x_buf_halfs = x_halfs;
        p->xs_buf_floats = xs_floats;
        p->x_bufs = bufs;
        p->smem_bytes = fixed + stages * kStageBytes;
        p->ksplit = ks;
        return true;
      }
    }
  }
  return false;
}

using StreamKernel = void (*)(const GemvItem *, const GemvTile *, const int *, int, const __nv_bfloat16 *, __nv_bfloat16 *,
                              int, int, int, int, unsigned long long *, int, unsigned int *, uint32_t, unsigned int);

StreamKernel stream_kernel(int m, int ks) {
  if (m < kDenseFrom) return ks == 1 ? gemv_w4a16_stream_kernel<1, 1> : gemv_w4a16_stream_kernel<1, 2>;
  return ks == 1 ? gemv_w4a16_stream_kernel<2, 1> : gemv_w4a16_stream_kernel<2, 2>;
}

// The plan for a list on the current device: the two-CTAs-per-SM shape only if two of its CTAs really fit on an SM
// (items that wait for other items rely on every CTA of the grid being resident).
cudaError_t plan_for_device(int m, int max_k, Plan * p, bool * fits) {
  *fits = make_plan(m, max_k, p);
  if (!*fits) return cudaSuccess;
  cudaError_t e = cudaFuncSetAttribute(stream_kernel(m, p->ksplit), cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       smem_budget(p->ksplit));
  if (e != cudaSuccess) return e;
  if (p->ksplit == 1) {
    int resident = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, stream_kernel(m, 1), cta_threads(1),
                                                      static_cast<size_t>(p->smem_bytes));
    if (e != cudaSuccess) return e;
    if (resident < 2) {
      *fits = make_plan(m, max_k, p, 2);
      if (*fits) e = cudaFuncSetAttribute(stream_kernel(m, 2), cudaFuncAttributeMaxDynamicSharedMemorySize, smem_budget(2));
    }
  }
  return e;
}

}  // namespace
}  // namespace q35b

using namespace q35b;

struct q35b_gemv_batch {
  int count = 0;
  int m = 0;
  int grid = 0;
  int device = 0;
  Plan plan;
  void * dev_base = nullptr;
  GemvItem * items = nullptr;
  GemvTile * tiles = nullptr;
  int * cta_begin = nullptr;
  unsigned int * status = nullptr;
  unsigned long long * item_done = nullptr;  // per item: storing warps that finished a tile in the current run
  bool has_dependencies = false;
  size_t bytes_per_run = 0;
  uint32_t wait_limit = kWaitLimit;   // polls every device-side wait of a run may take
  unsigned int wait_extra = 0;        // test hook: completions demanded on top of what a dependency really delivers
  q35b::WBatch * tensor = nullptr;   // set: the list runs on the tensor path (gemm_wstream.cu), nothing above is used
};

namespace q35b {

bool gemv_stream_eligible(const q35b_weight * w, int m) {
  if (w == nullptr || w->rows <= 0 || (w->k % 256) != 0 || w->negative_scales) return false;
  Plan p;
  return make_plan(m, w->k, &p);
}

int gemv_plan_debug(int m, int max_k, int * ctas, int * ring_stages, int * activation_buffers, int * smem_bytes) {
  if (m < 1 || m > 8 || max_k < 256 || (max_k % 256) != 0) return fail(Q35B_ERR_SHAPE, "NVFP4 decode projection supports 1..8 tokens and cols that are a multiple of 256.");
  Plan p;
  if (!make_plan(m, max_k, &p)) return fail(Q35B_ERR_SHAPE, "Activations of the NVFP4 projection work list do not fit in shared memory.");
  if (ctas != nullptr) *ctas = ctas_per_sm(p.ksplit);
  if (ring_stages != nullptr) *ring_stages = p.stages;
  if (activation_buffers != nullptr) *activation_buffers = p.x_bufs;
  if (smem_bytes != nullptr) *smem_bytes = p.smem_bytes;
  return Q35B_OK;
}

int gemv_batch_build(const q35b_gemv_item * items, int count, int m, q35b_gemv_batch ** out) {
  if (items == nullptr || out == nullptr || count <= 0) return fail(Q35B_ERR_ARGUMENT, "Invalid NVFP4 projection work list.");
  if (m < 1 || m > 8) return fail(Q35B_ERR_SHAPE, "NVFP4 decode projection supports 1..8 tokens.");
  *out = nullptr;
  int max_k = 0;
  for (int i = 0; i < count; ++i) {
    const q35b_weight * w = items[i].weight;
    if (w == nullptr) return fail(Q35B_ERR_ARGUMENT, "NVFP4 projection work list holds a null weight.");
    if ((w->k % 256) != 0) return fail(Q35B_ERR_SHAPE, "The streaming NVFP4 projection needs cols to be a multiple of 256.");
    if (w->negative_scales) return fail(Q35B_ERR_FORMAT, "The streaming NVFP4 projection needs unsigned E4M3 block scales.");
    if (w->gate_up && items[i].residual_bf16 != nullptr) {
      return fail(Q35B_ERR_ARGUMENT, "A gate/up projection takes no residual.");
    }
    if ((reinterpret_cast<uintptr_t>(items[i].x_bf16) & 15u) != 0) {
      return fail(Q35B_ERR_ARGUMENT, "Activations of the NVFP4 projection work list must be 16-byte aligned.");
    }
    if (items[i].after < 0 || items[i].after > i) {
      return fail(Q35B_ERR_ARGUMENT, "An NVFP4 projection work list item can only run after an earlier item of the list.");
    }
    max_k = std::max(max_k, w->k);
  }
  auto * b = new q35b_gemv_batch();
  b->count = count;
  b->m = m;
  if (cudaGetDevice(&b->device) != cudaSuccess) {
    delete b;
    return fail_cuda(cudaGetLastError(), "cudaGetDevice");
  }
  bool fits = false;
  if (const cudaError_t pe = plan_for_device(m, max_k, &b->plan, &fits); pe != cudaSuccess) {
    delete b;
    return fail_cuda(pe, "planning the projection work list");
  }
  if (!fits) {
    delete b;
    return fail(Q35B_ERR_SHAPE, "Activations of the NVFP4 projection work list do not fit in shared memory.");
  }
  const int grid_max = sm_count() * ctas_per_sm(b->plan.ksplit);

  std::vector<GemvTile> all;
  std::vector<GemvItem> h_items(count);
  for (int i = 0; i < count; ++i) {
    const q35b_weight * w = items[i].weight;
    GemvItem & it = h_items[i];
    if (const int st = make_code_map(&it.tmap, w->codes, std::max(w->rows, 1), w->k / 2, kTileRows)) {
      delete b;
      return st;
    }
    it.scales_tiled = w->scales_tiled;
    it.x = static_cast<const __nv_bfloat16 *>(items[i].x_bf16);
    it.y = static_cast<__nv_bfloat16 *>(items[i].y_bf16);
    it.rows = w->rows;
    it.k = w->k;
    it.k_steps = w->k / 256;
    it.s2 = w->s2;
    for (int rb = 0; rb < (w->rows + kTileRows - 1) / kTileRows; ++rb) {
      GemvTile tl;
      tl.item = i;
      tl.row_block = rb;
      tl.k = w->k;
      tl.k_steps = it.k_steps;
      tl.rows = w->rows;
      tl.s2 = w->s2;
      tl.scales = w->scales_tiled + static_cast<size_t>(rb) * it.k_steps * kScaleBytes;
      tl.codes = w->codes + static_cast<size_t>(rb) * kTileRows * (w->k / 2);
      tl.x = it.x;
      tl.y = it.y;
      tl.residual = static_cast<const __nv_bfloat16 *>(items[i].residual_bf16);
      tl.s2_up = w->s2_up;
      tl.epilogue = w->gate_up ? kEpiGateUp : kEpiPlain;
      tl.wait_item = items[i].after - 1;
      tl.wait_count = 0;
      tl.signal = 0;
      if (tl.wait_item >= 0) {
        const q35b_weight * dep = items[tl.wait_item].weight;
        tl.wait_count = static_cast<unsigned int>((dep->rows + kTileRows - 1) / kTileRows) * kRowGroups;
        b->has_dependencies = true;
      }
      for (int j = i + 1; j < count; ++j) {
        if (items[j].after - 1 == i) tl.signal = 1;
      }
      all.push_back(tl);
    }
    b->bytes_per_run += w->codes_bytes + w->scales_bytes;
  }
  std::vector<int> level(count, 0);
  int max_level = 0;
  for (int i = 0; i < count; ++i) {
    if (items[i].after > 0) level[i] = level[items[i].after - 1] + 1;
    max_level = std::max(max_level, level[i]);
  }
  const int grid = std::max(1, std::min<int>(grid_max, static_cast<int>(all.size())));
  std::vector<std::vector<GemvTile>> per_cta(grid);
  {
    // Each CTA gets a contiguous run of tiles (projection-major order) of about equal cost: it changes projection,
    // and therefore converts a new activation vector, as rarely as possible, and neighbouring CTAs stream
    // neighbouring rows.  A tile goes to the CTA in whose share of the total cost its midpoint falls, so no CTA
    // exceeds its share by more than half a tile.
    // With dependencies the list is cut into levels (an item's level is one more than that of the item it runs
    // after): every level is spread over all CTAs in this way by itself, and a CTA walks its levels in order, so the
    // whole grid works on the tiles something is waiting for instead of a few CTAs owning them.
    for (int lv = 0; lv <= max_level; ++lv) {
      long total = 0;
      for (const GemvTile & tl : all) total += level[tl.item] == lv ? tl.k_steps + 1 : 0;
      long done = 0;
      int c = 0;
      for (const GemvTile & tl : all) {
        if (level[tl.item] != lv) continue;
        const long cost = tl.k_steps + 1;
        while (c + 1 < grid && (done + cost / 2) * grid >= static_cast<long>(c + 1) * total) ++c;
        per_cta[c].push_back(tl);
        done += cost;
      }
    }
  }
  std::vector<GemvTile> h_tiles;
  std::vector<int> h_begin(grid + 1, 0);
  for (int c = 0; c < grid; ++c) {
    std::stable_sort(per_cta[c].begin(), per_cta[c].end(), [&](const GemvTile & a, const GemvTile & d) {
      if (level[a.item] != level[d.item]) return level[a.item] < level[d.item];
      return a.item != d.item ? a.item < d.item : a.row_block < d.row_block;
    });
    h_begin[c] = static_cast<int>(h_tiles.size());
    for (const GemvTile & tl : per_cta[c]) h_tiles.push_back(tl);
  }
  h_begin[grid] = static_cast<int>(h_tiles.size());
  b->grid = grid;

  const size_t o_tiles = sizeof(GemvItem) * count;
  const size_t o_begin = (o_tiles + sizeof(GemvTile) * h_tiles.size() + 15) / 16 * 16;
  const size_t o_status = (o_begin + sizeof(int) * (grid + 1) + 15) / 16 * 16;
  const size_t o_done = o_status + 16;
  const size_t total = o_done + sizeof(unsigned long long) * (count + 1);  // + the finished-CTA count
  cudaError_t e = cudaMalloc(&b->dev_base, total);
  if (e != cudaSuccess) {
    delete b;
    return fail_cuda(e, "cudaMalloc(projection work list)");
  }
  auto * base = static_cast<uint8_t *>(b->dev_base);
  b->items = reinterpret_cast<GemvItem *>(base);
  b->tiles = reinterpret_cast<GemvTile *>(base + o_tiles);
  b->cta_begin = reinterpret_cast<int *>(base + o_begin);
  b->status = reinterpret_cast<unsigned int *>(base + o_status);
  b->item_done = reinterpret_cast<unsigned long long *>(base + o_done);
  e = cudaMemcpy(b->items, h_items.data(), sizeof(GemvItem) * count, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(b->tiles, h_tiles.data(), sizeof(GemvTile) * h_tiles.size(), cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(b->cta_begin, h_begin.data(), sizeof(int) * (grid + 1), cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemset(b->status, 0, 16 + sizeof(unsigned long long) * (count + 1));
  if (e != cudaSuccess) {
    cudaFree(b->dev_base);
    delete b;
    return fail_cuda(e, "uploading the projection work list");
  }
  *out = b;
  return Q35B_OK;
}

int gemv_batch_build_tensor(const q35b_gemv_item * items, int count, int m, int digits, q35b_gemv_batch ** out) {
  if (out == nullptr) return fail(Q35B_ERR_ARGUMENT, "Invalid NVFP4 projection work list.");
  *out = nullptr;
  WBatch * t = nullptr;
  if (const int st = wbatch_build(items, count, m, digits, &t)) return st;
  auto * b = new q35b_gemv_batch();
  b->count = count;
  b->m = m;
  b->tensor = t;
  b->bytes_per_run = wbatch_bytes(t);
  *out = b;
  return Q35B_OK;
}

int gemv_batch_launch(const q35b_gemv_batch * b, const void * x_override, void * y_override, cudaStream_t s) {
  if (b == nullptr) return fail(Q35B_ERR_ARGUMENT, "Null NVFP4 projection work list.");
  if (b->tensor != nullptr) return wbatch_launch(b->tensor, s);
  const auto * xo = static_cast<const __nv_bfloat16 *>(x_override);
  auto * yo = static_cast<__nv_bfloat16 *>(y_override);
  const int counted = b->has_dependencies ? b->count : 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(b->grid));
  cfg.blockDim = dim3(static_cast<unsigned>(cta_threads(b->plan.ksplit)));
  cfg.dynamicSmemBytes = static_cast<size_t>(b->plan.smem_bytes);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const GemvItem * d_items = b->items;
  const GemvTile * d_tiles = b->tiles;
  const int * d_begin = b->cta_begin;
  const Plan & pl = b->plan;
  const cudaError_t le = cudaLaunchKernelEx(&cfg, stream_kernel(b->m, pl.ksplit), d_items,
                                            d_tiles, d_begin, b->m, xo, yo, pl.stages, pl.x_buf_halfs, pl.xs_buf_floats,
                                            pl.x_bufs, b->item_done, counted, b->status, b->wait_limit,
                                            b->wait_extra);
  count_launch();
  Q35B_CUDA_TRY(le, "gemv_w4a16_stream_kernel launch");
  return Q35B_OK;
}

void gemv_batch_free(q35b_gemv_batch * b) {
  if (b == nullptr) return;
  wbatch_free(b->tensor);
  if (b->dev_base != nullptr) cudaFree(b->dev_base);
  delete b;
}

int gemv_batch_read_status(const q35b_gemv_batch * b, unsigned int * out) {
  if (b == nullptr || out == nullptr) return fail(Q35B_ERR_ARGUMENT, "Null NVFP4 projection work list.");
  if (b->tensor != nullptr) return wbatch_status(b->tensor, out);
  Q35B_CUDA_TRY(cudaMemcpy(out, b->status, sizeof(unsigned int), cudaMemcpyDeviceToHost), "cudaMemcpy(work list status)");
  return Q35B_OK;
}

size_t gemv_batch_bytes(const q35b_gemv_batch * b) { return b ? b->bytes_per_run : 0; }

int gemv_batch_debug_wait(q35b_gemv_batch * b, unsigned int wait_limit, unsigned int extra_completions) {
  if (b == nullptr || b->tensor != nullptr || wait_limit == 0) return fail(Q35B_ERR_ARGUMENT, "Invalid NVFP4 projection work list.");
  b->wait_limit = wait_limit;
  b->wait_extra = extra_completions;
  // counts of a run that gave up stay behind: start the next run from zero
  if (b->item_done != nullptr) {
    Q35B_CUDA_TRY(cudaMemset(b->status, 0, 16 + sizeof(unsigned long long) * (b->count + 1)), "cudaMemset(work list counters)");
  }
  return Q35B_OK;
}

}  // namespace q35b
