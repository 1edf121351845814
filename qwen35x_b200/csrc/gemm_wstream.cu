// Weight-streaming block-scaled FP4 projection for few tokens (1..128 operand columns) on sm_100a.
//
// The prefill GEMMs put the tokens on the 128 rows of the tensor-core tile and stream weights as the narrow
// operand; with few tokens that wastes the tile and leaves most SMs without work.  Here the roles are swapped:
//
//   UMMA A (128 rows)  = one 128-row block of the WEIGHT, streamed once from HBM: codes in checkpoint order
//                        through the weight's 128-row TMA map, scale factors as the weight's 512-byte scale tiles;
//   UMMA B (N columns) = the activation operand, N = 16..128 rows of NVFP4 codes (re-read from L2 by every tile);
//   D [128, N] fp32    = in TMEM; a lane is a weight row, a column is an operand row.
//
// One persistent CTA per SM walks a list of (projection, row block) tiles, as the streaming decode kernel does, with
// a TMA-fed shared-memory ring (weights and activations have separate producer threads: weights are constant and
// start streaming before the previous kernel of the stream has finished, activations wait for it), one MMA thread
// issuing tcgen05.mma kind::mxf4nvf4.block_scale per 64 columns of K, two TMEM accumulators so that the epilogue of
// a tile runs under the MMAs of the next, and four epilogue warps that turn accumulator lanes into BF16 outputs
// y[token, row].
//
// Two uses:
//   * small-M prefill (W4A4, 1..128 tokens): the operand rows are the tokens of q35b_quantize_nvfp4_bf16;
//     replaces run_nvfp4_cublaslt_prefill_projection_device (src/runtime/cuda_bench.cu:1056-1167) for short
//     sequences, where it is bound by the weight stream (HBM), not by the tensor pipe;
//   * decode (W4A16, 1..8 tokens): every token is expanded into `digits` operand rows, an NVFP4 digit expansion of
//     its BF16 activations (expand_digits_kernel below): digit j quantises what digits 0..j-1 left over, so the sum
//     of the rows reproduces the activation to 6^-digits of its block's amax (digits = 5: 1.3e-4, far below BF16's
//     own 2^-9), and the epilogue adds the digits' accumulator columns.  Replaces nvfp4_row_dot / matvec_nvfp4_bf16
//     (src/kernels/cuda/decode_layers.cuh:200-284) with the FP4 decode done by the tensor core instead of by
//     conversion instructions.
//
// Every wait is bounded; an expired wait records a code in *status and the role stops; the CTA still frees TMEM.
#include <cuda_bf16.h>

#include <algorithm>
#include <vector>

#include "engine.h"
#include "nvfp4_codec.cuh"

namespace q35b {
namespace {

constexpr int kRows = 128;               // weight rows per tile (UMMA M)
constexpr int kStepBytes = 128;          // 256 FP4 columns of K per ring stage
constexpr int kMmaPerStage = 4;          // K = 64 per MMA
constexpr int kSfChunk = 512;            // scale factors of 128 rows x 64 columns
constexpr int kABytes = kRows * kStepBytes;          // 16 KB
constexpr int kSfBytes = kMmaPerStage * kSfChunk;    // 2 KB (weights, and activations: at most 128 operand rows)
constexpr int kMaxCols = 128;
constexpr int kMaxStages = 8;
constexpr int kThreads = 7 * 32;         // warp 0 weight producer, 1 MMA, 2 activation producer, 3..6 epilogue
constexpr int kTmemCols = 512;           // two accumulator buffers of up to 240 columns + 16 + 16 scale-factor columns
constexpr int kAccBufCols = 224;
constexpr int kSfaCol = 2 * kAccBufCols;   // two sets of scale-factor columns (A 16 + B 16 each), used by stages in turn,
constexpr int kSfbCol = kSfaCol + 16;      // so that the copies of one stage do not wait for the MMAs of the one before
constexpr int kSfSetCols = 32;
constexpr uint32_t kWaitLimit = 1u << 22;
constexpr int kSmemBudget = 220 * 1024;   // dynamic part; the staged tile descriptors are static shared memory

enum StatusCode : unsigned { kWeightWait = 41, kActWait = 42, kMmaWait = 43, kMmaDrainWait = 44, kEpilogueWait = 45 };
enum Epilogue : int { kEpiPlain = 0, kEpiGateUp = 1 };

// One projection of the list.  Lives in device memory (work lists) or in the kernel's parameter space (single
// projection); the tensor maps are read by the TMA unit from wherever the item is.
struct alignas(128) WItem {
  CUtensorMap tmap_w;            // weight codes [rows, K/2], box 128 rows x 128 bytes, 128B swizzle
  CUtensorMap tmap_x;            // operand codes [operand rows, K/2], box n_cols rows x 128 bytes, 128B swizzle
  const uint8_t * w_scales;      // weight scale tiles
  const uint8_t * x_scales;      // operand scale tiles (one 128-row block)
  const float * x_g;             // the operand's scale: one device scalar, or one per token (g_stride = 1)
  __nv_bfloat16 * y;             // [tokens, ldy]
  const __nv_bfloat16 * residual;  // NULL or [tokens, ldr]
  int rows;                      // weight rows
  int k_steps;                   // K / 256
  int n_cols;                    // operand rows padded to a multiple of 16 (UMMA N)
  int tokens;
  int digits;                    // operand rows per token (1: plain W4A4)
  int ldy, ldr;
  float s2, s2_up;
  int epilogue;
  int g_stride;
};

struct alignas(8) WTile {
  int item;
  int row_block;
};

// Everything the roles need to know about one tile, staged in shared memory at kernel start so that no role chases
// pointers through global memory at a tile boundary (a 128-row x 1024-column tile lasts under two microseconds).
struct alignas(16) STile {
  const CUtensorMap * tmap_w;
  const CUtensorMap * tmap_x;
  const uint8_t * w_scales;      // scale tiles of this row block
  const uint8_t * x_scales;
  const float * x_g;
  __nv_bfloat16 * y;
  const __nv_bfloat16 * residual;
  int row_block, rows, k_steps, n_cols, tokens, digits, ldy, ldr, epilogue;
  float s2, s2_up;
  int g_stride;
};
constexpr int kMaxTilesInSmem = 40;

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
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kWaitLimit; ++i) {
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
// K-major operand tile, 128B swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_k_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
// Scale-factor slab for tcgen05.cp: no swizzle, 8 rows of 16 bytes per core matrix, core matrices 128 bytes apart.
__device__ __forceinline__ uint64_t desc_sf(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(128 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}
// With few operand columns an MMA is far shorter than the tensor pipe's latency, and four MMAs per stage that all
// accumulate into the same TMEM columns run one after the other at that latency (measured: 1500 cycles per stage,
// against 900 for the stage's bytes to arrive from HBM).  So the MMAs of a stage go to different partial
// accumulators (as many as fit beside each other in a buffer), each of which then sees one MMA per stage, and the
// epilogue adds the partials.
__device__ __forceinline__ int partial_accumulators(int n_cols) { return 4 * n_cols <= kAccBufCols ? 4 : (2 * n_cols <= kAccBufCols ? 2 : 1); }

// kind::mxf4nvf4: E2M1 x E2M1, K-major, UE4M3 scales, M = 128, N = n_cols.
__device__ __forceinline__ uint32_t instr_desc(int n_cols) {
  uint32_t d = 0;
  d |= 1u << 7;
  d |= 1u << 10;
  d |= static_cast<uint32_t>(n_cols >> 3) << 17;
  d |= static_cast<uint32_t>(kRows >> 4) << 24;
  return d;
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t tmem_sfa,
                                     uint32_t tmem_sfb, uint32_t accumulate) {
  asm volatile(
    "{\n\t.reg .pred p;\n\t"
    "setp.ne.b32 p, %4, 0;\n\t"
    "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(tmem_d),
    "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
    : "memory");
}
__device__ __forceinline__ void utccp_sf(uint32_t tmem_dst, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_dst), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
    "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
      "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
    : "r"(taddr)
    : "memory");
}

__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

// items == nullptr: the one projection in `single`, tiles dealt round-robin (tile = row block);
// otherwise CTA b walks tiles[cta_begin[b] .. cta_begin[b + 1]).
__global__ void __launch_bounds__(kThreads, 1)
gemm_wstream_kernel(const __grid_constant__ WItem single, const WItem * __restrict__ items, const WTile * __restrict__ tiles,
                    const int * __restrict__ cta_begin, int single_tiles, int stages, int b_slot_bytes, unsigned int * status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t * smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t * smem_a = smem;
  uint8_t * smem_b = smem_a + stages * kABytes;
  uint8_t * smem_sfa = smem_b + stages * b_slot_bytes;
  uint8_t * smem_sfb = smem_sfa + stages * kSfBytes;
  uint64_t * bars = reinterpret_cast<uint64_t *>(smem_sfb + stages * kSfBytes);
  uint64_t * full = bars;                           // [stages]: both producers' bytes have landed
  uint64_t * empty = bars + kMaxStages;             // [stages]: the MMAs that read the stage have retired
  uint64_t * tmem_full = bars + 2 * kMaxStages;     // [2]: accumulator complete
  uint64_t * tmem_empty = tmem_full + 2;            // [2]: the epilogue warps have read the accumulator out
  uint32_t * tmem_slot = reinterpret_cast<uint32_t *>(tmem_empty + 2);
  __shared__ STile stile[kMaxTilesInSmem];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  int tile_begin, n_tiles, tile_stride;
  if (items == nullptr) {
    tile_begin = blockIdx.x;
    tile_stride = gridDim.x;
    n_tiles = single_tiles > static_cast<int>(blockIdx.x) ? (single_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  } else {
    tile_begin = cta_begin[blockIdx.x];
    tile_stride = 1;
    n_tiles = cta_begin[blockIdx.x + 1] - tile_begin;
  }
  auto describe = [&](int ti, STile & d) {
    const WItem * it = &single;
    int rb = tile_begin + ti * tile_stride;
    if (items != nullptr) {
      const WTile t = tiles[tile_begin + ti];
      rb = t.row_block;
      it = items + t.item;
    }
    d.tmap_w = &it->tmap_w;
    d.tmap_x = &it->tmap_x;
    d.k_steps = it->k_steps;
    d.w_scales = it->w_scales + static_cast<size_t>(rb) * d.k_steps * kSfBytes;
    d.x_scales = it->x_scales;
    d.x_g = it->x_g;
    d.y = it->y;
    d.residual = it->residual;
    d.row_block = rb;
    d.rows = it->rows;
    d.n_cols = it->n_cols;
    d.tokens = it->tokens;
    d.digits = it->digits;
    d.ldy = it->ldy;
    d.ldr = it->ldr;
    d.epilogue = it->epilogue;
    d.s2 = it->s2;
    d.s2_up = it->s2_up;
    d.g_stride = it->g_stride;
  };
  // tile descriptors are constant for the life of a work list (and of a launch): read them before anything else
  for (int ti = threadIdx.x; ti < min(n_tiles, kMaxTilesInSmem); ti += kThreads) describe(ti, stile[ti]);
  // tiles beyond the staged ones (a CTA with a very long list) are described on the fly
  auto tile_at = [&](int ti, STile & spill) -> const STile * {
    if (ti < kMaxTilesInSmem) return stile + ti;
    describe(ti, spill);
    return &spill;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < stages; ++i) {
      mbar_init(smem_u32(full + i), 2);
      mbar_init(smem_u32(empty + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(tmem_full + i), 1);
      mbar_init(smem_u32(tmem_empty + i), 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(static_cast<uint32_t>(kTmemCols))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  // The next kernel of the stream may be scheduled from here on; this one touches nothing an earlier kernel may
  // still be writing (activations, scales, outputs) before its own griddepcontrol.wait below.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == 0) {
    // ------------------------------------------------------------ weight producer (constant data: no wait)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      STile spill;
      for (int ti = 0; ti < n_tiles && ok; ++ti) {
        const STile * it = tile_at(ti, spill);
        const int k_steps = it->k_steps, rb = it->row_block;
        const uint8_t * sf = it->w_scales;
        for (int ks = 0; ks < k_steps; ++ks) {
          if (!mbar_wait(smem_u32(empty + stage), phase ^ 1)) {
            atomicExch(status, kWeightWait);
            ok = false;
            break;
          }
          const uint32_t bar = smem_u32(full + stage);
          mbar_expect_tx(bar, kABytes + kSfBytes);
          tma_load_2d(smem_u32(smem_a + stage * kABytes), it->tmap_w, bar, ks * kStepBytes, rb * kRows);
          bulk_load(smem_u32(smem_sfa + stage * kSfBytes), sf + static_cast<size_t>(ks) * kSfBytes, kSfBytes, bar);
          if (++stage == stages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------ activation producer
    if (lane == 0) {
      asm volatile("griddepcontrol.wait;" ::: "memory");
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      STile spill;
      for (int ti = 0; ti < n_tiles && ok; ++ti) {
        const STile * it = tile_at(ti, spill);
        const int k_steps = it->k_steps;
        const uint32_t b_bytes = static_cast<uint32_t>(it->n_cols) * kStepBytes;
        for (int ks = 0; ks < k_steps; ++ks) {
          if (!mbar_wait(smem_u32(empty + stage), phase ^ 1)) {
            atomicExch(status, kActWait);
            ok = false;
            break;
          }
          const uint32_t bar = smem_u32(full + stage);
          mbar_expect_tx(bar, b_bytes + kSfBytes);
          tma_load_2d(smem_u32(smem_b + stage * b_slot_bytes), it->tmap_x, bar, ks * kStepBytes, 0);
          bulk_load(smem_u32(smem_sfb + stage * kSfBytes), it->x_scales + static_cast<size_t>(ks) * kSfBytes, kSfBytes, bar);
          if (++stage == stages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // Per stage: eight scale-factor copies into one of two TMEM column sets, then four MMAs.  With operand tiles this
    // narrow the MMAs are far shorter than the copy-to-MMA turnaround of the tensor pipe (about 500 cycles per stage,
    // measured by switching copies and MMAs off in turn: 49 us per 0.8B-class step without either, 52 with copies
    // only, 51 with MMAs only, 73 with both); issuing the copies a stage ahead of their MMAs did not hide it (83 us).
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0, sf_turn = 0;
      bool ok = true;
      STile spill;
      for (int ti = 0; ti < n_tiles && ok; ++ti) {
        const STile * it = tile_at(ti, spill);
        const int k_steps = it->k_steps;
        const uint32_t idesc = instr_desc(it->n_cols);
        const uint32_t ab = ti & 1;
        if (!mbar_wait(smem_u32(tmem_empty + ab), ((ti >> 1) & 1) ^ 1)) {
          atomicExch(status, kMmaDrainWait);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t acc = tmem_base + ab * kAccBufCols;
        const int n_cols = it->n_cols, parts = partial_accumulators(n_cols);
        for (int ks = 0; ks < k_steps; ++ks) {
          if (!mbar_wait(smem_u32(full + stage), phase)) {
            atomicExch(status, kMmaWait);
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint64_t a_desc = desc_k_sw128(smem_u32(smem_a + stage * kABytes));
          const uint64_t b_desc = desc_k_sw128(smem_u32(smem_b + stage * b_slot_bytes));
          const uint64_t sfa_desc = desc_sf(smem_u32(smem_sfa + stage * kSfBytes));
          const uint64_t sfb_desc = desc_sf(smem_u32(smem_sfb + stage * kSfBytes));
          const uint32_t sf_set = tmem_base + (sf_turn ^= 1u) * kSfSetCols;
#pragma unroll
          for (int j = 0; j < kMmaPerStage; ++j) {
            utccp_sf(sf_set + kSfaCol + j * 4, sfa_desc + j * (kSfChunk >> 4));
            utccp_sf(sf_set + kSfbCol + j * 4, sfb_desc + j * (kSfChunk >> 4));
          }
#pragma unroll
          for (int j = 0; j < kMmaPerStage; ++j) {
            umma(acc + (j & (parts - 1)) * n_cols, a_desc + j * 2, b_desc + j * 2, idesc, sf_set + kSfaCol + j * 4,
                 sf_set + kSfbCol + j * 4, (ks * kMmaPerStage + j) >= parts ? 1u : 0u);
          }
          umma_commit(smem_u32(empty + stage));
          if (++stage == stages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(smem_u32(tmem_full + ab));
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue: lane = weight row, column = operand row
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    STile spill;
    for (int ti = 0; ti < n_tiles; ++ti) {
      const STile * it = tile_at(ti, spill);
      const int rb = it->row_block;
      const uint32_t ab = ti & 1;
      if (!mbar_wait(smem_u32(tmem_full + ab), (ti >> 1) & 1)) {
        if (lane == 0) atomicExch(status, kEpilogueWait);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int rows = it->rows, tokens = it->tokens, digits = it->digits, n_cols = it->n_cols;
      const int row = rb * kRows + row_in_tile;
      const float * x_g = it->x_g;
      const int g_stride = it->g_stride;
      const bool gate_up = it->epilogue == kEpiGateUp;
      const float s2 = it->s2, s2_up = it->s2_up;
      __nv_bfloat16 * y = it->y;
      const __nv_bfloat16 * residual = it->residual;
      const int ldy = it->ldy, ldr = it->ldr;
      const uint32_t taddr = tmem_base + ab * kAccBufCols + (static_cast<uint32_t>(quarter * 32) << 16);
      const int parts = partial_accumulators(n_cols);
      float sum = 0.0f;
      int jc = 0, token = 0;
      for (int c0 = 0; c0 < n_cols; c0 += 16) {
        uint32_t r[16];
        tmem_ld16(taddr + c0, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        for (int p = 1; p < parts; ++p) {
          uint32_t r2[16];
          tmem_ld16(taddr + p * n_cols + c0, r2);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) + __uint_as_float(r2[i]));
        }
        if (c0 + 16 >= n_cols) {
          // the accumulator is in registers: hand it back before the stores
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(tmem_empty + ab));
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          sum += __uint_as_float(r[i]);
          if (++jc == digits) {
            // one output value per (token, weight row); all lanes take the same path
            const float gval = token < tokens ? __ldg(x_g + token * g_stride) : 0.0f;
            const float alpha = gval * s2, alpha_up = gval * s2_up;
            if (gate_up) {
              // rows alternate 8 gate / 8 up: lane l holds gate row j, lane l ^ 8 the matching up row
              const float other = __shfl_xor_sync(0xffffffffu, sum, 8);
              if ((row & 8) == 0 && token < tokens && row + 8 < rows) {
                const int j = (row >> 4) * 8 + (row & 7);
                y[static_cast<size_t>(token) * ldy + j] = __float2bfloat16_rn(silu_mul(sum * alpha, other * alpha_up));
              }
            } else if (token < tokens && row < rows) {
              const float rv = residual != nullptr ? __bfloat162float(residual[static_cast<size_t>(token) * ldr + row]) : 0.0f;
              y[static_cast<size_t>(token) * ldy + row] = __float2bfloat16_rn(fmaf(sum, alpha, rv));
            }
            sum = 0.0f;
            jc = 0;
            ++token;
          }
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(static_cast<uint32_t>(kTmemCols))
                 : "memory");
  }
}

// ---- decode: BF16 activations -> NVFP4 digit expansion ---------------------------------------------------------

__device__ __forceinline__ uint32_t cvt_e2m1x8_w(const float (&q)[8]) {
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

struct ExpandItem {
  const __nv_bfloat16 * x;   // [tokens, k]
  uint8_t * codes;           // [tokens * digits, k / 2], operand row = token * digits + digit
  uint8_t * scales;          // tiled scales of one 128-row block: 128 * roundup(k / 16, 4) bytes
  float * g;                 // [tokens]: scale of each token's expansion
  int k;
};

// One CTA per (projection, token).  g = amax / (6 * 448) over the token's activations; per 16-element block, digit j
// takes the block's current residual r_j (r_0 = x): scale byte sb_j = UE4M3(amax(r_j) / 6 / g), d_j = decode(sb_j) * g,
// codes q_j = E2M1(r_j / d_j) (nearest), r_{j+1} = r_j - q_j * d_j.  |r_{j+1}| <= max(d_j, amax(r_j) / 16), so each
// digit shrinks the residual by about six; digits whose scale would underflow E4M3 stay zero.  Every scale byte of a
// real (row, block) is written by every run; the padding of the tiled layout was zeroed when the list was built.
__global__ void __launch_bounds__(128) expand_digits_kernel(const ExpandItem * __restrict__ items, int digits) {
  asm volatile("griddepcontrol.wait;" ::: "memory");  // the activations may come from the kernel before
  const ExpandItem it = items[blockIdx.x];
  const int token = blockIdx.y;
  const int k = it.k, blocks_per_row = k >> 4, slots = ((blocks_per_row + 3) >> 2) << 2;
  const __nv_bfloat16 * xt = it.x + static_cast<size_t>(token) * k;
  __shared__ float red[4];
  __shared__ float g_shared;
  float amax = 0.0f;
  for (int b = threadIdx.x; b < blocks_per_row * 2; b += blockDim.x) {
    const uint4 q = __ldg(reinterpret_cast<const uint4 *>(xt) + b);
    const uint32_t r[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float lo = fabsf(__uint_as_float(r[j] << 16)), hi = fabsf(__uint_as_float(r[j] & 0xffff0000u));
      if (lo < 3.0e38f) amax = fmaxf(amax, lo);  // NaN and inf do not take part
      if (hi < 3.0e38f) amax = fmaxf(amax, hi);
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    const float m = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    const float g = m > 0.0f ? m / (6.0f * 448.0f) : 1.0f;
    g_shared = g;
    it.g[token] = g;
  }
  __syncthreads();
  const float g = g_shared;
  const float inv_g6 = 1.0f / (6.0f * g);
  for (int blk = threadIdx.x; blk < blocks_per_row; blk += blockDim.x) {
    float v[16];
    {
      const uint4 * src = reinterpret_cast<const uint4 *>(xt + blk * 16);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint4 q = __ldg(src + h);
        const uint32_t r[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float lo = __uint_as_float(r[j] << 16), hi = __uint_as_float(r[j] & 0xffff0000u);
          // NaN and inf have no digit expansion: they contribute zero (the exact decode kernel propagates them)
          v[h * 8 + 2 * j] = fabsf(lo) < 3.0e38f ? lo : 0.0f;
          v[h * 8 + 2 * j + 1] = fabsf(hi) < 3.0e38f ? hi : 0.0f;
        }
      }
    }
    for (int dgt = 0; dgt < digits; ++dgt) {
      float bmax = 0.0f;
#pragma unroll
      for (int i = 0; i < 16; ++i) bmax = fmaxf(bmax, fabsf(v[i]));
      uint32_t sb = encode_ue4m3(bmax * inv_g6);
      sb = sb > 0x7eu ? 0x7eu : sb;
      const int op_row = token * digits + dgt;
      uint2 packed = make_uint2(0u, 0u);
      if (sb != 0u) {
        const float d = decode_e4m3(static_cast<uint8_t>(sb)) * g;
        const float r = 1.0f / d;
        float q0[8], q1[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          q0[i] = v[i] * r;
          q1[i] = v[8 + i] * r;
        }
        packed.x = cvt_e2m1x8_w(q0);
        packed.y = cvt_e2m1x8_w(q1);
        const uint32_t w[2] = {packed.x, packed.y};
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const uint32_t c = (w[i >> 3] >> (4 * (i & 7))) & 0xfu;
          v[i] = fmaf(-decode_e2m1(static_cast<uint8_t>(c)), d, v[i]);
        }
      }
      *reinterpret_cast<uint2 *>(it.codes + (static_cast<size_t>(op_row) * k + blk * 16) / 2) = packed;
      it.scales[tiled_scale_offset(op_row, blk, slots)] = static_cast<uint8_t>(sb);
    }
  }
}

int plan_stages(int b_slot_bytes) {
  const int stage = kABytes + b_slot_bytes + 2 * kSfBytes;
  return std::max(2, std::min(kMaxStages, (kSmemBudget - 1024 - 256) / stage));
}
int smem_for(int stages, int b_slot_bytes) { return stages * (kABytes + b_slot_bytes + 2 * kSfBytes) + 1024 + 256; }

int ensure_attr() {
  static std::atomic<bool> attr_set[64];
  int dev = 0;
  Q35B_CUDA_TRY(cudaGetDevice(&dev), "cudaGetDevice");
  if (!attr_set[dev & 63].load(std::memory_order_acquire)) {
    Q35B_CUDA_TRY(cudaFuncSetAttribute(gemm_wstream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget),
                  "cudaFuncSetAttribute(weight-streaming gemm smem)");
    attr_set[dev & 63].store(true, std::memory_order_release);
  }
  return Q35B_OK;
}

}  // namespace

// ---- small-M prefill: one projection, item in the kernel's parameter space, nothing allocated -------------------

// Prefill takes this kernel for up to 32 tokens (measured against the token-major 1-CTA kernel: 6.0 / 9.6 / 17.0 us
// against 8.5 / 12.3 / 22.8 us at 16 tokens on [3584,1024] / [9216,2560] / [32768,2560]; slower from about 64 tokens
// on, where its epilogue and the copy-to-MMA turnaround per stage outweigh the better spread over the SMs), unless
// the weight has so few row blocks and so long a K that most SMs would idle ([2560, 9216]: 20 tiles).
bool gemm_wstream_eligible(const q35b_weight * w, int m) {
  if (w == nullptr || !w->has_maps || m < 1 || m > 32 || (w->k % 256) != 0 || w->rows <= 0) return false;
  const int tiles = (w->rows + kRows - 1) / kRows, k_steps = w->k / 256;
  return !(tiles < 24 && k_steps > 16);
}

int launch_gemm_wstream(const q35b_weight * w, const uint8_t * a_codes, const uint8_t * a_scales_tiled, const float * g_dev,
                        int m, void * c_bf16, int ldc, const void * residual_bf16, int ldr, unsigned int * status_dev,
                        cudaStream_t s) {
  if (const int st = ensure_attr()) return st;
  WItem item = {};
  item.tmap_w = w->tmap_codes_128;
  item.n_cols = round_up_int(m, 16);
  if (const int st = make_code_map(&item.tmap_x, a_codes, m, w->k / 2, item.n_cols)) return st;
  item.w_scales = w->scales_tiled;
  item.x_scales = a_scales_tiled;
  item.x_g = g_dev;
  item.y = static_cast<__nv_bfloat16 *>(c_bf16);
  item.residual = static_cast<const __nv_bfloat16 *>(residual_bf16);
  item.rows = w->rows;
  item.k_steps = w->k / 256;
  item.tokens = m;
  item.digits = 1;
  item.ldy = ldc;
  item.ldr = ldr;
  item.s2 = w->s2;
  item.s2_up = w->s2_up;
  item.epilogue = w->gate_up ? kEpiGateUp : kEpiPlain;
  item.g_stride = 0;
  const int tiles = (w->rows + kRows - 1) / kRows;
  const int b_slot = item.n_cols * kStepBytes;
  const int stages = plan_stages(b_slot);
  const int grid = std::max(1, std::min(tiles, sm_count()));
  const cudaError_t le = launch_pdl(gemm_wstream_kernel, dim3(grid), dim3(kThreads), static_cast<size_t>(smem_for(stages, b_slot)), s,
                                    item, static_cast<const WItem *>(nullptr), static_cast<const WTile *>(nullptr),
                                    static_cast<const int *>(nullptr), tiles, stages, b_slot, status_dev);
  count_launch();
  Q35B_CUDA_TRY(le, "gemm_wstream_kernel launch");
  return Q35B_OK;
}


// ---- decode work list on the tensor path ------------------------------------------------------------------------

struct WBatch {
  int count = 0, m = 0, digits = 0, grid = 0, stages = 0, b_slot = 0, smem = 0;
  void * dev_base = nullptr;
  WItem * items = nullptr;
  WTile * tiles = nullptr;
  int * cta_begin = nullptr;
  ExpandItem * expand = nullptr;
  unsigned int * status = nullptr;
  size_t bytes_per_run = 0;
};

int wbatch_build(const q35b_gemv_item * items, int count, int m, int digits, WBatch ** out) {
  if (items == nullptr || out == nullptr || count <= 0) return fail(Q35B_ERR_ARGUMENT, "Invalid NVFP4 projection work list.");
  *out = nullptr;
  if (m < 1 || m > 8) return fail(Q35B_ERR_SHAPE, "NVFP4 decode projection supports 1..8 tokens.");
  if (digits < 1 || digits > 8 || m * digits > kMaxCols) {
    return fail(Q35B_ERR_ARGUMENT, "The tensor-core decode path takes 1..8 digits per token.");
  }
  for (int i = 0; i < count; ++i) {
    const q35b_weight * w = items[i].weight;
    if (w == nullptr || items[i].x_bf16 == nullptr || items[i].y_bf16 == nullptr) {
      return fail(Q35B_ERR_ARGUMENT, "NVFP4 projection work list holds a null weight or buffer.");
    }
    if (const int st = check_weight_device(w)) return st;
    if ((w->k % 256) != 0 || w->rows <= 0 || !w->has_maps) {
      return fail(Q35B_ERR_SHAPE, "The tensor-core decode path needs cols to be a multiple of 256.");
    }
    if (w->negative_scales) return fail(Q35B_ERR_FORMAT, "The tensor-core decode path needs unsigned E4M3 block scales.");
    if (w->gate_up && items[i].residual_bf16 != nullptr) return fail(Q35B_ERR_ARGUMENT, "A gate/up projection takes no residual.");
    if (items[i].after != 0) {
      return fail(Q35B_ERR_ARGUMENT, "The tensor-core decode path runs independent items only: an item that reads another "
                                     "item's output needs its activations expanded after that item has finished "
                                     "(use q35b_gemv_batch_create for such lists, or one list per level).");
    }
    if ((reinterpret_cast<uintptr_t>(items[i].x_bf16) & 15u) != 0) {
      return fail(Q35B_ERR_ARGUMENT, "Activations of the NVFP4 projection work list must be 16-byte aligned.");
    }
  }
  if (const int st = ensure_attr()) return st;
  auto * b = new WBatch();
  b->count = count;
  b->m = m;
  b->digits = digits;
  const int op_rows = m * digits;
  const int n_cols = round_up_int(op_rows, 16);
  b->b_slot = n_cols * kStepBytes;
  b->stages = plan_stages(b->b_slot);
  b->smem = smem_for(b->stages, b->b_slot);

  // layout of the one allocation: items | tiles | cta_begin | expand items | status | per-item digit buffers
  std::vector<WTile> all;
  std::vector<long> cost;
  for (int i = 0; i < count; ++i) {
    const q35b_weight * w = items[i].weight;
    for (int rb = 0; rb < (w->rows + kRows - 1) / kRows; ++rb) {
      all.push_back(WTile{i, rb});
      cost.push_back(w->k / 256 + 1);
    }
    b->bytes_per_run += w->codes_bytes + w->scales_bytes;
  }
  const int grid = std::max(1, std::min<int>(sm_count(), static_cast<int>(all.size())));
  b->grid = grid;
  // contiguous runs of about equal cost: a tile goes to the CTA in whose share of the total its midpoint falls
  std::vector<int> h_begin(grid + 1, 0);
  {
    long total = 0;
    for (long c : cost) total += c;
    long done = 0;
    int c = 0;
    for (size_t t = 0; t < all.size(); ++t) {
      while (c + 1 < grid && (done + cost[t] / 2) * grid >= static_cast<long>(c + 1) * total) h_begin[++c] = static_cast<int>(t);
      done += cost[t];
    }
    while (c + 1 <= grid) h_begin[++c] = static_cast<int>(all.size());
  }
  auto up = [](size_t v, size_t a) { return (v + a - 1) / a * a; };
  const size_t o_tiles = up(sizeof(WItem) * count, 256);
  const size_t o_begin = up(o_tiles + sizeof(WTile) * all.size(), 256);
  const size_t o_expand = up(o_begin + sizeof(int) * (grid + 1), 256);
  const size_t o_status = up(o_expand + sizeof(ExpandItem) * count, 256);
  size_t o_data = o_status + 256;
  std::vector<size_t> o_codes(count), o_scales(count), o_g(count);
  for (int i = 0; i < count; ++i) {
    const int k = items[i].weight->k;
    o_codes[i] = o_data;
    o_data = up(o_data + static_cast<size_t>(op_rows) * (k / 2), 256);
    o_scales[i] = o_data;
    o_data = up(o_data + static_cast<size_t>(128) * round_up_int(k / 16, 4), 256);
    o_g[i] = o_data;
    o_data += 256;
  }
  cudaError_t e = cudaMalloc(&b->dev_base, o_data);
  if (e != cudaSuccess) {
    delete b;
    return fail_cuda(e, "cudaMalloc(tensor-core projection work list)");
  }
  auto * base = static_cast<uint8_t *>(b->dev_base);
  b->items = reinterpret_cast<WItem *>(base);
  b->tiles = reinterpret_cast<WTile *>(base + o_tiles);
  b->cta_begin = reinterpret_cast<int *>(base + o_begin);
  b->expand = reinterpret_cast<ExpandItem *>(base + o_expand);
  b->status = reinterpret_cast<unsigned int *>(base + o_status);
  std::vector<WItem> h_items(count);
  std::vector<ExpandItem> h_expand(count);
  for (int i = 0; i < count; ++i) {
    const q35b_weight * w = items[i].weight;
    WItem & it = h_items[i];
    it = WItem{};
    it.tmap_w = w->tmap_codes_128;
    if (const int st = make_code_map(&it.tmap_x, base + o_codes[i], op_rows, w->k / 2, n_cols)) {
      cudaFree(b->dev_base);
      delete b;
      return st;
    }
    it.w_scales = w->scales_tiled;
    it.x_scales = base + o_scales[i];
    it.x_g = reinterpret_cast<const float *>(base + o_g[i]);
    it.y = static_cast<__nv_bfloat16 *>(items[i].y_bf16);
    it.residual = static_cast<const __nv_bfloat16 *>(items[i].residual_bf16);
    it.rows = w->rows;
    it.k_steps = w->k / 256;
    it.n_cols = n_cols;
    it.tokens = m;
    it.digits = digits;
    it.ldy = w->gate_up ? w->rows / 2 : w->rows;
    it.ldr = w->rows;
    it.s2 = w->s2;
    it.s2_up = w->s2_up;
    it.epilogue = w->gate_up ? kEpiGateUp : kEpiPlain;
    it.g_stride = 1;
    h_expand[i] = ExpandItem{static_cast<const __nv_bfloat16 *>(items[i].x_bf16), base + o_codes[i], base + o_scales[i],
                             reinterpret_cast<float *>(base + o_g[i]), w->k};
  }
  e = cudaMemset(b->dev_base, 0, o_data);
  if (e == cudaSuccess) e = cudaMemcpy(b->items, h_items.data(), sizeof(WItem) * count, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(b->tiles, all.data(), sizeof(WTile) * all.size(), cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(b->cta_begin, h_begin.data(), sizeof(int) * (grid + 1), cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(b->expand, h_expand.data(), sizeof(ExpandItem) * count, cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    cudaFree(b->dev_base);
    delete b;
    return fail_cuda(e, "uploading the tensor-core projection work list");
  }
  *out = b;
  return Q35B_OK;
}

int wbatch_launch(const WBatch * b, cudaStream_t s) {
  // 1. digit expansion of every item's activations (one CTA per item); 2. the streaming kernel, whose weight
  // producer starts at once while its activation producer waits for the expansion
  cudaError_t le = launch_pdl(expand_digits_kernel, dim3(b->count, b->m), dim3(128), 0, s, static_cast<const ExpandItem *>(b->expand),
                              b->digits);
  count_launch();
  Q35B_CUDA_TRY(le, "expand_digits_kernel launch");
  WItem unused = {};
  le = launch_pdl(gemm_wstream_kernel, dim3(b->grid), dim3(kThreads), static_cast<size_t>(b->smem), s, unused,
                  static_cast<const WItem *>(b->items), static_cast<const WTile *>(b->tiles), static_cast<const int *>(b->cta_begin), 0,
                  b->stages, b->b_slot, b->status);
  count_launch();
  Q35B_CUDA_TRY(le, "gemm_wstream_kernel launch");
  return Q35B_OK;
}

void wbatch_free(WBatch * b) {
  if (b == nullptr) return;
  if (b->dev_base != nullptr) cudaFree(b->dev_base);
  delete b;
}

int wbatch_status(const WBatch * b, unsigned int * out) {
  Q35B_CUDA_TRY(cudaMemcpy(out, b->status, sizeof(unsigned int), cudaMemcpyDeviceToHost), "cudaMemcpy(work list status)");
  return Q35B_OK;
}

size_t wbatch_bytes(const WBatch * b) { return b->bytes_per_run; }

}  // namespace q35b
