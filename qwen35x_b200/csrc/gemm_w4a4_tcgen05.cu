// W4A4 prefill GEMM for sm_100a: C[M, N] (bf16) = (Aq . Wq^T) * g * s2 with
// tcgen05.mma kind::mxf4nvf4 (block16, UE4M3 scale factors), TMEM accumulators,
// TMA-fed shared-memory ring.
//
// Replaces the reference's cuBLASLt FP4 call and the passes around it
// (src/runtime/cuda_bench.cu:1056-1167 run_nvfp4_cublaslt_prefill_projection_device,
// the fp32->bf16 pass at src/kernels/cuda/prefill.cu:639) and the SM120
// mma.sync projection (src/runtime/cuda_bench.cu:431-484).
//
// Operands in HBM
//   A codes  [M, K/2]  E2M1 pairs, K-major (activation quantiser output)
//   B codes  [N, K/2]  E2M1 pairs, K-major (checkpoint order, untouched)
//   SFA/SFB  128x4 tiles of 512 bytes (row-block major), one tile = the scale
//            factors of a 128-row x 64-column operand slab = exactly the
//            shared-memory image tcgen05.cp 32x128b.warpx4 copies to TMEM.
//
// One CTA computes a 128 x BLOCK_N output tile.  Per 256-element K step the
// producer warp lands A (128 rows x 128 B, 128B-swizzled) and B (BLOCK_N rows)
// by TMA and the two scale slabs by bulk copies; the MMA warp copies the scale
// factors to TMEM and issues four K=64 MMAs; four epilogue warps read the fp32
// accumulator from TMEM, scale by g*s2, convert to bf16 and store.
//
// Every mbarrier wait is bounded: on expiry the kernel writes a code to
// *status, abandons the tile, still frees its TMEM and returns.
#include <cuda_bf16.h>

#include <mutex>

#include "engine.h"
#include "gemm_epilogue.cuh"
#include "nvfp4_codec.cuh"

namespace q35b {
namespace {

constexpr int kBlockM = 128;
constexpr int kBlockKBytes = 128;        // one 128B swizzle row = 256 FP4 elements
constexpr int kMmaPerStage = 4;          // four K=64 MMAs per stage
constexpr int kSfChunk = 512;            // scale factors of 128 rows x 64 columns
constexpr int kThreads = 192;            // warp 0 TMA, warp 1 MMA, warps 2..5 epilogue
constexpr uint32_t kWaitLimit = 1u << 20;  // try_wait polls before giving up (well under a second)

enum StatusCode : unsigned { kStatusProducerWait = 1, kStatusMmaWait = 2, kStatusEpilogueWait = 3 };

template <int BLOCK_N>
struct Cfg {
  static constexpr int kStages = (BLOCK_N == 256) ? 4 : 6;
  static constexpr int kABytes = kBlockM * kBlockKBytes;
  static constexpr int kBBytes = BLOCK_N * kBlockKBytes;
  static constexpr int kSfaBytes = kMmaPerStage * kSfChunk;
  static constexpr int kSfbChunks = (BLOCK_N + 127) / 128;
  static constexpr int kSfbBytes = kSfbChunks * kMmaPerStage * kSfChunk;
  static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
  static constexpr int kAccCols = BLOCK_N;
  static constexpr int kSfaCols = kMmaPerStage * 4;
  static constexpr int kSfbCols = kMmaPerStage * 4 * kSfbChunks;
  static constexpr int kTmemCols = (kAccCols + kSfaCols + kSfbCols) <= 128 ? 128 : ((kAccCols + kSfaCols + kSfbCols) <= 256 ? 256 : 512);
};

// ---- PTX wrappers -----------------------------------------------------------

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

// Bounded wait on a phase parity; false when the limit ran out.
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

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
    "{\n\t.reg .pred p;\n\t"
    "elect.sync _|p, 0xffffffff;\n\t"
    "selp.u32 %0, 1, 0, p;\n\t}"
    : "=r"(pred));
  return pred != 0;
}

// Shared-memory matrix descriptor (tcgen05): K-major operand, 128B swizzle,
// 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_k_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3ffffu) >> 4);         // start address
  d |= static_cast<uint64_t>(0) << 16;                         // leading byte offset (unused for swizzled K-major)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;                 // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;                         // descriptor version (Blackwell)
  d |= static_cast<uint64_t>(2) << 61;                         // SWIZZLE_128B
  return d;
}

// Descriptor of a scale-factor slab for tcgen05.cp: no swizzle, 8 rows of 16
// bytes per core matrix, core matrices 128 bytes apart.
__device__ __forceinline__ uint64_t desc_sf(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(128 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}

// Instruction descriptor, kind::mxf4nvf4: A,B = E2M1 (1), K-major, UE4M3
// scale factors (0), M = 128, N = BLOCK_N, dense K = 64.
template <int BLOCK_N>
__device__ __forceinline__ uint32_t instr_desc() {
  uint32_t d = 0;
  d |= 1u << 7;                                  // a_format = E2M1
  d |= 1u << 10;                                 // b_format = E2M1
  d |= static_cast<uint32_t>(BLOCK_N >> 3) << 17;  // n_dim
  d |= 0u << 23;                                 // scale format UE4M3
  d |= static_cast<uint32_t>(kBlockM >> 4) << 24;  // m_dim
  return d;
}

__device__ __forceinline__ void umma_mxf4nvf4(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
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

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
      "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
      "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
      "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
    : "r"(taddr)
    : "memory");
}

// ---- kernel -------------------------------------------------------------------

template <int BLOCK_N>
__global__ void __launch_bounds__(kThreads, 1)
gemm_w4a4_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         const uint8_t * __restrict__ sfa, const uint8_t * __restrict__ sfb,
                         const float * __restrict__ g_dev, const GemmEpilogue ep, int m, int n, int k_bytes,
                         int sfb_row_blocks, __nv_bfloat16 * __restrict__ c, int ldc, unsigned int * status) {
  using C = Cfg<BLOCK_N>;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment for the 128B-swizzled operand tiles.
  uint8_t * smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t * smem_a = smem;
  uint8_t * smem_b = smem_a + C::kStages * C::kABytes;
  uint8_t * smem_sfa = smem_b + C::kStages * C::kBBytes;
  uint8_t * smem_sfb = smem_sfa + C::kStages * C::kSfaBytes;
  uint64_t * bars = reinterpret_cast<uint64_t *>(smem_sfb + C::kStages * C::kSfbBytes);
  // bars[0..S) full, bars[S..2S) empty, bars[2S] accumulator ready; then the TMEM base word.
  uint32_t * tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * C::kStages + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tile_n = blockIdx.x;
  const int tile_m = blockIdx.y;
  const int sf_col_blocks = k_bytes >> 5;                        // K/64: 512-byte scale tiles per row block
  const int k_steps = (sf_col_blocks + kMmaPerStage - 1) / kMmaPerStage;

  // Launched with programmatic stream serialisation: the grid may be scheduled under the tail of the previous kernel,
  // but reads and writes nothing before that kernel is complete.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // A tile that finds an error already recorded does nothing: after one expired wait the rest of the grid drains.
  __shared__ unsigned int s_abort;
  if (threadIdx.x == 0) s_abort = *reinterpret_cast<volatile unsigned int *>(status);
  __syncthreads();
  if (s_abort != 0u) return;

  if (threadIdx.x == 0) {
    for (int i = 0; i < C::kStages; ++i) {
      mbar_init(smem_u32(bars + i), 1);
      mbar_init(smem_u32(bars + C::kStages + i), 1);
    }
    mbar_init(smem_u32(bars + 2 * C::kStages), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(static_cast<uint32_t>(C::kTmemCols))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_acc = tmem_base;
  const uint32_t tmem_sfa = tmem_base + C::kAccCols;
  const uint32_t tmem_sfb = tmem_sfa + C::kSfaCols;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (elect_one()) {
      const uint8_t * sfa_rb = sfa + static_cast<size_t>(tile_m) * sf_col_blocks * kSfChunk;
      for (int ks = 0; ks < k_steps; ++ks) {
        const int stage = ks % C::kStages;
        const uint32_t phase = (ks / C::kStages) & 1;
        if (!mbar_wait(smem_u32(bars + C::kStages + stage), phase ^ 1)) {
          atomicExch(status, kStatusProducerWait);
          break;
        }
        const int valid = min(kMmaPerStage, sf_col_blocks - ks * kMmaPerStage);
        int sfb_valid_chunks = 0;
#pragma unroll
        for (int i = 0; i < C::kSfbChunks; ++i) {
          if (tile_n * C::kSfbChunks + i < sfb_row_blocks) ++sfb_valid_chunks;
        }
        const uint32_t full = smem_u32(bars + stage);
        const uint32_t tx = C::kABytes + C::kBBytes + valid * kSfChunk * (1 + sfb_valid_chunks);
        mbar_expect_tx(full, tx);
        tma_load_2d(smem_u32(smem_a + stage * C::kABytes), &tmap_a, full, ks * kBlockKBytes, tile_m * kBlockM);
        tma_load_2d(smem_u32(smem_b + stage * C::kBBytes), &tmap_b, full, ks * kBlockKBytes, tile_n * BLOCK_N);
        bulk_load(smem_u32(smem_sfa + stage * C::kSfaBytes), sfa_rb + static_cast<size_t>(ks) * kMmaPerStage * kSfChunk,
                  valid * kSfChunk, full);
#pragma unroll
        for (int i = 0; i < C::kSfbChunks; ++i) {
          const int rb = tile_n * C::kSfbChunks + i;
          if (rb < sfb_row_blocks) {
            bulk_load(smem_u32(smem_sfb + stage * C::kSfbBytes + i * kMmaPerStage * kSfChunk),
                      sfb + (static_cast<size_t>(rb) * sf_col_blocks + static_cast<size_t>(ks) * kMmaPerStage) * kSfChunk,
                      valid * kSfChunk, full);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (elect_one()) {
      const uint32_t idesc = instr_desc<BLOCK_N>();
      bool ok = true;
      for (int ks = 0; ks < k_steps && ok; ++ks) {
        const int stage = ks % C::kStages;
        const uint32_t phase = (ks / C::kStages) & 1;
        if (!mbar_wait(smem_u32(bars + stage), phase)) {
          atomicExch(status, kStatusMmaWait);
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int valid = min(kMmaPerStage, sf_col_blocks - ks * kMmaPerStage);
        const uint32_t a_base = smem_u32(smem_a + stage * C::kABytes);
        const uint32_t b_base = smem_u32(smem_b + stage * C::kBBytes);
        const uint32_t sfa_base = smem_u32(smem_sfa + stage * C::kSfaBytes);
        const uint32_t sfb_base = smem_u32(smem_sfb + stage * C::kSfbBytes);
        for (int j = 0; j < valid; ++j) {
          utccp_sf(tmem_sfa + j * 4, desc_sf(sfa_base + j * kSfChunk));
#pragma unroll
          for (int i = 0; i < C::kSfbChunks; ++i) {
            utccp_sf(tmem_sfb + (j * C::kSfbChunks + i) * 4, desc_sf(sfb_base + (i * kMmaPerStage + j) * kSfChunk));
          }
        }
        for (int j = 0; j < valid; ++j) {
          umma_mxf4nvf4(tmem_acc, desc_k_sw128(a_base + j * 32), desc_k_sw128(b_base + j * 32), idesc,
                        tmem_sfa + j * 4, tmem_sfb + j * C::kSfbChunks * 4, (ks | j) != 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(bars + C::kStages + stage));  // frees the stage when these MMAs and copies retire
      }
      if (ok) umma_commit(smem_u32(bars + 2 * C::kStages));  // accumulator complete
    }
  } else {
    // ---------------- epilogue: TMEM -> registers -> bf16 -> global ----------------
    const int quarter = warp & 3;                 // TMEM lanes this warp may touch
    const int row = tile_m * kBlockM + quarter * 32 + lane;
    const bool ready = mbar_wait(smem_u32(bars + 2 * C::kStages), 0);
    if (!ready) {
      if (lane == 0) atomicExch(status, kStatusEpilogueWait);
    } else {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float g = __ldg(g_dev);
      const float q_g = ep.q_g != nullptr ? __ldg(ep.q_g) : 1.0f;
      const uint32_t taddr = tmem_acc + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < BLOCK_N; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(taddr + c0, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (row < m) gemm_store_chunk32(r, row, tile_n * BLOCK_N + c0, n, g, ep, c, ldc, true, q_g);
      }
    }
  }

  gemm_signal_peers(ep, true);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(static_cast<uint32_t>(C::kTmemCols))
                 : "memory");
  }
}

// ---- host side ---------------------------------------------------------------

}  // namespace

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void * p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  });
  return fn;
}

// 2-D map over a K-major code matrix [rows, k_bytes] of bytes; box = box_rows x 128 bytes, 128B swizzle.
// Shared with the streaming decode kernel, whose tiles are 128-row boxes of the same matrix.
int make_code_map(CUtensorMap * map, const void * base, int rows, int k_bytes, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return fail(Q35B_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the CUDA driver.");
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k_bytes), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k_bytes)};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kBlockKBytes), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    return fail(Q35B_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult " + std::to_string(static_cast<int>(r)) + ".");
  }
  return Q35B_OK;
}

namespace {

template <int BLOCK_N>
int launch_tile(const q35b_weight * w, const CUtensorMap & tmap_a, const uint8_t * a_scales, const float * g_dev, int m,
                void * c, int ldc, const GemmEpilogue & ep, unsigned int * status, cudaStream_t s) {
  using C = Cfg<BLOCK_N>;
  static std::atomic<bool> attr_set[64];
  auto kernel = gemm_w4a4_tcgen05_kernel<BLOCK_N>;
  if (!attr_set[w->device & 63].load(std::memory_order_acquire)) {
    // idempotent, so two threads getting here together is harmless
    Q35B_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes),
                  "cudaFuncSetAttribute(gemm smem)");
    attr_set[w->device & 63].store(true, std::memory_order_release);
  }
  const dim3 grid((w->rows + BLOCK_N - 1) / BLOCK_N, (m + kBlockM - 1) / kBlockM);
  const cudaError_t le = launch_pdl(kernel, grid, dim3(kThreads), C::kSmemBytes, s, tmap_a,
                                    BLOCK_N == 256 ? w->tmap_codes_256 : w->tmap_codes_128, a_scales, w->scales_tiled, g_dev, ep, m,
                                    w->rows, w->k / 2, (w->rows + 127) / 128, static_cast<__nv_bfloat16 *>(c), ldc, status);
  count_launch();
  Q35B_CUDA_TRY(le, "gemm_w4a4_tcgen05_kernel launch");
  return Q35B_OK;
}

// What the GEMM entry points use as *status when the caller passes none: one word per device inside the library
// (no allocation anywhere on that path).
__device__ unsigned int g_default_status;

}  // namespace

int default_status_word(unsigned int ** out) {
  static std::mutex mutex;
  static unsigned int * word[64] = {nullptr};
  int dev = 0;
  Q35B_CUDA_TRY(cudaGetDevice(&dev), "cudaGetDevice");
  if (dev < 0 || dev >= 64) return fail(Q35B_ERR_ARGUMENT, "Device ordinal out of range.");
  std::lock_guard<std::mutex> lock(mutex);
  if (word[dev] == nullptr) {
    // the symbol's name is only a handle in host code; its address on the current device comes from the runtime
    void * p = nullptr;
    Q35B_CUDA_TRY(cudaGetSymbolAddress(&p, g_default_status), "cudaGetSymbolAddress(default status word)");
    word[dev] = static_cast<unsigned int *>(p);
  }
  *out = word[dev];
  return Q35B_OK;
}

}  // namespace q35b

extern "C" int q35b_gemm_default_status(unsigned int * status_out) {
  using namespace q35b;
  if (status_out == nullptr) return fail(Q35B_ERR_ARGUMENT, "Null status pointer.");
  unsigned int * word = nullptr;
  if (const int st = default_status_word(&word)) return st;
  Q35B_CUDA_TRY(cudaMemcpy(status_out, word, sizeof(unsigned int), cudaMemcpyDeviceToHost), "cudaMemcpy(default status word)");
  if (*status_out != 0u) Q35B_CUDA_TRY(cudaMemset(word, 0, sizeof(unsigned int)), "cudaMemset(default status word)");
  return Q35B_OK;
}

namespace q35b {

int launch_gemm_w4a4(const q35b_weight * w, const uint8_t * a_codes, const uint8_t * a_scales_tiled, const float * g_dev,
                     int m, void * c_bf16, int ldc, const void * residual_bf16, int ldr, unsigned int * status_dev,
                     cudaStream_t s, const GemmQuantOut * qout, const GemmGather * gather) {
  if (w == nullptr || a_codes == nullptr || a_scales_tiled == nullptr || g_dev == nullptr ||
      (c_bf16 == nullptr && qout == nullptr)) {
    return fail(Q35B_ERR_ARGUMENT, "NVFP4 prefill projection received a null device buffer.");
  }
  const int out_cols = w->gate_up ? w->rows / 2 : w->rows;
  if (m <= 0 || (qout == nullptr && ldc < out_cols)) return fail(Q35B_ERR_SHAPE, "Invalid dimensions for NVFP4 prefill projection.");
  if (qout != nullptr) {
    if (!w->gate_up) return fail(Q35B_ERR_ARGUMENT, "NVFP4 output of the prefill projection needs a gate/up weight.");
    if (qout->codes == nullptr || qout->scales_tiled == nullptr || qout->g_dev == nullptr) {
      return fail(Q35B_ERR_ARGUMENT, "NVFP4 prefill projection received a null device buffer.");
    }
    if ((out_cols % 64) != 0) return fail(Q35B_ERR_SHAPE, "NVFP4 output of the prefill projection needs rows / 2 to be a multiple of 64.");
    if ((w->row_begin % 128) != 0 || qout->total_cols < w->row_begin / 2 + out_cols || (qout->total_cols % 64) != 0) {
      return fail(Q35B_ERR_SHAPE, "NVFP4 output of the prefill projection: the shard's columns do not fit the given width.");
    }
    if ((reinterpret_cast<uintptr_t>(qout->codes) & 7u) != 0) {
      return fail(Q35B_ERR_ARGUMENT, "NVFP4 prefill projection buffers must be 16-byte aligned.");
    }
  }
  if (residual_bf16 != nullptr && (w->gate_up || ldr < w->rows)) {
    return fail(Q35B_ERR_ARGUMENT, "Invalid residual for NVFP4 prefill projection.");
  }
  GemmEpilogue ep;
  ep.s2 = w->s2;
  ep.s2_up = w->s2_up;
  ep.gate_up = w->gate_up ? 1 : 0;
  ep.residual = static_cast<const __nv_bfloat16 *>(residual_bf16);
  ep.ldr = ldr;
  if (qout != nullptr) {
    ep.q_codes = qout->codes + w->row_begin / 4;   // two output columns per byte, two weight rows per output column
    ep.q_scales = qout->scales_tiled;
    ep.q_g = qout->g_dev;
    ep.q_slots = round_up_int(qout->total_cols / 16, 4);
    ep.q_ld = qout->total_cols / 2;
    ep.q_slot0 = w->row_begin / 32;
  }
  if (gather != nullptr) {
    static_assert(sizeof(gather->peer_c) / sizeof(gather->peer_c[0]) == GemmEpilogue::kMaxPeers, "peer table size");
    if (qout != nullptr || residual_bf16 != nullptr) return fail(Q35B_ERR_ARGUMENT, "The gathering NVFP4 prefill projection takes no residual and writes BF16.");
    ep.n_peers = gather->n_peers;
    for (int i = 0; i < gather->n_peers; ++i) {
      ep.peer_c[i] = static_cast<__nv_bfloat16 *>(gather->peer_c[i]);
      ep.peer_flag[i] = gather->peer_flag[i];
    }
    ep.done_counter = gather->done_counter;
    ep.epoch = gather->epoch;
    ep.send_seq = gather->send_seq;
    // whole-row forwarding moves aligned 32-byte pieces; any other geometry takes the per-lane peer stores
    bool aligned = (ldc % 16) == 0 && (out_cols % 16) == 0 && (reinterpret_cast<uintptr_t>(c_bf16) & 31u) == 0;
    for (int i = 0; i < gather->n_peers; ++i) aligned = aligned && (reinterpret_cast<uintptr_t>(gather->peer_c[i]) & 31u) == 0;
    ep.forward_rows = aligned ? 1 : 0;
  }
  if ((w->k % 64) != 0) return fail(Q35B_ERR_SHAPE, "NVFP4 W4A4 GEMM needs cols to be a multiple of 64.");
  if ((reinterpret_cast<uintptr_t>(a_codes) & 15u) != 0 || (reinterpret_cast<uintptr_t>(a_scales_tiled) & 15u) != 0) {
    return fail(Q35B_ERR_ARGUMENT, "NVFP4 prefill projection buffers must be 16-byte aligned.");
  }
  if (w->rows == 0) return Q35B_OK;
  if (const int st = check_weight_device(w)) return st;
  if (!w->has_maps) return fail(Q35B_ERR_ARGUMENT, "NVFP4 weight has no tensor maps (it was not built by q35b_weight_create*).");
  if (status_dev == nullptr) {
    // the library's own word: kernels only ever write a nonzero code into it, q35b_gemm_default_status reads and
    // clears it (no memset in front of the launch: it would sit between this kernel and the one it overlaps with)
    if (const int st = default_status_word(&status_dev)) return st;
  }
  // Large problems: pairs of CTAs on 256 x 256 tiles, persistent (gemm_w4a4_2cta.cu).
  if (gemm_2cta_eligible(w, m)) {
    return launch_gemm_w4a4_2cta(w, a_codes, a_scales_tiled, g_dev, m, c_bf16, ldc, ep, status_dev, s);
  }
  // Up to 128 tokens: the weight streams through the 128-row side of the tile, every SM takes row blocks
  // (gemm_wstream.cu); bound by HBM, not by the tensor pipe.
  if (qout == nullptr && gather == nullptr && gemm_wstream_eligible(w, m)) {
    return launch_gemm_wstream(w, a_codes, a_scales_tiled, g_dev, m, c_bf16, ldc, residual_bf16, ldr, status_dev, s);
  }
  CUtensorMap tmap_a;
  if (const int st = make_code_map(&tmap_a, a_codes, m, w->k / 2, kBlockM)) return st;
  // Small problems get narrower tiles so that more SMs have work.
  const long tiles256 = static_cast<long>((w->rows + 255) / 256) * ((m + 127) / 128);
  if (tiles256 >= sm_count() || w->rows <= 128) {
    if (w->rows > 128) return launch_tile<256>(w, tmap_a, a_scales_tiled, g_dev, m, c_bf16, ldc, ep, status_dev, s);
  }
  return launch_tile<128>(w, tmap_a, a_scales_tiled, g_dev, m, c_bf16, ldc, ep, status_dev, s);
}

}  // namespace q35b
