// W4A4 prefill GEMM, 2-CTA persistent variant for sm_100a.
//
// Same contract as gemm_w4a4_tcgen05.cu (C[M,N] bf16 = (Aq . Wq^T) * g * s2, replacing
// run_nvfp4_cublaslt_prefill_projection_device, src/runtime/cuda_bench.cu:1056-1167), built for large M:
//
//   - a pair of CTAs on neighbouring SMs (cluster of 2) computes one 256 x 192 output tile with
//     tcgen05.mma.cta_group::2: each CTA stages only its own 128 rows of A and its own 96 rows of B.  No TMA
//     multicast is used: every load lands in the issuing CTA's own shared memory;
//   - N = 192 leaves room in TMEM (2 x 192 accumulator columns + 48 scale-factor columns <= 512) for TWO
//     accumulators, so the epilogue of one tile overlaps the MMAs of the next;
//   - persistent: 74 pairs walk the tile list (M-tiles fastest, so the pairs in flight share B tiles in L2);
//     barriers, TMEM and tensor maps are set up once per CTA, not once per tile;
//   - per K step (256 FP4 columns) a CTA lands A 16 KB + B 12 KB (128B-swizzled TMA boxes) and the scale
//     factors SFA 2 KB + SFB 4 KB (TMA boxes over the 512-byte scale tiles); 6-stage ring.  A 192-row tile
//     starts either on a 128-row scale tile or 64 rows into one: it always takes two scale tiles, and the MMA's
//     SFB address is moved by two TMEM columns (= 64 rows) in the second case;
//   - the leader CTA's MMA thread copies scale factors to TMEM in both CTAs (tcgen05.cp.cta_group::2) and
//     issues four M=256, N=192, K=64 block-scaled MMAs per K step; tcgen05.commit multicasts stage release and
//     accumulator-ready to both CTAs;
//   - four epilogue warps per CTA drain that CTA's 128 x 192 fp32 accumulator half from TMEM, scale, convert
//     and store BF16.
//
// Every mbarrier wait is bounded; an expired wait records a code in *status and the role stops, the kernel
// still runs to its cluster barrier and frees TMEM.
#include <cuda_bf16.h>

#include "engine.h"
#include "gemm_epilogue.cuh"
#include "nvfp4_codec.cuh"

namespace q35b {
namespace {

#ifndef Q35B_TILE_N
#define Q35B_TILE_N 256
#endif
constexpr int kCtaRows = 128;            // rows of A staged per CTA
constexpr int kTileM = 256;              // output tile of the pair: 256 tokens ...
constexpr int kTileN = Q35B_TILE_N;      // ... by 192 (two accumulators in TMEM) or 256 (one) weight rows
static_assert(kTileN == 192 || kTileN == 256, "tile width");
constexpr int kAccs = kTileN == 192 ? 2 : 1;  // accumulators that fit beside the scale factors in 512 TMEM columns
constexpr int kCtaBRows = kTileN / 2;    // rows of B staged per CTA
constexpr int kStepBytes = 128;          // 256 FP4 columns
constexpr int kMmaPerStage = 4;
constexpr int kSfChunk = 512;
constexpr int kABytes = kCtaRows * kStepBytes;
constexpr int kBBytes = kCtaBRows * kStepBytes;
constexpr int kSfaBytes = kMmaPerStage * kSfChunk;
constexpr int kSfbBytes = 2 * kMmaPerStage * kSfChunk;
constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;   // 34816
#ifndef Q35B_STAGES
#define Q35B_STAGES (Q35B_TILE_N == 192 ? 6 : 5)
#endif
constexpr int kStages = Q35B_STAGES;
// Epilogue warps per CTA (template parameter of the kernel), a multiple of four: kEpilogueWarps / 4 per TMEM lane
// quarter, each draining a column slice of the accumulator.  Sixteen for the epilogues that do arithmetic on what they
// drain (SiLU, NVFP4 output) and for launches that forward rows to peers (their 64-column grain); eight for the plain
// and the residual epilogue, which measured 1-5 % faster with fewer, wider warps.
constexpr int kEpiWarpsWide = kTileN == 192 ? 12 : 16;
constexpr int kEpiWarpsPlain = kTileN == 192 ? 12 : 8;
constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
static_assert(kStages * kStageBytes + 1024 + 256 <= 227 * 1024, "shared memory");
constexpr int kAccCols = kAccs * kTileN;
constexpr int kSfaCols = kMmaPerStage * 4;
constexpr int kSfbCols = kMmaPerStage * 8;
constexpr int kTmemCols = 512;
constexpr uint32_t kWaitLimit = 1u << 20;
constexpr uint32_t kPeerMask = 0xFEFFFFFFu;  // clears the CTA-rank bit of a shared::cluster address: the pair's leader

enum StatusCode : unsigned { kProducerWait = 21, kMmaWait = 22, kEpilogueWait = 23, kMmaDrainWait = 24 };

__device__ __forceinline__ uint32_t smem_u32(const void * p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Arrive on the barrier at the same offset in CTA `cta` of the cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar, uint32_t cta) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(bar), "r"(cta));
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kWaitLimit; ++i) {
    uint32_t ok;
    asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
    if (ok) return true;
  }
  return false;
}
// TMA box load into this CTA's shared memory, completion bytes go to the pair leader's barrier.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap * map, uint32_t leader_bar, int x, int y) {
  asm volatile(
    "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::
      "r"(dst),
    "l"(map), "r"(leader_bar), "r"(x), "r"(y)
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
__device__ __forceinline__ uint64_t desc_k_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
__device__ __forceinline__ uint64_t desc_sf(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(128 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}
// kind::mxf4nvf4 instruction descriptor: E2M1 x E2M1, K-major, UE4M3 scales, M = 256 (pair), N = 192.
__device__ __forceinline__ uint32_t instr_desc_pair() {
  uint32_t d = 0;
  d |= 1u << 7;
  d |= 1u << 10;
  d |= static_cast<uint32_t>(kTileN >> 3) << 17;
  d |= static_cast<uint32_t>(kTileM >> 4) << 24;
  return d;
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t tmem_sfa,
                                          uint32_t tmem_sfb, uint32_t accumulate) {
  asm volatile(
    "{\n\t.reg .pred p;\n\t"
    "setp.ne.b32 p, %4, 0;\n\t"
    "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(tmem_d),
    "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
    : "memory");
}
__device__ __forceinline__ void utccp_sf_pair(uint32_t tmem_dst, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmem_dst), "l"(sdesc) : "memory");
}
// Arrive (once all earlier tcgen05 work of this thread has retired) on the barrier at this offset in both CTAs.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"(static_cast<uint16_t>(3))
               : "memory");
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
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <int kEpilogueWarps>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__((2 + kEpilogueWarps) * 32, 1)
gemm_w4a4_2cta_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
                      const float * __restrict__ g_dev, const GemmEpilogue ep, int m, int n, int k_bytes, int m_tiles, int num_tiles,
                      __nv_bfloat16 * __restrict__ c, int ldc, unsigned int * status) {
  constexpr int kEpiCols = kTileN / (kEpilogueWarps / 4);  // columns drained by one epilogue warp
  static_assert(kEpilogueWarps % 4 == 0 && kEpiCols % 32 == 0 && kEpiCols * (kEpilogueWarps / 4) == kTileN, "epilogue column split");
  extern __shared__ uint8_t smem_raw[];
  uint8_t * smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t * smem_a = smem;
  uint8_t * smem_b = smem_a + kStages * kABytes;
  uint8_t * smem_sfa = smem_b + kStages * kBBytes;
  uint8_t * smem_sfb = smem_sfa + kStages * kSfaBytes;
  uint64_t * bars = reinterpret_cast<uint64_t *>(smem_sfb + kStages * kSfbBytes);
  uint64_t * full = bars;                       // used in the leader: bytes of both CTAs
  uint64_t * empty = bars + kStages;            // in each CTA: its own stages are free
  uint64_t * tmem_full = bars + 2 * kStages;    // [2] in each CTA: accumulator b is complete
  uint64_t * drained = tmem_full + 2;           // [2] in each CTA: its epilogue warps have read accumulator b out of TMEM
  uint64_t * peer_drained = drained + 2;        // [2] used in the leader: the partner CTA has drained accumulator b
  uint32_t * tmem_slot = reinterpret_cast<uint32_t *>(peer_drained + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int sf_col_blocks = k_bytes >> 5;
  const int k_steps = (sf_col_blocks + kMmaPerStage - 1) / kMmaPerStage;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(smem_u32(full + i), 1);
      mbar_init(smem_u32(empty + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(tmem_full + i), 1);
      mbar_init(smem_u32(drained + i), kEpilogueWarps);
      mbar_init(smem_u32(peer_drained + i), 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(static_cast<uint32_t>(kTmemCols))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync();  // both CTAs' barriers exist before anything signals across the pair
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_acc = tmem_base;
  const uint32_t tmem_sfa = tmem_base + kAccCols;
  const uint32_t tmem_sfb = tmem_sfa + kSfaCols;
  // Launched with programmatic stream serialisation: everything above (barriers, TMEM, the pair's rendezvous) may run
  // under the tail of the previous kernel; nothing below touches global memory before that kernel is complete.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // An error recorded by an earlier launch: run no tiles (every CTA still goes through alloc, barriers, dealloc).
  const bool aborted = *reinterpret_cast<volatile unsigned int *>(status) != 0u;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (elect_one() && !aborted) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const int tm = tile % m_tiles;
        const int tn = tile / m_tiles;
        const int a_row = tm * kTileM + static_cast<int>(rank) * kCtaRows;
        const int b_row = tn * kTileN + static_cast<int>(rank) * kCtaBRows;
        const int sfa_chunk0 = (tm * 2 + static_cast<int>(rank)) * sf_col_blocks;
        const int sfb_rb = (tn * kTileN) >> 7;  // first 128-row scale tile the 192 rows touch
        const int sfb_chunk0 = sfb_rb * sf_col_blocks;
        const int sfb_chunk1 = (sfb_rb + 1) * sf_col_blocks;
        for (int ks = 0; ks < k_steps; ++ks) {
          if (!mbar_wait(smem_u32(empty + stage), phase ^ 1)) {
            atomicExch(status, kProducerWait);
            ok = false;
            break;
          }
          const uint32_t leader_full = smem_u32(full + stage) & kPeerMask;
          if (rank == 0) mbar_expect_tx(smem_u32(full + stage), 2 * kStageBytes);
          tma_load_2d_pair(smem_u32(smem_a + stage * kABytes), &tmap_a, leader_full, ks * kStepBytes, a_row);
          tma_load_2d_pair(smem_u32(smem_b + stage * kBBytes), &tmap_b, leader_full, ks * kStepBytes, b_row);
          tma_load_2d_pair(smem_u32(smem_sfa + stage * kSfaBytes), &tmap_sfa, leader_full, 0, sfa_chunk0 + ks * kMmaPerStage);
          tma_load_2d_pair(smem_u32(smem_sfb + stage * kSfbBytes), &tmap_sfb, leader_full, 0, sfb_chunk0 + ks * kMmaPerStage);
          tma_load_2d_pair(smem_u32(smem_sfb + stage * kSfbBytes + kSfaBytes), &tmap_sfb, leader_full, 0,
                           sfb_chunk1 + ks * kMmaPerStage);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (rank == 0 && elect_one() && !aborted) {
      const uint32_t idesc = instr_desc_pair();
      int stage = 0;
      uint32_t phase = 0;
      uint32_t li = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++li) {
        const uint32_t ab = li % kAccs;
        const uint32_t acc_phase = (li / kAccs) & 1;
        if (!mbar_wait(smem_u32(drained + ab), acc_phase ^ 1) || !mbar_wait(smem_u32(peer_drained + ab), acc_phase ^ 1)) {
          atomicExch(status, kMmaDrainWait);
          ok = false;
          break;
        }
        const uint32_t acc = tmem_acc + ab * kTileN;
        const uint32_t sfb_off = ((static_cast<uint32_t>(tile / m_tiles) * kTileN) & 127u) >> 5;  // 0 or 2 columns
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        for (int ks = 0; ks < k_steps; ++ks) {
          if (!mbar_wait(smem_u32(full + stage), phase)) {
            atomicExch(status, kMmaWait);
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const int valid = min(kMmaPerStage, sf_col_blocks - ks * kMmaPerStage);
          // descriptors of this stage: the address field counts 16-byte units, so stepping a descriptor is an add
          const uint64_t a_desc = desc_k_sw128(smem_u32(smem_a + stage * kABytes));
          const uint64_t b_desc = desc_k_sw128(smem_u32(smem_b + stage * kBBytes));
          const uint64_t sfa_desc = desc_sf(smem_u32(smem_sfa + stage * kSfaBytes));
          const uint64_t sfb_desc = desc_sf(smem_u32(smem_sfb + stage * kSfbBytes));
#pragma unroll
          for (int j = 0; j < kMmaPerStage; ++j) {
            if (j < valid) {
              utccp_sf_pair(tmem_sfa + j * 4, sfa_desc + j * (kSfChunk >> 4));
              utccp_sf_pair(tmem_sfb + j * 8, sfb_desc + j * (kSfChunk >> 4));
              utccp_sf_pair(tmem_sfb + j * 8 + 4, sfb_desc + (kSfaBytes >> 4) + j * (kSfChunk >> 4));
            }
          }
#pragma unroll
          for (int j = 0; j < kMmaPerStage; ++j) {
            if (j < valid) {
              umma_pair(acc, a_desc + j * 2, b_desc + j * 2, idesc, tmem_sfa + j * 4, tmem_sfb + j * 8 + sfb_off,
                        (ks | j) != 0 ? 1u : 0u);
            }
          }
          umma_commit_pair(smem_u32(empty + stage));
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit_pair(smem_u32(tmem_full + ab));
      }
    } else if (rank == 1 && elect_one() && !aborted) {
      // ---------------- drain forwarder (partner CTA): tells the leader when this CTA's epilogue warps have
      // read an accumulator out, so that none of them spends a cluster round trip on it ----------------
      uint32_t li = 0;
      for (int tile = pair; tile < num_tiles; tile += num_pairs, ++li) {
        const uint32_t ab = li % kAccs;
        if (!mbar_wait(smem_u32(drained + ab), (li / kAccs) & 1)) {
          atomicExch(status, kEpilogueWait);
          break;
        }
        mbar_arrive_cluster(smem_u32(peer_drained + ab), 0);
      }
    }
  } else {
    // ---------------- epilogue (both CTAs): this CTA's 128 rows of the pair's tile ----------------
    const int quarter = warp & 3;                 // TMEM lanes 32 * quarter .. + 31 (fixed by the warp's index)
    const int col_base = ((warp - 2) >> 2) * kEpiCols;
    const float g = __ldg(g_dev);
    const float q_g = ep.q_g != nullptr ? __ldg(ep.q_g) : 1.0f;
    uint32_t li = 0;
    bool ok = !aborted;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++li) {
      const int tm = tile % m_tiles;
      const int tn = tile / m_tiles;
      const uint32_t ab = li % kAccs;
      if (!mbar_wait(smem_u32(tmem_full + ab), (li / kAccs) & 1)) {
        if (lane == 0) atomicExch(status, kEpilogueWait);
        ok = false;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int row = tm * kTileM + static_cast<int>(rank) * kCtaRows + quarter * 32 + lane;
      const uint32_t taddr = tmem_acc + ab * kTileN + col_base + (static_cast<uint32_t>(quarter * 32) << 16);
      // read the warp's whole share into registers, give the accumulator back at once, then convert and store
      uint32_t r[kEpiCols / 32][32];
#pragma unroll
      for (int j = 0; j < kEpiCols / 32; ++j) tmem_ld32(taddr + 32 * j, r[j]);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(drained + ab));
      // plain BF16 output of a gathering launch: store locally, then forward whole rows; the fused epilogues (and a
      // launch without peers) store per lane
      const bool forward = ep.n_peers > 0 && !ep.gate_up && ep.forward_rows != 0;
      if (row < m) {
#pragma unroll
        for (int j = 0; j < kEpiCols / 32; ++j) {
          gemm_store_chunk32(r[j], row, tn * kTileN + col_base + 32 * j, n, g, ep, c, ldc, !forward, q_g);
        }
      }
      if (forward) {
        gemm_forward_rows_to_peers<kEpiCols>(ep, c, ldc, tm * kTileM + static_cast<int>(rank) * kCtaRows + quarter * 32, m,
                                             tn * kTileN + col_base, n, lane);
      }
    }
  }

  gemm_signal_peers(ep, !aborted);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync();  // neither CTA may leave while its partner can still signal its barriers or read its tiles
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(static_cast<uint32_t>(kTmemCols))
                 : "memory");
  }
}

}  // namespace

// 2-D map over a tiled scale array seen as [chunks, 128 x u32]: box = 4 consecutive 512-byte chunks.
int make_sf_map(CUtensorMap * map, const void * base, long long chunks) {
  using Fn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                          const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                          CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static Fn fn = nullptr;
  if (fn == nullptr) {
    void * p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) {
      return fail(Q35B_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the CUDA driver.");
    }
    fn = reinterpret_cast<Fn>(p);
  }
  const cuuint64_t dims[2] = {128, static_cast<cuuint64_t>(chunks)};
  const cuuint64_t strides[1] = {512};
  const cuuint32_t box[2] = {128, 4};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void *>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    return fail(Q35B_ERR_CUDA, "cuTensorMapEncodeTiled(scale factors) failed with CUresult " + std::to_string(static_cast<int>(r)) + ".");
  }
  return Q35B_OK;
}

int build_weight_maps(q35b_weight * w) {
  if (w->rows <= 0 || (w->k % 64) != 0) return Q35B_OK;  // such a weight never reaches a GEMM
  if (const int st = make_code_map(&w->tmap_codes_128, w->codes, w->rows, w->k / 2, 128)) return st;
  if (const int st = make_code_map(&w->tmap_codes_256, w->codes, w->rows, w->k / 2, 256)) return st;
  if (const int st = make_code_map(&w->tmap2_codes, w->codes, w->rows, w->k / 2, kCtaBRows)) return st;
  const long long chunks = static_cast<long long>((w->rows + 127) / 128) * (w->k / 64);
  if (const int st = make_sf_map(&w->tmap2_sf, w->scales_tiled, chunks)) return st;
  w->has_maps = true;
  return Q35B_OK;
}

bool gemm_2cta_eligible(const q35b_weight * w, int m) {
  return w->rows >= 192 && m >= 256 && (w->k % 64) == 0;
}

int launch_gemm_w4a4_2cta(const q35b_weight * w, const uint8_t * a_codes, const uint8_t * a_scales_tiled, const float * g_dev,
                          int m, void * c_bf16, int ldc, const GemmEpilogue & ep, unsigned int * status_dev,
                          cudaStream_t s) {
  static std::atomic<bool> attr_set[64];
  if (!attr_set[w->device & 63].load(std::memory_order_acquire)) {
    Q35B_CUDA_TRY(cudaFuncSetAttribute(gemm_w4a4_2cta_kernel<kEpiWarpsWide>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes),
                  "cudaFuncSetAttribute(2-CTA gemm smem)");
    Q35B_CUDA_TRY(cudaFuncSetAttribute(gemm_w4a4_2cta_kernel<kEpiWarpsPlain>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes),
                  "cudaFuncSetAttribute(2-CTA gemm smem)");
    attr_set[w->device & 63].store(true, std::memory_order_release);
  }
  CUtensorMap tmap_a, tmap_sfa;
  if (const int st = make_code_map(&tmap_a, a_codes, m, w->k / 2, kCtaRows)) return st;
  if (const int st = make_sf_map(&tmap_sfa, a_scales_tiled, static_cast<long long>((m + 127) / 128) * (w->k / 64))) return st;
  const int m_tiles = (m + kTileM - 1) / kTileM;
  const int n_tiles = (w->rows + kTileN - 1) / kTileN;
  const int num_tiles = m_tiles * n_tiles;
  const int pairs = std::max(1, std::min(num_tiles, sm_count() / 2));
  // plain and residual epilogues without peers: the narrow set of epilogue warps
  const bool plain = !ep.gate_up && ep.q_codes == nullptr && ep.n_peers == 0;
  const int epi_warps = plain ? kEpiWarpsPlain : kEpiWarpsWide;
  const auto kernel = plain ? gemm_w4a4_2cta_kernel<kEpiWarpsPlain> : gemm_w4a4_2cta_kernel<kEpiWarpsWide>;
  const cudaError_t le = launch_pdl(kernel, dim3(2 * pairs), dim3((2 + epi_warps) * 32), kSmemBytes, s, tmap_a, w->tmap2_codes,
                                    tmap_sfa, w->tmap2_sf, g_dev, ep, m, w->rows, w->k / 2, m_tiles, num_tiles,
                                    static_cast<__nv_bfloat16 *>(c_bf16), ldc, status_dev);
  count_launch();
  Q35B_CUDA_TRY(le, "gemm_w4a4_2cta_kernel launch");
  return Q35B_OK;
}

}  // namespace q35b
