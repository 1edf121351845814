// Prefill GEMM whose stores are the all-gather: rows of a projection are sharded over the GPUs of one box, every
// rank computes C[:, its rows] and its epilogue writes each BF16 vector into the full [M, N] matrix of every rank
// (its own with local stores, the others' with plain peer-memory stores over NVLink), so the transfer runs under
// the MMAs tile by tile and no separate collective follows.  Replaces the exchange step of the N-sharded prefill
// projection (one ncclAllGather of the BF16 slabs after the GEMM).
//
// A q35b_peer_buffer is the full output matrix of one rank plus a few words of flags, allocated with cudaMalloc so
// that it can be opened in the other ranks' processes through a CUDA IPC handle.  Completion: when the whole grid of
// a rank has stored (and fenced system-wide), its last CTA writes the launch's epoch into that rank's slot of every
// rank's flag words; q35b_peer_gather_wait then polls the local slots of all other ranks with a bounded wait.
// No TMA and no multicast touch peer memory: only st.global from the epilogue warps and one flag word per peer.
#include <cuda_bf16.h>

#include <algorithm>
#include <cstring>

#include "engine.h"
#include "gemm_epilogue.cuh"

struct q35b_peer_buffer {
  uint8_t * base = nullptr;
  size_t data_bytes = 0;
  size_t flags_offset = 0;
  int device = 0;
  bool owner = false;
  cudaIpcMemHandle_t handle{};
};

namespace q35b {
namespace {

constexpr int kMaxRanks = GemmEpilogue::kMaxPeers + 1;
constexpr size_t kFlagBytes = 256;  // [kMaxRanks] epoch slots, the owner's done counter, its send and wait counts
constexpr int kSendSeqWord = kMaxRanks + 1;  // sends this rank has signalled with a self-counted epoch
constexpr int kWaitSeqWord = kMaxRanks + 2;  // waits this rank has completed with a self-counted epoch
constexpr uint32_t kGatherWaitLimit = 1u << 22;
constexpr unsigned kStatusGatherWait = 31;

inline unsigned int * flag_words(const q35b_peer_buffer * b) { return reinterpret_cast<unsigned int *>(b->base + b->flags_offset); }

// One thread per rank: wait until that rank's slot carries this epoch (or a later one).  epoch == 0: the epoch is
// this rank's own count of such waits plus one (kept in the flag block, advanced here), which matches the senders'
// self-counted epochs as long as every rank sends and waits the same number of times: a captured wait can be
// replayed.
__global__ void peer_gather_wait_kernel(unsigned int * flags, int world, int rank, unsigned int epoch,
                                        unsigned int * status, uint32_t limit) {
  asm volatile("griddepcontrol.wait;" ::: "memory");  // launched under the tail of the kernel before it
  const int r = threadIdx.x;
  __shared__ unsigned int expected;
  if (r == 0) expected = epoch != 0u ? epoch : flags[kWaitSeqWord] + 1u;
  __syncthreads();
  const unsigned int want = expected;
  if (r < world && r != rank) {
    const volatile unsigned int * slot = flags + r;
    bool seen = false;
    for (uint32_t i = 0; i < limit; ++i) {
      if (static_cast<int>(*slot - want) >= 0) {
        __threadfence_system();  // the peer's matrix stores were fenced before its flag store
        seen = true;
        break;
      }
      __nanosleep(64);
    }
    if (!seen) atomicExch(status, kStatusGatherWait);
  }
  __syncthreads();
  if (r == 0 && epoch == 0u) flags[kWaitSeqWord] = want;
}

// Copies up to four 2-D byte regions of this rank's buffer to the same place in every other rank's buffer and
// then signals the epoch, with the protocol of the gathering GEMM (system-wide fence, CTA count, last CTA writes
// this rank's flag slot on every peer).  A thread moves 16-byte pieces: it reads one from local memory and stores
// it to each peer, so a warp's store instruction covers 512 contiguous bytes of one peer (whole 128-byte lines,
// the unit NVLink moves well).  Used where the producer kernel writes pieces too small to forward itself: the
// NVFP4 codes (8 bytes per row per thread) and scale bytes of the gate/up epilogue, and narrow BF16 shards.
struct PushRegion {
  unsigned long long offset;    // of the region's first byte inside the buffer
  unsigned long long ld;        // bytes between rows
  unsigned int row_pieces;      // 16-byte pieces per row
  unsigned int rows;
};
struct PushArgs {
  PushRegion region[4];
  int n_regions;
  int n_peers;
  uint8_t * local;
  uint8_t * peer[GemmEpilogue::kMaxPeers];
  unsigned int * peer_flag[GemmEpilogue::kMaxPeers];
  unsigned int * done_counter;
  unsigned int * send_seq;
  unsigned int epoch;
};

__global__ void __launch_bounds__(256) peer_push_kernel(const PushArgs a) {
  asm volatile("griddepcontrol.wait;" ::: "memory");  // the bytes to forward come from the kernel before
  constexpr int kUnroll = 4;
  const unsigned long long stride = static_cast<unsigned long long>(gridDim.x) * blockDim.x;
  for (int ri = 0; ri < a.n_regions; ++ri) {
    const PushRegion rg = a.region[ri];
    const unsigned long long pieces = static_cast<unsigned long long>(rg.rows) * rg.row_pieces;
    for (unsigned long long i0 = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < pieces;
         i0 += stride * kUnroll) {
      uint4 v[kUnroll];
      unsigned long long off[kUnroll];
      // loads first, then the stores: the stores of one piece never hold back the load of the next
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const unsigned long long i = i0 + u * stride;
        if (i < pieces) {
          off[u] = rg.offset + (i / rg.row_pieces) * rg.ld + (i % rg.row_pieces) * 16ull;
          v[u] = __ldcg(reinterpret_cast<const uint4 *>(a.local + off[u]));
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (i0 + u * stride < pieces) {
#pragma unroll
          for (int p = 0; p < GemmEpilogue::kMaxPeers; ++p) {
            if (p < a.n_peers) *reinterpret_cast<uint4 *>(a.peer[p] + off[u]) = v[u];
          }
        }
      }
    }
  }
  GemmEpilogue ep;
  ep.n_peers = a.n_peers;
#pragma unroll
  for (int p = 0; p < GemmEpilogue::kMaxPeers; ++p) ep.peer_flag[p] = a.peer_flag[p];
  ep.done_counter = a.done_counter;
  ep.epoch = a.epoch;
  ep.send_seq = a.send_seq;
  gemm_signal_peers(ep, true);
}

// A rank whose shard is empty (more ranks than 128-row blocks) computes nothing but still has to tell the others
// that its part of the epoch is complete.
__global__ void peer_signal_kernel(GemmEpilogue ep) {
  __shared__ unsigned int epoch;
  if (threadIdx.x == 0) {
    epoch = ep.epoch;
    if (epoch == 0u && ep.send_seq != nullptr) {
      epoch = *ep.send_seq + 1u;
      *ep.send_seq = epoch;
    }
  }
  __syncthreads();
  if (threadIdx.x < ep.n_peers) *reinterpret_cast<volatile unsigned int *>(ep.peer_flag[threadIdx.x]) = epoch;
}

}  // namespace
}  // namespace q35b

using namespace q35b;

int q35b_peer_buffer_create(size_t data_bytes, q35b_peer_buffer ** out) {
  if (out == nullptr || data_bytes == 0) return fail(Q35B_ERR_ARGUMENT, "Invalid peer buffer request.");
  *out = nullptr;
  auto * b = new q35b_peer_buffer();
  b->data_bytes = data_bytes;
  b->flags_offset = (data_bytes + 255) / 256 * 256;
  b->owner = true;
  cudaError_t e = cudaGetDevice(&b->device);
  if (e == cudaSuccess) e = cudaMalloc(&b->base, b->flags_offset + kFlagBytes);
  if (e == cudaSuccess) e = cudaMemset(b->base + b->flags_offset, 0, kFlagBytes);
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&b->handle, b->base);
  if (e != cudaSuccess) {
    if (b->base != nullptr) cudaFree(b->base);
    delete b;
    return fail_cuda(e, "allocating a peer buffer");
  }
  *out = b;
  return Q35B_OK;
}

size_t q35b_peer_buffer_handle_bytes(void) { return sizeof(cudaIpcMemHandle_t); }

int q35b_peer_buffer_export(const q35b_peer_buffer * b, void * handle_out) {
  if (b == nullptr || handle_out == nullptr || !b->owner) return fail(Q35B_ERR_ARGUMENT, "Only the owner of a peer buffer can export it.");
  memcpy(handle_out, &b->handle, sizeof(cudaIpcMemHandle_t));
  return Q35B_OK;
}

int q35b_peer_buffer_open(const void * handle, size_t data_bytes, q35b_peer_buffer ** out) {
  if (handle == nullptr || out == nullptr || data_bytes == 0) return fail(Q35B_ERR_ARGUMENT, "Invalid peer buffer handle.");
  *out = nullptr;
  auto * b = new q35b_peer_buffer();
  b->data_bytes = data_bytes;
  b->flags_offset = (data_bytes + 255) / 256 * 256;
  memcpy(&b->handle, handle, sizeof(cudaIpcMemHandle_t));
  void * p = nullptr;
  cudaError_t e = cudaGetDevice(&b->device);
  if (e == cudaSuccess) e = cudaIpcOpenMemHandle(&p, b->handle, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    delete b;
    return fail_cuda(e, "opening a peer buffer");
  }
  b->base = static_cast<uint8_t *>(p);
  *out = b;
  return Q35B_OK;
}

void * q35b_peer_buffer_data(const q35b_peer_buffer * b) { return b ? b->base : nullptr; }

void q35b_peer_buffer_destroy(q35b_peer_buffer * b) {
  if (b == nullptr) return;
  if (b->base != nullptr) {
    if (b->owner) {
      cudaFree(b->base);
    } else {
      cudaIpcCloseMemHandle(b->base);
    }
  }
  delete b;
}

int q35b_gemm_w4a4_bf16_allgather(const q35b_weight * w, const uint8_t * a_codes, const uint8_t * a_scales_tiled,
                                  const float * input_scale_dev, int m, q35b_peer_buffer * const * buffers, int world,
                                  int rank, int ldc, unsigned int epoch, unsigned int * status_dev, q35b_stream stream) {
  if (w == nullptr || buffers == nullptr || world < 1 || world > kMaxRanks || rank < 0 || rank >= world) {
    return fail(Q35B_ERR_ARGUMENT, "Invalid rank layout for the gathering NVFP4 prefill projection.");
  }
  const int out_cols = w->gate_up ? w->rows / 2 : w->rows;
  const int col0 = w->gate_up ? w->row_begin / 2 : w->row_begin;
  if (m <= 0 || ldc < col0 + out_cols) return fail(Q35B_ERR_SHAPE, "Invalid dimensions for NVFP4 prefill projection.");
  const size_t need = (static_cast<size_t>(m - 1) * ldc + col0 + out_cols) * sizeof(__nv_bfloat16);
  GemmGather gather;
  for (int r = 0; r < world; ++r) {
    if (buffers[r] == nullptr || buffers[r]->base == nullptr || buffers[r]->data_bytes < need) {
      return fail(Q35B_ERR_ARGUMENT, "A peer buffer of the gathering NVFP4 prefill projection is missing or too small.");
    }
    if (r == rank) continue;
    gather.peer_c[gather.n_peers] = reinterpret_cast<__nv_bfloat16 *>(buffers[r]->base) + col0;
    gather.peer_flag[gather.n_peers] = flag_words(buffers[r]) + rank;
    ++gather.n_peers;
  }
  gather.done_counter = flag_words(buffers[rank]) + kMaxRanks;
  gather.epoch = epoch;
  gather.send_seq = flag_words(buffers[rank]) + kSendSeqWord;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (w->rows == 0) {
    GemmEpilogue ep;
    ep.n_peers = gather.n_peers;
    for (int i = 0; i < gather.n_peers; ++i) ep.peer_flag[i] = gather.peer_flag[i];
    ep.epoch = epoch;
    ep.send_seq = gather.send_seq;
    peer_signal_kernel<<<1, 32, 0, s>>>(ep);
    count_launch();
    Q35B_CUDA_TRY(cudaGetLastError(), "peer_signal_kernel launch");
    return Q35B_OK;
  }
  // the closing count is left at zero by the last CTA of every launch (the flag block starts zeroed): no memset here
  auto * c = reinterpret_cast<__nv_bfloat16 *>(buffers[rank]->base) + col0;
  return launch_gemm_w4a4(w, a_codes, a_scales_tiled, input_scale_dev, m, c, ldc, nullptr, 0,
                          status_dev, s, nullptr, &gather);
}

int q35b_peer_gather_wait(q35b_peer_buffer * const * buffers, int world, int rank, unsigned int epoch,
                          unsigned int * status_dev, q35b_stream stream) {
  if (buffers == nullptr || world < 1 || world > kMaxRanks || rank < 0 || rank >= world || buffers[rank] == nullptr ||
      status_dev == nullptr) {
    return fail(Q35B_ERR_ARGUMENT, "Invalid rank layout for the gathering NVFP4 prefill projection.");
  }
  if (world == 1) return Q35B_OK;
  const cudaError_t le = launch_pdl(peer_gather_wait_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream),
                                    flag_words(buffers[rank]), world, rank, epoch, status_dev, kGatherWaitLimit);
  count_launch();
  Q35B_CUDA_TRY(le, "peer_gather_wait_kernel launch");
  return Q35B_OK;
}

int q35b_peer_push(q35b_peer_buffer * const * buffers, int world, int rank, const q35b_peer_region * regions, int n_regions,
                   unsigned int epoch, q35b_stream stream) {
  if (buffers == nullptr || world < 1 || world > kMaxRanks || rank < 0 || rank >= world || buffers[rank] == nullptr ||
      regions == nullptr || n_regions < 1 || n_regions > 4) {
    return fail(Q35B_ERR_ARGUMENT, "Invalid rank layout or region list for the peer push.");
  }
  PushArgs a = {};
  unsigned long long pieces = 0;
  for (int i = 0; i < n_regions; ++i) {
    const q35b_peer_region & r = regions[i];
    if (r.rows < 0 || (r.offset % 16) != 0 || (r.row_bytes % 16) != 0 || (r.ld_bytes % 16) != 0 || r.ld_bytes < r.row_bytes) {
      return fail(Q35B_ERR_ARGUMENT, "Peer push regions need 16-byte aligned offsets, row sizes and row strides.");
    }
    const size_t end = r.rows > 0 ? r.offset + static_cast<size_t>(r.rows - 1) * r.ld_bytes + r.row_bytes : r.offset;
    for (int q = 0; q < world; ++q) {
      if (buffers[q] == nullptr || buffers[q]->base == nullptr || buffers[q]->data_bytes < end) {
        return fail(Q35B_ERR_ARGUMENT, "A peer buffer of the push is missing or too small for a region.");
      }
    }
    a.region[i].offset = r.offset;
    a.region[i].ld = r.ld_bytes;
    a.region[i].row_pieces = static_cast<unsigned int>(r.row_bytes / 16);
    a.region[i].rows = static_cast<unsigned int>(r.rows);
    pieces += static_cast<unsigned long long>(r.rows) * (r.row_bytes / 16);
  }
  a.n_regions = n_regions;
  a.local = buffers[rank]->base;
  for (int q = 0; q < world; ++q) {
    if (q == rank) continue;
    a.peer[a.n_peers] = buffers[q]->base;
    a.peer_flag[a.n_peers] = flag_words(buffers[q]) + rank;
    ++a.n_peers;
  }
  a.done_counter = flag_words(buffers[rank]) + kMaxRanks;
  a.send_seq = flag_words(buffers[rank]) + kSendSeqWord;
  a.epoch = epoch;
  if (world == 1) return Q35B_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // enough threads to keep every NVLink busy, few enough that the closing count stays cheap
  const unsigned long long want = (pieces + 256ull * 4 - 1) / (256ull * 4);
  const int blocks = static_cast<int>(std::max<unsigned long long>(1, std::min<unsigned long long>(want, 2ull * sm_count())));
  const cudaError_t le = launch_pdl(peer_push_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, s, a);
  count_launch();
  Q35B_CUDA_TRY(le, "peer_push_kernel launch");
  return Q35B_OK;
}
