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
constexpr size_t kFlagBytes = 256;  // [kMaxRanks] epoch slots, then the owner's done counter
constexpr uint32_t kGatherWaitLimit = 1u << 22;
constexpr unsigned kStatusGatherWait = 31;

inline unsigned int * flag_words(const q35b_peer_buffer * b) { return reinterpret_cast<unsigned int *>(b->base + b->flags_offset); }

// One thread per rank: wait until that rank's slot carries this epoch (or a later one).
__global__ void peer_gather_wait_kernel(const unsigned int * flags, int world, int rank, unsigned int epoch,
                                        unsigned int * status) {
  const int r = threadIdx.x;
  if (r >= world || r == rank) return;
  const volatile unsigned int * slot = flags + r;
  for (uint32_t i = 0; i < kGatherWaitLimit; ++i) {
    if (static_cast<int>(*slot - epoch) >= 0) {
      __threadfence_system();  // the peer's matrix stores were fenced before its flag store
      return;
    }
    __nanosleep(64);
  }
  atomicExch(status, kStatusGatherWait);
}

// A rank whose shard is empty (more ranks than 128-row blocks) computes nothing but still has to tell the others
// that its part of the epoch is complete.
__global__ void peer_signal_kernel(GemmEpilogue ep) {
  if (threadIdx.x < ep.n_peers) *reinterpret_cast<volatile unsigned int *>(ep.peer_flag[threadIdx.x]) = ep.epoch;
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
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (w->rows == 0) {
    GemmEpilogue ep;
    ep.n_peers = gather.n_peers;
    for (int i = 0; i < gather.n_peers; ++i) ep.peer_flag[i] = gather.peer_flag[i];
    ep.epoch = epoch;
    peer_signal_kernel<<<1, 32, 0, s>>>(ep);
    count_launch();
    Q35B_CUDA_TRY(cudaGetLastError(), "peer_signal_kernel launch");
    return Q35B_OK;
  }
  Q35B_CUDA_TRY(cudaMemsetAsync(gather.done_counter, 0, sizeof(unsigned int), s), "cudaMemsetAsync(gather counter)");
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
  peer_gather_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(flag_words(buffers[rank]), world, rank, epoch,
                                                                         status_dev);
  count_launch();
  Q35B_CUDA_TRY(cudaGetLastError(), "peer_gather_wait_kernel launch");
  return Q35B_OK;
}
