/*
 * q35b — B200 (sm_100a) NVFP4 projection engine: C ABI.
 *
 * Drop-in boundary for the NVFP4 linear projections of the qwen35x runtime
 * (reference: Danmoreng/qwen35x; citations are paths inside that project).
 * Every function returns a q35b_status; on a nonzero status
 * q35b_last_error() holds a human-readable message for the calling thread,
 * mirroring the reference's `bool f(..., std::string & error_message)`
 * convention (include/qwen35x/runtime/cuda_bench.h:7-283).
 *
 * Conventions
 *   - N = output rows ("rows"), K = input columns ("cols"), M = tokens.
 *   - Checkpoint ("ModelOpt") layout of a weight, as validated by the
 *     reference in src/weights/modelopt_nvfp4.cpp:105-136:
 *       codes   uint8 [N, K/2]   E2M1, element 2j in the low nibble
 *       scales  uint8 [N, K/16]  E4M3, one per 16 K-elements
 *       weight_scale_2 fp32, input_scale fp32
 *   - All device pointers belong to the caller except the repacked weight,
 *     which the engine owns.  No call below allocates or synchronises unless
 *     it says so; every launch goes to the given stream.
 *   - A weight belongs to the device that was current when it was created;
 *     calls that take it must be made with that device current
 *     (Q35B_ERR_ARGUMENT otherwise).
 *   - Threads: a weight is immutable after q35b_weight_create* (its tensor
 *     maps are encoded there), so any number of host threads may project
 *     through the same weight at once, each on its own stream; the one piece
 *     of state built later (the single-projection work list of
 *     Q35B_GEMV_STREAM, per token count) is created under a lock.  A
 *     q35b_gemv_batch, a q35b_peer_buffer and the built-in scratch of
 *     q35b_project_prefill_bf16_static serve one call at a time.
 *   - There is no CPU fallback: without a CUDA device every compute entry
 *     point fails with Q35B_ERR_CUDA.
 */
#ifndef Q35B_NVFP4_H
#define Q35B_NVFP4_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define Q35B_API
#else
#define Q35B_API __attribute__((visibility("default")))
#endif

typedef enum q35b_status {
  Q35B_OK = 0,
  Q35B_ERR_ARGUMENT = 1,    /* null pointer, bad count */
  Q35B_ERR_SHAPE = 2,       /* dimensions the kernels do not support */
  Q35B_ERR_CUDA = 3,        /* a CUDA runtime/driver call failed (message has the call) */
  Q35B_ERR_DEVICE_WAIT = 4, /* a bounded device-side wait expired */
  Q35B_ERR_FORMAT = 5       /* tensor bytes violate the NVFP4 contract */
} q35b_status;

/* A weight repacked for the device.  Replaces the reference's
 * PackedNvfp4Weight (src/runtime/qwen35x_cuda_backend.cpp:194-210) and its
 * device twin Nvfp4Weight (src/kernels/cuda/weights.cuh:6-22). */
typedef struct q35b_weight q35b_weight;

/* CUDA stream handle (cudaStream_t) passed as an opaque pointer. */
typedef void * q35b_stream;

/* Kernel selector for the W4A16 decode projection; the names the CLI flag
 * --nvfp4-projection-kernel accepts map onto these (reference:
 * src/runtime/runtime.cpp:378-390, values 0..3 are the reference's). */
typedef enum q35b_gemv_kernel {
  Q35B_GEMV_AUTO = -1,  /* STREAM for a weight of 24 MiB or more that it can take (unless that would allocate on a
                         * capturing stream), else SIMT */
  Q35B_GEMV_SIMT = 10,  /* 128-bit loads, in-register dequant, fp32 FMA, warp-shuffle reduction */
  Q35B_GEMV_STREAM = 11 /* persistent, TMA-fed shared-memory ring; first use per (weight, m) allocates its work list */
} q35b_gemv_kernel;

/* ---- library ---------------------------------------------------------- */

Q35B_API const char * q35b_last_error(void);
Q35B_API const char * q35b_version(void);
/* Number of kernels this library has launched in the calling process. */
Q35B_API unsigned long long q35b_launch_count(void);

/* ---- weights ---------------------------------------------------------- */

/* Repack one checkpoint tensor family from HOST memory onto the current
 * device.  Replaces load_modelopt_nvfp4_state's per-module repack
 * (src/runtime/qwen35x_cuda_backend.cpp:1582-1695: pad_nvfp4_weight_for_tensor_core :967,
 * swizzle_nvfp4_block_scale_for_tensor_core :990, pack_nvfp4_weight_for_sm120_mma :1029).
 * Keeps the rows q35b_shard_range(n, shard_index, shard_count) names: the tensor's 128-row blocks (the height of
 * a scale tile) are dealt out as evenly as possible, shard i taking blocks [B*i/count, B*(i+1)/count) of
 * B = ceil(n/128), so every shard starts on a multiple of 128 rows and shards differ by at most one block
 * (n = 2560 over 8 shards: 384, 256, 384, 256, ...).
 * Allocates device memory, encodes the weight's tensor maps and synchronises the legacy default stream. */
Q35B_API int q35b_weight_create(const uint8_t * codes_host, const uint8_t * scales_host, float weight_scale_2,
                                float input_scale, int n, int k, int shard_index, int shard_count,
                                q35b_weight ** out);

/* Same, from DEVICE buffers in checkpoint layout (the shard's rows are
 * copied; the source may be freed afterwards). */
Q35B_API int q35b_weight_create_from_device(const uint8_t * codes_dev, const uint8_t * scales_dev,
                                            float weight_scale_2, float input_scale, int n, int k, int shard_index,
                                            int shard_count, q35b_stream stream, q35b_weight ** out);

/* A gate_proj / up_proj pair as ONE weight whose rows alternate in groups of eight (8 gate rows, 8 up rows, ...),
 * so that a work-list projection over it can finish with y[j] = bf16(silu(gate_j . x) * (up_j . x)), j < n_half: the
 * fused epilogue of matvec_gate_up_silu_nvfp4 (src/kernels/cuda/decode_layers.cuh:339-365) and of the
 * silu_multiply_kernel bridges (src/runtime/cuda_bench.cu:215-222), silu(g) = g / (1 + exp(-g)).  Each half keeps its
 * own weight_scale_2.  n_half must be a multiple of 8.  Host tensors in checkpoint layout. */
Q35B_API int q35b_weight_create_gate_up(const uint8_t * gate_codes_host, const uint8_t * gate_scales_host,
                                        float gate_weight_scale_2, const uint8_t * up_codes_host,
                                        const uint8_t * up_scales_host, float up_weight_scale_2, int n_half, int k,
                                        q35b_weight ** out);
/* Row shard of such a pair, for the N-sharded prefill MLP: the interleaved matrix (2 * n_half rows) is cut like any
 * other weight (q35b_shard_range(2 * n_half, ...), 128-row blocks), so shard i yields the output columns
 * [row_begin / 2, row_begin / 2 + rows / 2) of silu(gate) * up, a multiple of 64 of them. */
Q35B_API int q35b_weight_create_gate_up_shard(const uint8_t * gate_codes_host, const uint8_t * gate_scales_host,
                                              float gate_weight_scale_2, const uint8_t * up_codes_host,
                                              const uint8_t * up_scales_host, float up_weight_scale_2, int n_half,
                                              int k, int shard_index, int shard_count, q35b_weight ** out);
/* 1 if the weight was built by q35b_weight_create_gate_up(_shard). */
Q35B_API int q35b_weight_is_gate_up(const q35b_weight * w);

/* NVFP4 -> BF16 dequantisation of the whole weight, w_bf16 [rows, K] device: bf16(e2m1 * (e4m3 * s2)), the
 * conversion the reference does on the CPU at load for its BF16 prefill path
 * (src/runtime/qwen35x_cuda_backend.cpp:742-755). */
Q35B_API int q35b_weight_dequant_bf16(const q35b_weight * w, void * w_bf16, q35b_stream stream);

Q35B_API void q35b_weight_destroy(q35b_weight * w);

/* Shard geometry: first global row and row count held by this weight. */
Q35B_API int q35b_weight_row_begin(const q35b_weight * w);
Q35B_API int q35b_weight_rows(const q35b_weight * w);
Q35B_API int q35b_weight_cols(const q35b_weight * w);
/* Bytes one projection call streams from this weight (codes + scales). */
Q35B_API size_t q35b_weight_stream_bytes(const q35b_weight * w);
/* Row range of shard `shard_index` of an n-row tensor. */
Q35B_API int q35b_shard_range(int n, int shard_index, int shard_count, int * row_begin, int * row_count);

/* ---- decode: W4A16 projection, M = 1..8 ------------------------------- */

/* y[m, r] = bf16( sum_c e2m1(w[r,c]) * e4m3(s[r,c/16]) * s2 * x[m, c] ), fp32
 * accumulation, BF16 activations and output, input_scale not applied
 * (the live decode of the reference passes 1.0,
 * src/runtime/qwen35x_cuda_backend.cpp:2320).  Replaces matvec_nvfp4_bf16 /
 * nvfp4_row_dot (src/kernels/cuda/decode_layers.cuh:200-284) and the scalar
 * projection kernels (src/runtime/cuda_bench.cu:283-429).
 * x: [m, K] bf16 device, y: [m, rows] bf16 device (rows = this shard's). */
Q35B_API int q35b_gemv_w4a16_bf16(const q35b_weight * w, const void * x_bf16, int m, void * y_bf16, int kernel,
                                  q35b_stream stream);

/* The reference benchmark's contract (src/runtime/cuda_bench.cu:2042-2188):
 * fp32 input of one token, activations multiplied by input_scale, fp32 output. */
Q35B_API int q35b_gemv_w4a16_f32(const q35b_weight * w, const float * x_f32, float input_scale, float * y_f32,
                                 int kernel, q35b_stream stream);

/* One persistent launch over several projections (the work list of a decode step, or of one phase of it).
 * Replaces the per-phase matvec loops of the reference's persistent decode kernel
 * (src/kernels/cuda/decode_kernel.cuh:58-84).  Every weight needs cols % 256 == 0 and unsigned block scales.
 * Items are independent unless one names an earlier item in `after`: then its x_bf16 may be that item's y_bf16 (the
 * down projection reading the gate/up output), and the kernel holds its activations back until every tile of the
 * earlier item has been stored -- where the reference's decode kernel puts a grid-wide barrier between the two
 * phases (decode_kernel.cuh:76-84), with a bounded wait instead of an unbounded one. */
typedef struct q35b_gemv_item {
  const q35b_weight * weight;
  const void * x_bf16;        /* [m, K] device */
  void * y_bf16;              /* [m, out_rows] device; out_rows = rows, or rows/2 for a gate/up weight */
  const void * residual_bf16; /* NULL, or [m, rows] device: y = bf16(projection + residual), the fused epilogue of
                                 matvec_down_residual_nvfp4 / matvec_o_residual_nvfp4
                                 (src/kernels/cuda/decode_layers.cuh:404-428, 465-489) */
  int after;                  /* 0: independent; k > 0: runs after item k - 1 of the same list (k - 1 < own index) */
} q35b_gemv_item;

/* sizeof(q35b_gemv_item) as this library was built: lets a foreign-function binding check its own struct layout. */
Q35B_API size_t q35b_gemv_item_bytes(void);

typedef struct q35b_gemv_batch q35b_gemv_batch;
/* Builds the tile schedule and uploads the descriptors (allocates, synchronises). */
Q35B_API int q35b_gemv_batch_create(const q35b_gemv_item * items, int count, int m, q35b_gemv_batch ** out);
/* The same work list on the tensor cores (no counterpart in the reference, whose decode dequantises in registers,
 * src/kernels/cuda/decode_layers.cuh:200-261): the weight streams through tcgen05.mma as the 128-row operand and
 * every token's BF16 activations enter as `digits` rows of NVFP4, a digit expansion computed on the device before
 * each run: digit j quantises (16-element blocks, E4M3 block scale, one fp32 scale per token) what digits 0..j-1
 * left over, so their sum reproduces the activation to within 6^-digits of its block's largest element (5 digits:
 * 1.3e-4 at worst; BF16's own rounding step is 3.9e-3).  Outputs stay within the relative L2 bound of 1e-3 against
 * the exact W4A16 result.  Measured on B200 it is NOT the faster path: 73 us per 0.8B-class step at one token and
 * 96 us at eight, against 44.5 and 57 us for q35b_gemv_batch_create (with operand tiles this narrow the tensor pipe's
 * copy-to-MMA turnaround per 256 columns of K sets the pace); it is kept as the variant whose cost does not grow
 * with the conversion work and as the decode-side user of the weight-streaming kernel.  Items must be independent
 * (after = 0); non-finite activations count as zero.  digits: 1..8 with m * digits <= 128; 5 is the intended
 * setting.  q35b_gemv_batch_run launches two kernels (the expansion, then the projection, whose weight stream
 * starts at once). */
Q35B_API int q35b_gemv_batch_create_tensor(const q35b_gemv_item * items, int count, int m, int digits,
                                           q35b_gemv_batch ** out);
/* One kernel launch on `stream`; no allocation, no synchronisation.  The launch uses programmatic stream
 * serialisation: the kernel may begin streaming WEIGHTS while the previous kernel of the stream is still finishing
 * (activations, residuals and outputs are touched only after that kernel is complete).  Weights are therefore
 * treated as constant from q35b_weight_create* on; a host that rewrites weight memory must synchronise the stream
 * before the next run. */
Q35B_API int q35b_gemv_batch_run(const q35b_gemv_batch * batch, q35b_stream stream);
Q35B_API void q35b_gemv_batch_destroy(q35b_gemv_batch * batch);
/* Copies the batch's device status word to the host (synchronises): 0, or the code of a bounded device-side wait
 * that expired during a run. */
Q35B_API int q35b_gemv_batch_status(const q35b_gemv_batch * batch, unsigned int * status_out);
/* Test hook for the bounded device-side waits of a work list built by q35b_gemv_batch_create: every wait of the
 * following runs (ring barriers, activation hand-over, dependency poll) gives up after `wait_limit_polls` polls
 * instead of 2^22, and a dependent item demands `extra_completions` more completions of the item it runs after than
 * that item can deliver.  With a small limit and one extra completion the dependency poll runs out within
 * microseconds, 15 lands in the status word, the remaining roles run out on their own waits and the kernel returns:
 * what an item whose producer never finishes looks like, without a kernel that hangs.  (0 extra completions and
 * 1 << 22 polls restore normal operation.)  Also clears the list's status word and completion counts. */
Q35B_API int q35b_debug_gemv_batch_wait(q35b_gemv_batch * batch, unsigned int wait_limit_polls,
                                        unsigned int extra_completions);
/* The shared-memory plan a work list of `m` tokens over weights of at most `max_k` columns would get (host
 * arithmetic only, no device needed): ctas_per_sm is 2 for the shape with eight consumer warps and half an SM's
 * shared memory, 1 for the shape with sixteen consumer warps and all of it; ring_stages are 18 KB each;
 * activation_buffers is 1 or 2; smem_bytes is the dynamic shared memory of one CTA.  Q35B_ERR_SHAPE when the
 * activations fit neither shape. */
Q35B_API int q35b_debug_gemv_plan(int m, int max_k, int * ctas_per_sm, int * ring_stages, int * activation_buffers,
                                  int * smem_bytes);
/* Weight bytes (codes + scales) one run streams. */
Q35B_API size_t q35b_gemv_batch_stream_bytes(const q35b_gemv_batch * batch);

/* ---- prefill: activation quantisation + W4A4 GEMM --------------------- */

/* Scratch sizes for an [m, k] activation: packed codes m*k/2 bytes; tiled
 * scales roundup(m,128) * roundup(k/16,4) bytes (the reference's rule,
 * src/runtime/cuda_bench.cu:2616-2619). */
Q35B_API size_t q35b_act_codes_bytes(int m, int k);
Q35B_API size_t q35b_act_scales_bytes(int m, int k);
/* Bytes of the quantiser's workspace; must be zero before its first use and
 * is left zero by every call. */
Q35B_API size_t q35b_quant_workspace_bytes(void);

/* BF16 [m, k] -> NVFP4: E2M1 codes [m, k/2] (element 2j in the low nibble),
 * E4M3 block scales in the 128x4 tiled layout, and the fp32 per-tensor scale
 * g written to *input_scale_dev.  g = amax/(6*448) when global_scale <= 0,
 * else global_scale.  Replaces nvfp4_quantize_bf16_matrix_for_cublaslt_kernel
 * (src/runtime/cuda_bench.cu:178-213) and the two cudaMemset calls before it
 * (:2621-2624). */
Q35B_API int q35b_quantize_nvfp4_bf16(const void * x_bf16, int m, int k, float global_scale, uint8_t * codes,
                                      uint8_t * scales_tiled, float * input_scale_dev, void * workspace,
                                      q35b_stream stream);

/* Same from fp32 activations [m, k], the input type of the reference's prefill benchmark
 * (nvfp4_quantize_matrix_for_cublaslt_kernel, src/runtime/cuda_bench.cu:141-176, fed by
 * src/runtime/runtime.cpp:498-501).  x_f32 16-byte aligned. */
Q35B_API int q35b_quantize_nvfp4_f32(const float * x_f32, int m, int k, float global_scale, uint8_t * codes,
                                     uint8_t * scales_tiled, float * input_scale_dev, void * workspace,
                                     q35b_stream stream);

/* The reference's own activation recipe (no per-tensor scale, divisor =
 * unrounded block scale, src/runtime/cuda_bench.cu:178-213), kept so the
 * quantiser can be checked byte-for-byte against the reference's kernel.
 * swap_nibbles != 0 writes element 2j in the HIGH nibble as that kernel does. */
Q35B_API int q35b_quantize_nvfp4_bf16_reference_recipe(const void * x_bf16, int m, int k, int swap_nibbles,
                                                       uint8_t * codes, uint8_t * scales_tiled,
                                                       q35b_stream stream);

/* c[m, rows] (bf16, row stride ldc elements) = (Aq . Wq^T) * g * s2 with
 * tcgen05 block-scaled FP4 MMA.  Replaces
 * run_nvfp4_cublaslt_prefill_projection_device (src/runtime/cuda_bench.cu:1056-1167)
 * and the fp32->bf16 pass after it (src/kernels/cuda/prefill.cu:639).
 * Requires k % 64 == 0.  status_dev: 4 bytes of device memory, zero on entry,
 * nonzero afterwards if a bounded device-side wait expired.  With status_dev
 * NULL the call uses a word inside the library (one per device, nothing
 * allocated, nothing launched in front of the kernel): a code stays in it until
 * q35b_gemm_default_status reads it, which also clears it.  All calls of a
 * device without an own word share it: pass one where the call that failed
 * has to be told apart. */
Q35B_API int q35b_gemm_w4a4_bf16(const q35b_weight * w, const uint8_t * a_codes, const uint8_t * a_scales_tiled,
                                 const float * input_scale_dev, int m, void * c_bf16, int ldc,
                                 unsigned int * status_dev, q35b_stream stream);

/* Copies the library's status word of the current device to the host (synchronises the device) and clears it. */
Q35B_API int q35b_gemm_default_status(unsigned int * status_out);

/* Same GEMM with the residual add fused into the epilogue: c = bf16(projection + residual), residual [m, rows] BF16
 * with row stride ldr.  Replaces pf_add_residual_bf16 after the down / o projections
 * (src/kernels/cuda/prefill.cu:679, pf_mlp_chunked :647-680).
 * On a gate/up weight (q35b_weight_create_gate_up) q35b_gemm_w4a4_bf16 itself ends with silu(gate) * up and writes
 * c [m, rows/2], replacing pf_silu_mul_bf16 (src/kernels/cuda/prefill.cu:674-678). */
Q35B_API int q35b_gemm_w4a4_bf16_residual(const q35b_weight * w, const uint8_t * a_codes, const uint8_t * a_scales_tiled,
                                          const float * input_scale_dev, int m, const void * residual_bf16, int ldr,
                                          void * c_bf16, int ldc, unsigned int * status_dev, q35b_stream stream);

/* Gate/up GEMM whose epilogue writes silu(gate) * up as an NVFP4 activation (codes [m, rows/4] bytes, tiled block
 * scales sized by q35b_act_scales_bytes(m, rows/2)), ready to be the A operand of the down projection's
 * q35b_gemm_w4a4_bf16(_residual) with out_scale_dev as its input_scale_dev.  Replaces pf_silu_mul_bf16 plus the
 * quantise pass between the reference's gate/up and down GEMMs (src/kernels/cuda/prefill.cu:674-678,
 * src/runtime/cuda_bench.cu:2621-2660).  out_scale_dev is that activation's per-tensor scale and must be known
 * in advance (the checkpoint's input_scale of the down projection, or amax / 2688 from a calibration run); values
 * beyond 2688 * scale saturate.  The bits equal q35b_quantize_nvfp4_bf16 applied, with the same scale, to the BF16
 * output of q35b_gemm_w4a4_bf16 on the same weight.  w must be a gate/up weight with rows/2 a multiple of 64.
 * out_codes / out_scales_tiled always describe the WHOLE activation [m, n_half]: a shard
 * (q35b_weight_create_gate_up_shard) writes only its own columns of it, code bytes [row_begin / 4, ...) of every
 * row and the matching scale tiles, so that the shards of all ranks together fill one activation. */
Q35B_API int q35b_gemm_w4a4_gate_up_nvfp4(const q35b_weight * w, const uint8_t * a_codes,
                                          const uint8_t * a_scales_tiled, const float * input_scale_dev, int m,
                                          uint8_t * out_codes, uint8_t * out_scales_tiled,
                                          const float * out_scale_dev, unsigned int * status_dev, q35b_stream stream);

/* ---- N-sharded prefill projection with the gather fused into the GEMM's stores ----
 * Replaces the exchange step of the row-sharded projection (one ncclAllGather of the BF16 slabs after the GEMM):
 * every rank holds the full output matrix [m, N] in a peer buffer; the GEMM on a shard (q35b_weight_create with
 * shard_index / shard_count) stores its columns into the local matrix and, with plain peer-memory stores over
 * NVLink, into every other rank's, and finally writes `epoch` into its flag slot on every rank.
 * q35b_peer_gather_wait (same stream, after the GEMM) returns once the local slots of all other ranks carry that
 * epoch, i.e. the whole matrix is in place; its wait is bounded and records 31 in *status_dev on expiry.
 * Use a new, larger epoch per gathered matrix, or pass epoch 0 everywhere: then sender and receiver count their
 * sends and waits in device memory (send k of a rank is matched by wait k of every other rank), nothing in the
 * kernel arguments changes from call to call, and a captured sequence of gathers can be replayed as a CUDA graph.
 * Every rank must then issue the same sequence of sends and waits on a buffer.  One process per GPU: create the local buffer, pass its handle
 * (q35b_peer_buffer_handle_bytes() bytes) to the other ranks by any host channel, open theirs.  buffers[world] lists
 * the mappings by rank, buffers[rank] being the local one.  In one process (tests, several GPUs under one host
 * thread) created buffers can be listed directly.
 * Any ldc >= the full width works; when ldc, the shard's column count and the matrices' bases are multiples of 16
 * elements (true for every 128-row shard cut of a contiguous [m, N] matrix) the remote stores are whole 128-byte
 * lines, otherwise each lane repeats its own 32-byte (or scalar) stores. */
typedef struct q35b_peer_buffer q35b_peer_buffer;
Q35B_API int q35b_peer_buffer_create(size_t data_bytes, q35b_peer_buffer ** out);
Q35B_API size_t q35b_peer_buffer_handle_bytes(void);
Q35B_API int q35b_peer_buffer_export(const q35b_peer_buffer * buffer, void * handle_out);
Q35B_API int q35b_peer_buffer_open(const void * handle, size_t data_bytes, q35b_peer_buffer ** out);
Q35B_API void * q35b_peer_buffer_data(const q35b_peer_buffer * buffer);
Q35B_API void q35b_peer_buffer_destroy(q35b_peer_buffer * buffer);
Q35B_API int q35b_gemm_w4a4_bf16_allgather(const q35b_weight * w, const uint8_t * a_codes, const uint8_t * a_scales_tiled,
                                           const float * input_scale_dev, int m, q35b_peer_buffer * const * buffers,
                                           int world, int rank, int ldc, unsigned int epoch, unsigned int * status_dev,
                                           q35b_stream stream);
Q35B_API int q35b_peer_gather_wait(q35b_peer_buffer * const * buffers, int world, int rank, unsigned int epoch,
                                   unsigned int * status_dev, q35b_stream stream);

/* Pushes regions of this rank's peer buffer into the same place of every other rank's buffer (plain peer-memory
 * stores over NVLink, 16 bytes per thread, whole 128-byte lines per warp) and then writes `epoch` into this rank's
 * flag slot on every rank: q35b_peer_gather_wait(.., epoch, ..) on the receiving side returns when all ranks'
 * pushes of that epoch have arrived.  It is the exchange step for outputs whose producer writes pieces too small to
 * forward itself: the NVFP4 codes and scale tiles of q35b_gemm_w4a4_gate_up_nvfp4 on a shard (an N-sharded MLP
 * block gathers 0.5625 bytes per intermediate element instead of 2), or a narrow BF16 shard.
 * A region is `rows` rows of `row_bytes` bytes, `ld_bytes` apart, starting `offset` bytes into the buffer's data;
 * all three multiples of 16; at most 4 regions per call.  Replaces the ncclAllGather of the row-sharded projection
 * where the data is not one contiguous slab per rank.  (Measured on 2 x B200: 10.4 MB per direction in ~27 us,
 * the same with bulk copies through shared memory instead of stores: the links, not the SMs, set the rate when both
 * directions are busy.) */
typedef struct q35b_peer_region {
  size_t offset;
  size_t row_bytes;
  size_t ld_bytes;
  int rows;
} q35b_peer_region;
Q35B_API int q35b_peer_push(q35b_peer_buffer * const * buffers, int world, int rank, const q35b_peer_region * regions,
                            int n_regions, unsigned int epoch, q35b_stream stream);

/* Prefill projection for callers that cannot allocate device memory (no counterpart in the reference, whose
 * bridges all take caller-allocated scratch, include/qwen35x/runtime/cuda_bench.h:70-83).
 *
 * c[m, rows] (bf16, row stride ldc) = NVFP4-quantise(x[m, K]) projected through w: the same two kernels as
 * q35b_quantize_nvfp4_bf16 followed by q35b_gemm_w4a4_bf16, but the quantised activation, its scales, the
 * per-tensor scale word, the quantiser workspace and the status word live in a scratch area built into the
 * library (a file-scope device array, 24 MiB, held by every GPU that loads the library until the process exits).
 * It is meant for hosts that own all device memory themselves (a pre-sized arena, a fixed memory budget) or that
 * must not hit the device-wide synchronisation an allocation implies.  The call itself makes no cudaMalloc,
 * cudaFree or other allocating call.
 *
 *  - m * K / 2 (rounded up to 256) + roundup(m,128) * roundup(K/16,4) must fit in
 *    q35b_static_prefill_capacity_bytes(); larger activations are rejected with Q35B_ERR_SHAPE.
 *  - The first call on each device resolves the scratch's device address (and sets kernel attributes): make that
 *    first call outside any stream capture.
 *  - All calls on a device share the one scratch area: two calls that may overlap on the GPU (different streams
 *    without an ordering between them, or different threads) race on it.  Serialise them.
 *  - The area keeps the previous call's bytes; the words that must start at zero are cleared by every call.
 *  - A bounded device-side wait that expired leaves its code in the scratch's status word until the next call
 *    clears it: q35b_static_prefill_status copies that word of the current device to the host (it synchronises
 *    the device, so it also waits for the call it reports on). */
Q35B_API size_t q35b_static_prefill_capacity_bytes(void);
Q35B_API int q35b_static_prefill_status(unsigned int * status_out);
Q35B_API int q35b_project_prefill_bf16_static(const q35b_weight * w, const void * x_bf16, int m, float global_scale,
                                              void * c_bf16, int ldc, q35b_stream stream);

/* ---- synthetic checkpoints ---------------------------------------------- */

/* fp32 [n, k] -> NVFP4 in checkpoint layout (codes [n, k/2], row-major scales
 * [n, k/16]) with weight_scale_2 = amax/(6*448) written to *s2_dev, the
 * recipe of q35b_quantize_nvfp4_bf16.  The reference has no weight quantiser
 * (it consumes pre-quantised ModelOpt checkpoints, docs/development_plan.md:389);
 * this exists to build synthetic tensors for benchmarks and tests. */
Q35B_API int q35b_quantize_weight_f32(const float * w_f32, int n, int k, uint8_t * codes, uint8_t * scales,
                                      float * s2_dev, void * workspace, q35b_stream stream);

/* ---- host twins of the device codecs (no GPU needed) ------------------- */

/* The encoders/decoders the kernels use, compiled for the host, so their
 * equivalence with the reference's scan encoders
 * (src/runtime/cuda_bench.cu:902-940) can be checked on any machine. */
Q35B_API uint8_t q35b_debug_encode_ue4m3(float v);
Q35B_API uint8_t q35b_debug_encode_e2m1(float v);
Q35B_API float q35b_debug_decode_e4m3(uint8_t b);
Q35B_API float q35b_debug_decode_e2m1(uint8_t c);
Q35B_API long long q35b_debug_tiled_scale_offset(int row, int col, int padded_cols);

#ifdef __cplusplus
}
#endif
#endif /* Q35B_NVFP4_H */
