/*
 * b200q — C ABI of the B200 (sm_100a) quantized-linear hot path.
 *
 * This is the drop-in boundary: a maintainer of Torch-TensorRT binds these entry points
 * (ctypes, a torch.library C++ shim, or a TensorRT plugin `enqueue`) in place of the
 * TensorRT layers / third-party eager kernels the reference uses for the same step.
 *
 * Conventions for every compute entry point
 *   - all buffers are caller-owned DEVICE pointers, row-major, contiguous;
 *   - nothing is allocated or freed, nothing synchronises: work is enqueued on `stream`
 *     (a `cudaStream_t` passed as `void*`; NULL = the legacy default stream);
 *   - the return value is B200Q_OK (0) or a negative B200Q_ERR_* code; nothing throws;
 *   - `dtype` is one of B200Q_F32 / B200Q_F16 / B200Q_BF16 and names the element type of
 *     the floating-point tensor `x` / `out`.
 *
 * Reference citations are paths inside the pytorch/TensorRT tree.
 */
#ifndef B200Q_H_
#define B200Q_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200Q_OK 0
#define B200Q_ERR_INVALID (-1)   /* bad shape / null pointer / unsupported dtype      */
#define B200Q_ERR_ALIGN (-2)     /* pointer or leading dimension not aligned as needed */
#define B200Q_ERR_ARCH (-3)      /* device is not compute capability 10.x              */
#define B200Q_ERR_CUDA (-4)      /* a CUDA runtime / driver call failed                */
#define B200Q_ERR_WORKSPACE (-5) /* workspace missing or too small                     */
#define B200Q_ERR_TIMEOUT (-6)   /* a bounded device-side wait gave up                 */
#define B200Q_ERR_TOO_LARGE (-7) /* size beyond what a fixed built-in scratch can serve    */

#define B200Q_F32 0
#define B200Q_F16 1
#define B200Q_BF16 2

typedef void* b200q_stream_t;

/* Library identification. */
int b200q_version(void);
const char* b200q_status_string(int status);

/* ------------------------------------------------------------------ abs-max reductions
 * The `amax` operand of both quantize ops is an input the caller supplies
 * (tests/py/dynamo/models/test_models_export.py:789 passes it explicitly); these produce
 * it on the device for dynamic quantization.
 *
 * b200q_amax: max(|x|) over n elements -> amax_out[0].  Needs a workspace of
 * b200q_amax_workspace_bytes() bytes (a ticket counter and the running maximum of the CTAs);
 * the workspace must be zero the first time it is used and is left zero again on return,
 * so one memset at allocation is enough.  Calls sharing a workspace must not overlap.
 * b200q_row_amax: max(|x|) per row -> amax_out[rows].
 */
size_t b200q_amax_workspace_bytes(void);
int b200q_amax(const void* x, int dtype, int64_t n, float* amax_out, void* workspace,
               size_t workspace_bytes, b200q_stream_t stream);
int b200q_row_amax(const void* x, int dtype, int64_t rows, int64_t cols, float* amax_out,
                   b200q_stream_t stream);

/* b200q_amax_static: the same tensor abs-max for callers that have no way to provide a
 * workspace.  No counterpart in the reference; it exists because some hosts of this library
 * must not allocate device memory at the point where they call it: a TensorRT plugin's
 * enqueue() only gets the workspace TensorRT sized at build time, a stream being captured
 * into a CUDA graph rejects cudaMalloc, and a serving process may have handed all device
 * memory to its own pool.  The ticket counter and the running maximum of the CTAs live in a
 * 4352-byte array compiled into the library (every GPU that loads the library holds it
 * until the process exits), so nothing is allocated or freed here, by this library or by
 * any library it calls.
 *   - n may be at most b200q_amax_static_max_elements() (2^28: one partial per 2^18-element
 *     chunk, 1024 partials); larger n returns B200Q_ERR_TOO_LARGE and launches nothing.
 *   - The first call on each device looks up the array's device address (a host-side
 *     runtime query); make that first call outside any stream capture.
 *   - All calls on a device share the one array: calls that can overlap on the GPU (two
 *     streams, two host threads) race with each other and give wrong results; serialise
 *     them or use b200q_amax with separate workspaces.
 *   - The ticket counter and the running maximum in the array are re-armed by the last CTA of every launch.  A launch that
 *     dies part-way (a fault elsewhere in the context) can leave it non-zero, and since the caller
 *     cannot reach the array to clear it, later calls on that device then return wrong maxima:
 *     after a failed launch treat the context as lost, as for any other sticky CUDA error.
 * Results are identical to b200q_amax. */
int64_t b200q_amax_static_max_elements(void);
int b200q_amax_static(const void* x, int dtype, int64_t n, float* amax_out, b200q_stream_t stream);

/* ------------------------------------------------------------------ FP8 E4M3
 * Replaces the Q half of the IQuantizeLayer/IDequantizeLayer pair built by
 * py/torch_tensorrt/dynamo/conversion/impl/quantize.py:73-134 (scale = amax / 448,
 * round to nearest even, saturate), producing real codes for the FP8 GEMM.
 *
 * amax_numel selects the scaling granularity:
 *   1      per-tensor: amax[0]                       (what impl/quantize.py:96-100 accepts)
 *   rows   one amax per row: amax[r]                 (per-token / per-channel extension)
 *   0      dynamic per-row: the row abs-max is reduced inside the kernel, amax is ignored
 * scales_out receives max(amax_numel, 1) fp32 scales (rows of them when amax_numel == 0);
 * it may be NULL when amax_numel == 1.  cols must be a multiple of 16.
 */
int b200q_fp8_quantize(const void* x, int dtype, int64_t rows, int64_t cols, const float* amax,
                       int64_t amax_numel, uint8_t* codes_out, float* scales_out,
                       b200q_stream_t stream);

/* Eager semantics of `tensorrt::quantize_op(input, amax, 8, 4, unsigned, narrow_range)`:
 * quantize then dequantize back to the input dtype (impl/quantize.py:126-138).  Same
 * amax_numel convention as above.  cols must be a multiple of 8. */
int b200q_fp8_fake_quantize(const void* x, int dtype, int64_t rows, int64_t cols,
                            const float* amax, int64_t amax_numel, void* out,
                            b200q_stream_t stream);

/* codes * scale -> out (dtype).  scales_numel is 1 or rows. */
int b200q_fp8_dequantize(const uint8_t* codes, const float* scales, int64_t scales_numel,
                         int64_t rows, int64_t cols, void* out, int dtype, b200q_stream_t stream);

/* ------------------------------------------------------------------ NVFP4 (E2M1 codes, block 16, E4M3 block scales)
 * Replaces IDynamicQuantizeLayer (impl/dynamic_block_quantize.py:149-156) for activations
 * and the offline weight quantization (impl/dynamic_block_quantize.py:248-270) for weights.
 *   global scale = (amax[0] / 6) / 448, zero -> 1     (impl/dynamic_block_quantize.py:299-308)
 *   codes_out    [rows, cols/2] bytes, element 2i in the low nibble
 *   scales_out   b200q_nvfp4_scale_bytes(rows, cols) bytes in the 128x4 swizzled layout
 *                (rows padded to 128, scale columns to 4; tile (rt, ct) at
 *                (rt * n_col_tiles + ct) * 512; row r, column c inside a tile at
 *                (r % 32) * 16 + (r / 32) * 4 + c); padding is written as zero
 *   global_scale_out  one fp32 (may be NULL)
 * cols must be a multiple of 16.
 */
size_t b200q_nvfp4_scale_bytes(int64_t rows, int64_t cols);
int b200q_nvfp4_quantize(const void* x, int dtype, int64_t rows, int64_t cols, const float* amax,
                         uint8_t* codes_out, uint8_t* scales_out, float* global_scale_out,
                         b200q_stream_t stream);

/* Eager semantics of `tensorrt::dynamic_block_quantize_op(input, 16, amax, 4, 2, 8, 4)`:
 * quantize then double-dequantize, x_hat = e2m1 * (e4m3 * global), back to the input dtype
 * (impl/dynamic_block_quantize.py:201-221). */
int b200q_nvfp4_fake_quantize(const void* x, int dtype, int64_t rows, int64_t cols,
                              const float* amax, void* out, b200q_stream_t stream);

int b200q_nvfp4_dequantize(const uint8_t* codes, const uint8_t* scales_swizzled,
                           const float* global_scale, int64_t rows, int64_t cols, void* out,
                           int dtype, b200q_stream_t stream);

/* ------------------------------------------------------------------ per-call options
 * Last argument of the GEMM entry points and of the peer-memory reductions; NULL = all defaults.
 * Nothing here is process-wide: two callers (threads, stacks, graphs) never see each other's choices.
 *   tile_n          GEMM tile selection.  0 = chosen per problem (default); 128 or 256 = single-CTA
 *                   tiles of 128 x tile_n; 512 = CTA-pair kernels (256 x 256 tiles, cta_group::2; chosen
 *                   automatically when the problem has at least one such tile per SM pair);
 *                   1001 / 1002 / 1004 / 1008 = small-M kernel (weights on the tensor core's M side,
 *                   K split over a cluster of 1 / 2 / 4 / 8 CTAs, partial tiles summed through
 *                   distributed shared memory; chosen automatically for M <= 128, ignored for larger
 *                   M).  Results do not depend on it beyond fp32 summation order.  Any other value:
 *                   B200Q_ERR_INVALID.
 *   static_weights  promise about the B operand (weights, their scales, the bias) of THIS call:
 *                   non-zero = the work that wrote it has FINISHED on the device (weights quantized at
 *                   load time, followed by a synchronisation), so no kernel still in flight when the
 *                   GEMM starts can be writing it.  The small-M GEMM is launched programmatically
 *                   dependent on its predecessor and through a chain of such launches may start while
 *                   several earlier kernels still run; with the promise it requests its first weight
 *                   tiles right away and waits for its predecessors only before reading the
 *                   activations.  Without it (default) it waits before reading anything.
 *   peer_wait_ms    limit of every device-side wait for another rank (flag words of the peer-memory
 *                   reductions), in milliseconds; 0 = the default of 2000.  A wait that runs out sets
 *                   the device status word (b200q_device_status) and the reduction skips its work.
 */
typedef struct b200q_cfg {
  int32_t tile_n;
  int32_t static_weights;
  uint32_t peer_wait_ms;
  uint32_t reserved;       /* must be 0 */
} b200q_cfg;

/* ------------------------------------------------------------------ quantized GEMMs (tcgen05)
 * Replace the IMatrixMultiplyLayer (+ bias add) TensorRT fuses with its Q/DQ neighbours
 * (impl/linear.py:40-67, impl/matmul.py:62-64):   out[m, n] = sum_k a[m,k] * b[n,k]  (+ bias[n])
 * with a, b the dequantized operands.  out is bf16 [M, N]; bias is bf16 [N] or NULL.
 *
 * FP8: a_codes [M, K], b_codes [N, K] E4M3; a_scales has a_scales_numel (1 or M) fp32
 * entries, b_scales has b_scales_numel (1 or N).  K must be a multiple of 16.
 *
 * NVFP4: a_codes [M, K/2], b_codes [N, K/2]; block scales in the swizzled layout above;
 * a_global / b_global point at one fp32 each.  K must be a multiple of 32.
 */
int b200q_fp8_gemm(const uint8_t* a_codes, const float* a_scales, int64_t a_scales_numel,
                   const uint8_t* b_codes, const float* b_scales, int64_t b_scales_numel,
                   const void* bias, void* out, int64_t M, int64_t N, int64_t K,
                   b200q_stream_t stream, const b200q_cfg* cfg);

/* b200q_fp8_gemm with the gate/up activation fused into its epilogue (producer fusion):
 * b holds F gate rows followed by F up rows (N = 2 F, F a multiple of 128; scales and bias indexed the
 * same way), out is [M, F] bf16 = silu(g) * u with g, u the two linear outputs rounded to bf16 first,
 * i.e. the same bits as b200q_fp8_gemm followed by b200q_silu_mul, without the [M, 2 F] round trip
 * through memory.  Replaces linear + silu + mul of a gated MLP (the graph the reference lowers
 * tools/llm models to; aten_ops_converters.py linear / silu / mul converters).  cfg: tile_n must be 0. */
int b200q_fp8_gemm_silu_mul(const uint8_t* a_codes, const float* a_scales, int64_t a_scales_numel,
                            const uint8_t* b_codes, const float* b_scales, int64_t b_scales_numel,
                            const void* bias, void* out, int64_t M, int64_t N, int64_t K,
                            b200q_stream_t stream, const b200q_cfg* cfg);

/* The same with the activation's FP8 quantizer folded in as well, for a STATIC per-tensor amax (what the
 * input quantizer of the down projection holds after calibration): codes_out [M, F] uint8 =
 * e4m3(clamp(bf16(silu(g) * u) / scale)), scale = act_amax[0] / 448 (0 -> 1) also written to scale_out[0]
 * when that is not NULL.  The same bits as b200q_fp8_gemm_silu_mul followed by b200q_fp8_quantize with
 * amax_numel = 1; no bf16 activation is written at all. */
int b200q_fp8_gemm_silu_mul_quantize(const uint8_t* a_codes, const float* a_scales, int64_t a_scales_numel,
                                     const uint8_t* b_codes, const float* b_scales, int64_t b_scales_numel,
                                     const void* bias, const float* act_amax, uint8_t* codes_out,
                                     float* scale_out, int64_t M, int64_t N, int64_t K,
                                     b200q_stream_t stream, const b200q_cfg* cfg);
int b200q_nvfp4_gemm(const uint8_t* a_codes, const uint8_t* a_scales, const float* a_global,
                     const uint8_t* b_codes, const uint8_t* b_scales, const float* b_global,
                     const void* bias, void* out, int64_t M, int64_t N, int64_t K,
                     b200q_stream_t stream, const b200q_cfg* cfg);

/* ------------------------------------------------------------------ fused row-parallel linear (GEMM + all-reduce over peer memory)
 * Replaces "row-parallel linear, then tensorrt::fused_nccl_all_reduce" (the reference's
 * _RowParallelLinear, tools/llm/tensor_parallel_llama_export.py:109-125: out = linear(x);
 * all_reduce(out, "sum"); and the ALL_REDUCE collective layer of
 * py/torch_tensorrt/dynamo/conversion/impl/nccl_ops.py:440-451) by two launches:
 *
 *   b200q_*_gemm_reduce_scatter  the GEMM; its epilogue TMA-stores every 32-row panel of the
 *                                partial result straight into the receive buffer of the rank
 *                                that owns those rows (rank r owns rows [r*M/world, (r+1)*M/world)),
 *                                so the transfer overlaps the math tile by tile;
 *   b200q_reduce_gather          each rank sums the `world` partials of its rows, adds the bias
 *                                once, and stores the bf16 result into every rank's output.
 *
 * `b200q_peers` holds device pointers that are valid in THIS process for every rank's buffers
 * (peer mappings, e.g. from CUDA IPC or a symmetric-memory allocator):
 *   recv[r]   rank r's receive buffer, world * (M/world) * N bf16
 *   out[r]    rank r's output, M * N bf16
 *   flags[r]  rank r's flag words, at least 2 * world + 1 uint32, zeroed once before first use
 * M must be a multiple of world * 128 and N of 8.  `epoch` must increase by one with every
 * reduce_gather call on the group (all ranks pass the same value).  Both calls only enqueue
 * work; device-side waits for peers are bounded and reported through b200q_device_status().
 * The result is in out[rank] when the stream reaches the end of b200q_reduce_gather and stays
 * valid until the next b200q_reduce_gather of the group.
 */
typedef struct b200q_peers {
  int32_t rank;
  int32_t world;
  void* recv[8];
  void* out[8];
  uint32_t* flags[8];
} b200q_peers;

int b200q_fp8_gemm_reduce_scatter(const uint8_t* a_codes, const float* a_scales, int64_t a_scales_numel,
                                  const uint8_t* b_codes, const float* b_scales, int64_t b_scales_numel,
                                  const b200q_peers* peers, int64_t M, int64_t N, int64_t K,
                                  b200q_stream_t stream, const b200q_cfg* cfg);
int b200q_nvfp4_gemm_reduce_scatter(const uint8_t* a_codes, const uint8_t* a_scales, const float* a_global,
                                    const uint8_t* b_codes, const uint8_t* b_scales, const float* b_global,
                                    const b200q_peers* peers, int64_t M, int64_t N, int64_t K,
                                    b200q_stream_t stream, const b200q_cfg* cfg);
int b200q_reduce_gather(const b200q_peers* peers, const void* bias, int64_t M, int64_t N, uint32_t epoch,
                        b200q_stream_t stream, const b200q_cfg* cfg);

/* Native communication context: where the peer pointers of b200q_peers / b200q_gather_peers /
 * b200q_pull_peers come from when the host is C or C++ (one process per GPU on one node).  Takes the place
 * of TRTEngine::bind_nccl_comm (core/runtime/TRTEngine.cpp:821-928), which hands the process group's
 * communicator to the engine: these kernels need no communicator, only a pointer valid in this process for
 * every rank's copy of a buffer.  b200q_comm_alloc allocates `bytes` (zeroed) on the current device on
 * every rank, exchanges CUDA IPC handles through the host's own all-gather and opens the peers' handles:
 * ptrs[r] is rank r's buffer (ptrs[rank] the local one).  Collective: every rank calls it in the same
 * order with the same size.  This is set-up code: it allocates and synchronises; the compute entry points
 * never do.  b200q_comm_destroy (collective) unmaps and frees everything the context allocated.
 * `allgather(user, send, recv, bytes)`: every rank contributes `bytes` bytes, recv receives world * bytes
 * in rank order; returns 0 on success.  May be NULL when world == 1. */
typedef int (*b200q_allgather_fn)(void* user, const void* send, void* recv, size_t bytes);
typedef struct b200q_comm b200q_comm;
int b200q_comm_create(int rank, int world, b200q_allgather_fn allgather, void* user, b200q_comm** out);
int b200q_comm_alloc(b200q_comm* comm, size_t bytes, void* ptrs[8]);
int b200q_comm_destroy(b200q_comm* comm);

/* Token-sharded residual stream (sequence-parallel form of the same TP plan,
 * tools/llm/tensor_parallel_llama_llm.py:134-157): every rank keeps the residual rows it owns
 * ([M/world, N] bf16) and the reduction of a row-parallel linear is fused with what follows it.
 *   b200q_reduce_add_rms_norm_fp8_quantize_gather
 *        after b200q_*_gemm_reduce_scatter: sum the partials of this rank's rows, add the bias,
 *        h_shard += that (in place, bf16 rounding as b200q_add_rms_norm_fp8_quantize), RMSNorm
 *        with `norm_weight`, per-token FP8 quantize, and store codes and scales into codes[r] /
 *        scales[r] of EVERY rank: the gathered [M, N] operand of the next column-parallel GEMM.
 *        Only the 1-byte codes cross NVLink.  N % 16 == 0, N <= 16384.
 *   b200q_reduce_add_gather
 *        the last step of a stack: out[r] rows of this rank = residual_shard + sum + bias.
 * `b200q_gather_peers`: recv / flags as in b200q_peers; codes[r] = rank r's M * N bytes,
 * scales[r] = rank r's M floats.  Same epoch and flag rules as b200q_reduce_gather (one counter
 * for all three calls on a group). */
typedef struct b200q_gather_peers {
  int32_t rank;
  int32_t world;
  void* recv[8];
  uint8_t* codes[8];
  float* scales[8];
  uint32_t* flags[8];
} b200q_gather_peers;

int b200q_reduce_add_rms_norm_fp8_quantize_gather(const b200q_gather_peers* peers, const void* bias, void* h_shard,
                                                  const void* norm_weight, float eps, int64_t M, int64_t N,
                                                  uint32_t epoch, b200q_stream_t stream, const b200q_cfg* cfg);
int b200q_reduce_add_gather(const b200q_peers* peers, const void* bias, const void* residual_shard, int64_t M,
                            int64_t N, uint32_t epoch, b200q_stream_t stream, const b200q_cfg* cfg);

/* Decode-sized all-reduce by pulling (M <= 1024 rows, meant for the few tokens of a decode step).
 * Replaces the same ALL_REDUCE layer as above (py/torch_tensorrt/dynamo/conversion/impl/nccl_ops.py:440-451)
 * where the message is about a megabyte and one collective call per linear costs more than the
 * transfer.  The row-parallel GEMM (b200q_fp8_gemm / b200q_nvfp4_gemm, `out` = this rank's partial
 * buffer) is followed by
 *   b200q_pull_signal   tells every peer that this rank's partial is complete;
 *   b200q_pull_reduce_add_rms_norm_fp8_quantize
 *                       on EVERY rank: waits (bounded) for all peers' signals, reads all `world`
 *                       partials over peer memory, sums them in rank order (fp32), adds the bias once,
 *                       h += that (in place, the replicated residual stream [M, N] bf16), RMSNorm with
 *                       `norm_weight`, per-token FP8 codes [M, N] and scales [M] into LOCAL buffers;
 *   b200q_pull_reduce_add   the same without norm and quantize (end of a stack): h += sum + bias.
 * All ranks compute identical bits.  partial[r] = rank r's partial [M, N] bf16 for THIS all-reduce;
 * consecutive all-reduces of a group must alternate between two buffers per rank (a rank may
 * overwrite a buffer only after the next all-reduce on the other buffer has completed).
 * flags[r] = rank r's world + 1 uint32 words for this protocol, zeroed once; the call counter lives
 * in them on the device, so the launches can be captured in a CUDA graph and replayed.  N % 16 == 0,
 * N <= 16384. */
typedef struct b200q_pull_peers {
  int32_t rank;
  int32_t world;
  void* partial[8];
  uint32_t* flags[8];
} b200q_pull_peers;

int b200q_pull_signal(const b200q_pull_peers* peers, b200q_stream_t stream);
int b200q_pull_reduce_add_rms_norm_fp8_quantize(const b200q_pull_peers* peers, const void* bias, void* h,
                                                const void* norm_weight, float eps, uint8_t* codes_out,
                                                float* scales_out, int64_t M, int64_t N, b200q_stream_t stream,
                                                const b200q_cfg* cfg);
int b200q_pull_reduce_add(const b200q_pull_peers* peers, const void* bias, void* h, int64_t M, int64_t N,
                          b200q_stream_t stream, const b200q_cfg* cfg);

/* ------------------------------------------------------------------ FP8 attention
 * Replaces the TensorRT attention layer the reference builds for an SDPA whose Q, K and V all come from
 * `quantize_op(.., 8, 4, ..)` (py/torch_tensorrt/dynamo/lowering/passes/annotate_fp8_sdpa.py:34-76 marks it,
 * py/torch_tensorrt/dynamo/conversion/impl/attention.py:272-337 builds it): softmax output quantized to FP8
 * with the fixed scale 1/448, static `softmax_scale` (1/sqrt(D)) on the query.
 *   S = (Q_hat K_hat^T) * softmax_scale;  P = softmax(S) over the keys (causal = lower-right aligned mask);
 *   P_hat = e4m3(P * 448) / 448;  out = P_hat V_hat   in `out_dtype` (B200Q_BF16 / F16 / F32)
 * q_codes [B, Hq, Sq, D], k_codes [B, Hkv, Sk, D]: E4M3 codes (b200q_fp8_quantize with a per-tensor amax);
 * vt_codes [B, Hkv, D, vt_stride]: the codes of V TRANSPOSED per head, keys contiguous, zero beyond Sk
 * (b200q_fp8_quantize_transpose; vt_stride >= Sk, a multiple of 16).  q/k/v_scale: one fp32 each on the
 * device (the scales those quantize calls return).  Hq % Hkv == 0 (grouped-query attention: query head h
 * reads kv head h / (Hq / Hkv)); D % 16 == 0, D <= 128; B * Hq <= 65535.  Rows whose keys are all masked
 * get zeros.
 *
 * b200q_fp8_quantize_transpose: x [heads, S, D] (dtype) with a per-tensor amax -> codes [heads, D, s_stride],
 * scale_out (may be NULL) receives amax / 448 (zero -> 1). */
int b200q_fp8_quantize_transpose(const void* x, int dtype, int64_t heads, int64_t S, int64_t D, const float* amax,
                                 uint8_t* out_t, int64_t s_stride, float* scale_out, b200q_stream_t stream);
int b200q_fp8_sdpa(const uint8_t* q_codes, const uint8_t* k_codes, const uint8_t* vt_codes, const float* q_scale,
                   const float* k_scale, const float* v_scale, void* out, int out_dtype, int64_t B, int64_t Hq,
                   int64_t Hkv, int64_t Sq, int64_t Sk, int64_t vt_stride, int64_t D, float softmax_scale, int causal,
                   b200q_stream_t stream);

/* ------------------------------------------------------------------ glue of the decoder linear stack
 * The benchmark workloads wrap the quantized linears in a Llama-shaped decoder layer
 * (RMSNorm -> QKV -> attention replaced by identity on V -> O -> residual -> RMSNorm ->
 * gate/up -> silu(gate)*up -> down -> residual).  The reference lowers these to TensorRT
 * elementwise layers (RMSNorm: lowering/passes/replace_fused_rms_norm.py:12-92); here they are
 * plain streaming kernels over bf16 so that the stack runs without any library kernel.
 *   b200q_rms_norm      out = x * rsqrt(mean(x^2) + eps) * weight, per row; cols % 8 == 0
 *   b200q_add_rms_norm_fp8_quantize   the three steps in front of a quantized linear in one pass:
 *                       h_out = h + delta (delta NULL: no add, h_out unused), x = rms_norm(h_out),
 *                       per-token FP8 codes and scales of x; cols % 16 == 0, cols <= 16384
 *   b200q_silu_mul      out[t, j] = silu(gu[t, j]) * gu[t, f + j], gu is [rows, 2f]; f % 8 == 0
 *   b200q_add           out = a + b over n elements (n % 8 == 0)
 *   b200q_expand_heads  out[t, h*hd + d] = src[t*src_stride + src_col0 + (h / rep)*hd + d]
 *                       (every kv head repeated `rep` times: grouped-query V -> query width)
 */
int b200q_rms_norm(const void* x, const void* weight, void* out, int64_t rows, int64_t cols, float eps,
                   b200q_stream_t stream);
int b200q_add_rms_norm_fp8_quantize(const void* h, const void* delta, const void* weight, void* h_out,
                                    uint8_t* codes_out, float* scales_out, int64_t rows, int64_t cols,
                                    float eps, b200q_stream_t stream);
int b200q_silu_mul(const void* gate_up, void* out, int64_t rows, int64_t f, b200q_stream_t stream);
/* silu(gate) * up followed by the per-token FP8 quantize (b200q_fp8_quantize, dynamic per-row
 * amax) in one pass: codes [rows, f] and scales [rows] equal those of the two separate calls,
 * the bf16 activation is never written.  f % 8 == 0, f <= 32768. */
int b200q_silu_mul_fp8_quantize(const void* gate_up, uint8_t* codes_out, float* scales_out, int64_t rows, int64_t f,
                                b200q_stream_t stream);
int b200q_add(const void* a, const void* b, void* out, int64_t n, b200q_stream_t stream);
int b200q_expand_heads(const void* src, int64_t src_stride, int64_t src_col0, void* out, int64_t rows,
                       int heads_out, int rep, int head_dim, b200q_stream_t stream);
/* b200q_expand_heads followed by b200q_fp8_quantize (dynamic per-row amax) in one pass: codes
 * [rows, heads_out * head_dim] and scales [rows] equal those of the two separate calls; the kv slice of a
 * token ((heads_out / rep) * head_dim elements) may hold at most 2048 elements. */
int b200q_expand_heads_fp8_quantize(const void* src, int64_t src_stride, int64_t src_col0, uint8_t* codes_out,
                                    float* scales_out, int64_t rows, int heads_out, int rep, int head_dim,
                                    b200q_stream_t stream);

/* The GEMM kernels bound every device-side wait; a wait that gives up records it in a
 * device status word instead of hanging.  This call synchronises with the device, returns
 * B200Q_OK or B200Q_ERR_TIMEOUT, and clears the word when `reset` is non-zero. */
int b200q_device_status(int reset);

#ifdef __cplusplus
}
#endif
#endif /* B200Q_H_ */
