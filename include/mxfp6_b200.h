/*
 * C ABI of libmxfp6_b200.so: the W6A8 (packed MXFP6 E3M2 weights x MXFP8 E4M3
 * activations, UE8M0 scale per 32 K values) kernel library for NVIDIA B200
 * (sm_100a).
 *
 * Conventions
 *  - every pointer named *_dev or documented as "device" is a device pointer on
 *    the CUDA device that is current when the call is made;
 *  - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream);
 *  - calls only enqueue work; they never synchronise unless stated;
 *  - the return value is 0 on success; otherwise mxfp6_b200_last_error() returns a
 *    thread-local message (the reference raises TORCH_CHECK errors at the same
 *    places, e.g. csrc/torch_extension.cu:1769-1845);
 *  - dtype codes: 0 = float16, 1 = bfloat16.
 *
 * Each entry point names the reference operator it stands in for
 * (file:line inside Nekofish-L/mxfp6_sm120).
 */
#ifndef MXFP6_B200_H_
#define MXFP6_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MXFP6_B200_ABI_VERSION 5

#define MXFP6_DTYPE_F16 0
#define MXFP6_DTYPE_BF16 1

#define MXFP6_OK 0
#define MXFP6_ERR_INVALID_ARGUMENT 1
#define MXFP6_ERR_CUDA 2
#define MXFP6_ERR_UNSUPPORTED 3
#define MXFP6_ERR_DEVICE_TIMEOUT 4
#define MXFP6_ERR_WORKSPACE 5

int mxfp6_b200_abi_version(void);
const char* mxfp6_b200_last_error(void);

/* Synchronises the current device and reads the status word that kernels with
 * bounded waits write when a wait expires (0 = none did).  `reset` != 0 clears it. */
int mxfp6_b200_device_status(int* value, int reset);

/* ---- layout utilities ------------------------------------------------- */

/* torch.ops.mxfp6.pack_fp6 (csrc/torch_extension.cu:2121-2156, kernels
 * csrc/packing.cu:93-160): n codes (n % 4 == 0) -> n*3/4 bytes. */
int mxfp6_pack_fp6(const uint8_t* codes_dev, int64_t n, uint8_t* packed_dev, void* stream);
/* torch.ops.mxfp6.unpack_fp6 (csrc/packing.cu:162-200). */
int mxfp6_unpack_fp6(const uint8_t* packed_dev, int64_t rows, int64_t k, uint8_t* codes_dev,
                     void* stream);
/* torch.ops.mxfp6.pad_fp6 (csrc/packing.cu:202-218): every 12 bytes -> 16 bytes. */
int mxfp6_pad_fp6(const uint8_t* packed_dev, int64_t bytes, uint8_t* padded_dev, void* stream);
/* torch.ops.mxfp6.expand_fp6_to_fp8 (csrc/packing.cu:61-89,220-237). */
int mxfp6_expand_fp6_to_fp8(const uint8_t* packed_dev, int64_t rows, int64_t k,
                            uint8_t* e4m3_dev, void* stream);
/* torch.ops.mxfp6.pack_scales / unpack_scales (csrc/packing.cu:239-283): logical
 * [rows, k/32] <-> packed ceil128(rows) * ceil4(k/32) bytes, padding = 0x7f. */
int mxfp6_pack_scales(const uint8_t* logical_dev, int64_t rows, int64_t k, uint8_t* packed_dev,
                      void* stream);
int mxfp6_unpack_scales(const uint8_t* packed_dev, int64_t rows, int64_t k,
                        uint8_t* logical_dev, void* stream);
int64_t mxfp6_packed_scale_bytes(int64_t rows, int64_t k);
/* torch.ops.mxfp6.pack_grouped_scales (csrc/moe.cu:4206-4224,4790-4826):
 * scale_offsets[e] = sum of ceil128(rows of experts before e). */
int mxfp6_grouped_scale_offsets(const int64_t* expert_offsets_dev, int experts,
                                int64_t* scale_offsets_dev, void* stream);
int mxfp6_pack_grouped_scales(const uint8_t* logical_dev, const int64_t* expert_offsets_dev,
                              const int64_t* scale_offsets_dev, int experts,
                              int64_t padded_rows, int64_t k, uint8_t* packed_dev, void* stream);

/* ---- quantizers --------------------------------------------------------- */

/* torch.ops.mxfp6.quantize_mxfp8 / _logical / _dual / _dual_out
 * (csrc/quantization.cu:70-191,247-404).  Either scale output may be NULL. */
int mxfp6_quantize_mxfp8(const void* input_dev, int dtype, int64_t rows, int64_t k,
                         uint8_t* values_dev, uint8_t* packed_scales_dev,
                         uint8_t* logical_scales_dev, void* stream);
/* Residual add + RMSNorm fused into the MXFP8 quantizer.  With residual_dev: x <-
 * round(x + residual) is written to updated_dev (may equal input_dev) first; both NULL
 * skips the add.  Then y = round((x * rsqrt(mean(x^2) + eps)) * weight) in the input dtype
 * (one rounding, as torch.nn.functional.rms_norm) and the rule of mxfp6_quantize_mxfp8 on
 * y.  One pass over the row; k <= 16384.  No reference counterpart: the reference leaves
 * the residual stream and normalisation to the serving runtime
 * (docs/runtime-integration.md:13-22) and quantizes its BF16 output
 * (csrc/quantization.cu:70-191). */
int mxfp6_rmsnorm_quantize_mxfp8(const void* input_dev, const void* residual_dev,
                                 void* updated_dev, int dtype, const void* weight_dev, float eps,
                                 int64_t rows, int64_t k, uint8_t* values_dev,
                                 uint8_t* packed_scales_dev, uint8_t* logical_scales_dev,
                                 void* stream);
/* torch.ops.mxfp6.quantize_mxfp6 (csrc/quantization.cu:193-243,406-409):
 * values are the packed 6-bit stream (rows * k * 3/4 bytes). */
int mxfp6_quantize_mxfp6(const void* input_dev, int dtype, int64_t rows, int64_t k,
                         uint8_t* values_dev, uint8_t* packed_scales_dev,
                         uint8_t* logical_scales_dev, void* stream);

/* ---- tensor-parallel decode path over peer memory ------------------------------ */

/* All-reduce of a row-parallel projection fused with the residual add, RMSNorm and MXFP8
 * quantization that consume it (the B200 successor of the reference's two-rank reducer with
 * peer signal pointers, csrc/moe.cu:7698-7925; every wait here is bounded).
 *
 * Set-up, once: every rank allocates a symmetric block (flags + state + two partial
 * buffers of partial_bytes each, a multiple of 256), sends its 64-byte CUDA IPC handle to
 * its peers (any host channel) and opens theirs.  A row-parallel GEMM writes its BF16
 * [rows, k] partial at block + MXFP6_TP_BLOCK_HEADER_BYTES + buffer * partial_bytes of its
 * OWN block, alternating buffer 0 / 1 from one fused call to the next.  Then on every rank,
 * on the stream the GEMM ran on:
 *   x <- bf16(x + bf16(sum over ranks, in rank order, of the partials));
 *   values / packed_scales <- MXFP8(round(x * rsqrt(mean(x^2) + eps) * weight)).
 * blocks_host[r] is this process's mapping of rank r's block (its own allocation for
 * r == rank).  All ranks must issue the same sequence of calls.  A peer that does not
 * arrive within about 2 s sets device status 301 and leaves x unchanged. */
#define MXFP6_TP_BLOCK_HEADER_BYTES 1024
int mxfp6_tp_block_alloc(size_t partial_bytes, void** block_dev_out, unsigned char handle_out[64]);
int mxfp6_tp_block_open(const unsigned char handle[64], void** block_dev_out);
int mxfp6_tp_block_close(void* block_dev);
int mxfp6_tp_block_free(void* block_dev);
/* Consecutive collectives on one set of blocks must alternate the two partial buffers: a
 * rank that has passed step s + 1 has seen every peer finish step s, nothing more.  The
 * last buffer is recorded in the block; a step that names it again (a replayed graph with
 * an odd number of collectives) sets device status 302 and moves no data.
 * The limit of the flag wait (the reference's spin is unbounded, csrc/moe.cu:7774,7795),
 * in GPU clock ticks (about 1.9e9 per second); the default is about two seconds. */
int mxfp6_tp_set_wait_limit(int64_t clock_ticks);
int64_t mxfp6_tp_get_wait_limit(void);
/* The plain form of the same collective: out <- bf16(sum over ranks, in rank order, of the
 * [rows, k] BF16 partials in buffer `buffer` of every block).  Used by the MoE reducer's
 * tensor-parallel sum (the reference's moe_reduce_tp2_out, csrc/moe.cu:7698-7925).  It counts
 * as one step of the alternating-buffer sequence like the fused call below. */
int mxfp6_tp_allreduce_bf16(void* const* blocks_host, int world, int rank, int buffer,
                            size_t partial_bytes, void* out_dev, int64_t rows, int64_t k,
                            void* stream);
/* The same sum for bandwidth-bound sizes, in two launches that count as two steps on ONE
 * buffer: every rank sums its slice of rows (rows % world == 0) over all ranks in place,
 * then all ranks gather the reduced slices into out.  2 * (world - 1) / world of the
 * tensor crosses NVLink per rank instead of world - 1 times the tensor. */
int mxfp6_tp_allreduce_two_phase_bf16(void* const* blocks_host, int world, int rank, int buffer,
                                      size_t partial_bytes, void* out_dev, int64_t rows,
                                      int64_t k, void* stream);
/* Reduce-scatter form: out [rows_per_rank, k] <- bf16(sum over ranks of rows
 * [rank * rows_per_rank, (rank + 1) * rows_per_rank) of every rank's [world * rows_per_rank, k]
 * BF16 partial).  The expert-parallel combine: every rank sums the partial rows of ITS tokens
 * (the reference leaves this exchange to the caller, csrc/moe.cu:4243-4261). */
int mxfp6_tp_reduce_scatter_bf16(void* const* blocks_host, int world, int rank, int buffer,
                                 size_t partial_bytes, void* out_dev, int64_t rows_per_rank,
                                 int64_t k, void* stream);
/* All-gather of 1..4 byte segments with one handshake: segment s of rank r, found at
 * offsets[s] inside r's partial buffer, lands at dsts_dev[s] + r * bytes[s].  Offsets and
 * sizes are multiples of 16.  The expert-parallel dispatch (MXFP8 rows, scale rows, top-k
 * ids and weights of every rank's tokens). */
int mxfp6_tp_allgather(void* const* blocks_host, int world, int rank, int buffer,
                       size_t partial_bytes, int segments, const int64_t* offsets,
                       const int64_t* bytes, void* const* dsts_dev, void* stream);
int mxfp6_tp_allreduce_rmsnorm_quantize_mxfp8(void* const* blocks_host, int world, int rank,
                                              int buffer, size_t partial_bytes, void* x_dev,
                                              const void* weight_dev, float eps, int64_t rows,
                                              int64_t k, uint8_t* values_dev,
                                              uint8_t* packed_scales_dev, void* stream);

/* ---- dense W6A8 GEMM ------------------------------------------------------ */

/* torch.ops.mxfp6.gemm_w6a8 (csrc/torch_extension.cu:1769-1845):
 * out[m, n] = alpha * A8[m, k] x W6[n, k]^T.  m > 0, n % 8 == 0, k % 128 == 0.
 * Split-K scratch comes from the per-device workspace arena (below). */
int mxfp6_gemm_w6a8(const uint8_t* a_values_dev, const uint8_t* a_scales_dev,
                    const uint8_t* w_values_dev, const uint8_t* w_scales_dev, int64_t m,
                    int64_t n, int64_t k, float alpha, void* out_dev, int out_dtype,
                    void* stream);
/* Same with an explicit tile/split choice and caller-owned scratch
 * (tile_tokens / splits = 0 selects from the built-in table; the stand-in for
 * torch.ops.mxfp6.gemm_w6a8_config, csrc/torch_extension.cu:1847-1867).  When the
 * chosen plan splits K, scratch_dev must hold mxfp6_gemm_w6a8_scratch_bytes()
 * bytes whose trailing counter region was zeroed once. */
int mxfp6_gemm_w6a8_ex(const uint8_t* a_values_dev, const uint8_t* a_scales_dev,
                       const uint8_t* w_values_dev, const uint8_t* w_scales_dev, int64_t m,
                       int64_t n, int64_t k, float alpha, void* out_dev, int out_dtype,
                       int tile_tokens, int splits, void* scratch_dev, size_t scratch_bytes,
                       void* stream);
/* No counterpart in the reference.  The same GEMM for callers that cannot allocate
 * device memory: code running inside somebody else's CUDA-graph capture, servers
 * whose memory pool is fixed at start-up, plugins that may not touch their host's
 * allocator.  The split-K scratch and the status word live in a fixed array inside
 * the library image (4 MiB of partial tiles + 4 KiB of tile counters, held by every
 * GPU that loads the library until the process exits), and the call performs no
 * cudaMalloc / cudaFree / stream-ordered allocation.  A problem whose plan needs
 * more scratch than that is rejected with MXFP6_ERR_INVALID_ARGUMENT and a message
 * that gives both sizes.  The first call on each device looks up the array's device
 * address, and the first launch of each tile width on a device sets a kernel attribute
 * and loads its code: make one call per batch-size class (m <= 16, 32, 64, 96, 128,
 * larger) outside any stream capture first.  All calls share the one
 * array: the counters are cleared on the stream at every call, and two calls whose
 * kernels overlap on the GPU (different streams) race on it. */
int mxfp6_gemm_w6a8_static_scratch(const uint8_t* a_values_dev, const uint8_t* a_scales_dev,
                                   const uint8_t* w_values_dev, const uint8_t* w_scales_dev,
                                   int64_t m, int64_t n, int64_t k, float alpha, void* out_dev,
                                   int out_dtype, void* stream);
/* Plan query: fills tile_tokens, scratch splits, stages, grid, partial bytes, counter
 * bytes, cluster split factor, 1 when the two-CTA kernel runs the problem, the kernel
 * family (0 persistent single-CTA, 1 CTA pair, 2 weight streaming) and the dynamic shared
 * memory of a CTA.  A registered override of the exact problem with BF16 output
 * (mxfp6_set_w6a8_config) is applied when tile_tokens and splits are both 0. */
int mxfp6_gemm_w6a8_plan(int64_t m, int64_t n, int64_t k, int tile_tokens, int splits,
                         int64_t out_plan[10]);
/* Dense launches of at most 64 rows run on the weight-streaming kernel (two CTAs per SM,
 * weights prefetched ahead of the programmatic-launch wait, cluster push reduction);
 * 0 sends them to the persistent kernel instead.  Default 1. */
int mxfp6_set_stream_kernel_mode(int enabled);
int mxfp6_get_stream_kernel_mode(void);
/* torch.ops.mxfp6.w6a8_config_abi (csrc/torch_extension.cu:1169-1172, schema :2138):
 * names the set of explicit configurations; ids are only meaningful under the same string. */
const char* mxfp6_w6a8_config_abi(void);
int mxfp6_w6a8_config_count(void);
/* out = {kernel family, tile_tokens, cluster_k, scratch splits} of a configuration id. */
int mxfp6_w6a8_config_describe(int config_id, int out[4]);
/* torch.ops.mxfp6.set_w6a8_config (csrc/torch_extension.cu:1139-1167, schema :2135):
 * later mxfp6_gemm_w6a8 / mxfp6_gemm_from_float calls on the current device with exactly
 * this (m, n, k, out_dtype) run configuration `config_id`; a negative id erases the entry.
 * A configuration that cannot run the problem is rejected here. */
int mxfp6_set_w6a8_config(int64_t m, int64_t n, int64_t k, int out_dtype, int config_id);
/* torch.ops.mxfp6.gemm_w6a8_config (csrc/torch_extension.cu:1847-1867, schema :2127):
 * one launch of an explicit configuration; scratch splits use the workspace arena. */
int mxfp6_gemm_w6a8_config(const uint8_t* a_values_dev, const uint8_t* a_scales_dev,
                           const uint8_t* w_values_dev, const uint8_t* w_scales_dev, int64_t m,
                           int64_t n, int64_t k, float alpha, void* out_dev, int out_dtype,
                           int config_id, void* stream);
/* How launches with too few tiles split K (the stand-in for the reference's
 * MXFP6_STREAM_K switch, csrc/torch_extension.cu:35-57): 1 = thread-block clusters
 * that reduce through distributed shared memory (default, no scratch), 2 = FP32
 * partial tiles in the scratch arena, 3 = never split. */
int mxfp6_set_split_k_mode(int mode);
int mxfp6_get_split_k_mode(void);
/* Dense launches with m > 128, n % 128 == 0 and n >= 256 run on CTA pairs (tcgen05 cta_group::2:
 * 256 weight rows per tile, each CTA stages half of the activation tile); 0 keeps them
 * on the single-CTA kernel.  Default 1.  Results are bit-identical either way.  No
 * reference counterpart: the reference picks kernels in its autotuner,
 * python/mxfp6/autotune.py:33-85 (candidate list), :552-885 (search). */
int mxfp6_set_cta_pair_mode(int enabled);
int mxfp6_get_cta_pair_mode(void);
/* torch.ops.mxfp6.gemm_from_float (csrc/torch_extension.cu:1869-1925): quantize the
 * FP16/BF16 activation to MXFP8 into caller-provided staging buffers
 * (m*k bytes and mxfp6_packed_scale_bytes(m, k) bytes), then run the GEMM. */
int mxfp6_gemm_from_float(const void* a_dev, int a_dtype, const uint8_t* w_values_dev,
                          const uint8_t* w_scales_dev, int64_t m, int64_t n, int64_t k,
                          float alpha, void* out_dev, int out_dtype, uint8_t* a_values_stage_dev,
                          uint8_t* a_scales_stage_dev, void* stream);

/* ---- routed MoE -----------------------------------------------------------------
 * All calls are allocation-free and capturable in a CUDA graph. */

/* torch.ops.mxfp6.qwen35_topk_quant_out (csrc/moe.cu:620-962, host :9716-10008):
 * per token, MXFP8-quantize the BF16 hidden row (values, logical scales [T, H/32]
 * and/or dense packed scales; all three optional together with `quantized` NULL)
 * and take the softmax top-k of its BF16 router logits (FP32 weights, INT32 ids;
 * ties go to the smaller id; renormalize divides by the sum of the k weights).
 * Generic in H (multiple of 32), experts (<= 1024) and k (<= 16). */
int mxfp6_moe_topk_quant(const void* hidden_dev, const void* logits_dev, int64_t tokens,
                         int hidden_size, int experts, int topk, int renormalize,
                         uint8_t* quantized_dev, uint8_t* logical_scales_dev,
                         uint8_t* dense_scales_dev, float* topk_weights_dev,
                         int32_t* topk_ids_dev, void* stream);
/* torch.ops.mxfp6.route_mxfp8_out / qwen35_route_mxfp8_out (csrc/moe.cu:4263-4446):
 * expert_offsets[E+1] (exclusive prefix of counts), scale_offsets[E+1] (prefix of
 * 128-padded counts), cursors[E] (scratch), inverse_permutation[T*k] (route -> row,
 * -1 for routes whose expert is not local), optional source_tokens[row], optional
 * copy of the MXFP8 rows into permuted[T*k, H], and the rows' scales in the grouped
 * packed layout.  expert_map (global id -> local id or -1) may be NULL. */
int mxfp6_moe_route(const uint8_t* activation_dev, const uint8_t* logical_scales_dev,
                    const void* topk_ids_dev, int ids_are_int64, int64_t tokens, int topk,
                    int hidden_size, const int32_t* expert_map_dev, int expert_map_size,
                    int local_experts, int64_t* expert_offsets_dev, int64_t* scale_offsets_dev,
                    int32_t* cursors_dev, uint8_t* permuted_dev, uint8_t* grouped_scales_dev,
                    int32_t* inverse_permutation_dev, int32_t* source_tokens_dev, void* stream);
/* The same with the reference's include_shared flag (csrc/moe.cu:4449-4631, the shared_rows
 * of its histogram and gather kernels): when set, local_experts counts one TRAILING shared
 * expert that no id selects (ids and expert_map values must lie below local_experts - 1, others
 * are dropped); its group holds one row per token, token t at row
 * expert_offsets[local_experts - 1] + t, after all routed rows.  permuted then has
 * T*k + T rows, the scale buffer one more padded group, and inverse_permutation still T*k
 * entries (the shared rows are addressed through the offset, not through it). */
int mxfp6_moe_route_shared(const uint8_t* activation_dev, const uint8_t* logical_scales_dev,
                           const void* topk_ids_dev, int ids_are_int64, int64_t tokens, int topk,
                           int hidden_size, const int32_t* expert_map_dev, int expert_map_size,
                           int local_experts, int include_shared, int64_t* expert_offsets_dev,
                           int64_t* scale_offsets_dev, int32_t* cursors_dev,
                           uint8_t* permuted_dev, uint8_t* grouped_scales_dev,
                           int32_t* inverse_permutation_dev, int32_t* source_tokens_dev,
                           void* stream);
/* torch.ops.mxfp6.qwen35_topk_quant_route_out (csrc/moe.cu:620-962, host :9716-10008):
 * mxfp6_moe_topk_quant followed by mxfp6_moe_route.  Batches of at most 8 tokens
 * (and tokens * topk <= 1024) run as ONE single-CTA kernel; larger ones as three. */
int mxfp6_moe_topk_quant_route(const void* hidden_dev, const void* logits_dev, int64_t tokens,
                               int hidden_size, int experts, int topk, int renormalize,
                               uint8_t* quantized_dev, uint8_t* logical_scales_dev,
                               uint8_t* dense_scales_dev, float* topk_weights_dev,
                               int32_t* topk_ids_dev, const int32_t* expert_map_dev,
                               int expert_map_size, int local_experts,
                               int64_t* expert_offsets_dev, int64_t* scale_offsets_dev,
                               int32_t* cursors_dev, uint8_t* permuted_dev,
                               uint8_t* grouped_scales_dev, int32_t* inverse_permutation_dev,
                               int32_t* source_tokens_dev, void* stream);
/* torch.ops.mxfp6.grouped_gemm_w6a8_out (csrc/moe.cu:7551-7676): rows
 * [expert_offsets[e], expert_offsets[e+1]) of the activation times weight e
 * ([E, n, k*3/4] bytes, scales [E, n*k/32]); n % 128 == 0, k % 128 == 0.
 * m_total is the row capacity of the activation / output buffers. */
int mxfp6_grouped_gemm_w6a8(void* out_dev, int out_dtype, const uint8_t* activation_dev,
                            const uint8_t* activation_scales_dev, int64_t activation_scale_rows,
                            const uint8_t* weight_dev, const uint8_t* weight_scales_dev,
                            const int64_t* expert_offsets_dev, const int64_t* scale_offsets_dev,
                            int experts, int64_t m_total, int64_t n, int64_t k, int tile_tokens,
                            void* stream);
/* torch.ops.mxfp6.qwen35_grouped_w1_silu_mxfp8_out (csrc/moe.cu:2288-2687, host
 * :4106-4204): W1 = [E, 2*inter, k] (gate rows, then up rows); output E4M3
 * [m_total, inter] = MXFP8(bf16(silu(bf16 gate)) * bf16 up) with scales in the grouped
 * packed layout (same scale_offsets) and/or logical [m_total, inter/32].  With
 * expert_offsets == NULL and experts == 1 it is the dense form used for the shared
 * expert (activation scales and output scales in the dense packed layout). */
int mxfp6_w1_swiglu_mxfp8(uint8_t* output_dev, uint8_t* out_packed_scales_dev,
                          uint8_t* out_logical_scales_dev, const uint8_t* activation_dev,
                          const uint8_t* activation_scales_dev, int64_t activation_scale_rows,
                          const uint8_t* weight_dev, const uint8_t* weight_scales_dev,
                          const int64_t* expert_offsets_dev, const int64_t* scale_offsets_dev,
                          int experts, int64_t m_total, int64_t inter, int64_t k, int tile_tokens,
                          void* stream);
/* torch.ops.mxfp6.silu_and_mul_mxfp8_{grouped,grouped_out,logical,packed_out}
 * (csrc/moe.cu:5135-5282): input FP16/BF16 [rows, 2*inter]; output E4M3 [rows, inter];
 * scales logical and/or packed (grouped when the offset arrays are given). */
int mxfp6_silu_and_mul_mxfp8(const void* input_dev, int dtype, int64_t rows, int64_t inter,
                             uint8_t* output_dev, uint8_t* logical_scales_dev,
                             uint8_t* packed_scales_dev, const int64_t* expert_offsets_dev,
                             const int64_t* scale_offsets_dev, int experts, void* stream);
/* ---- decode batches: one single-row GEMM per route, no permutation ------------------
 * Route r = token * lanes + lane, lanes = topk + (include_shared ? 1 : 0); its expert is
 * topk_ids[token, lane] (int32, or int64 with ids_are_int64), the lane after the last routed
 * one is the always-on shared expert: the last matrix of the stack, or a separate matrix.
 * Routes whose id is outside [0, experts) are left unwritten.  Activation scales are LOGICAL
 * [rows, k/32]; activation_rows is tokens (all lanes of a token read one row) or
 * tokens * lanes.  n % 128 == 0, k % 128 == 0, k <= 8192.
 *
 * torch.ops.mxfp6.array_gemm_w6a8_out (schema csrc/moe.cu:10048-10051, host :6713-6864):
 * output FP16/BF16 [routes, n]. */
int mxfp6_array_gemm_w6a8(void* output_dev, int out_dtype, const uint8_t* activation_dev,
                          const uint8_t* logical_scales_dev, int64_t activation_rows,
                          const uint8_t* weight_dev, const uint8_t* weight_scales_dev, int experts,
                          const void* topk_ids_dev, int ids_are_int64, int64_t tokens, int topk,
                          int include_shared, int64_t n, int64_t k, void* stream);
/* torch.ops.mxfp6.array_gemm_w6a8_silu_mxfp8_out and qwen35_w1_splitk_silu_mxfp8_out (schemas
 * csrc/moe.cu:10052-10057, 10089-10096; hosts :6866-6982, :8648-8916): weights hold 2 * inter
 * rows per expert (gate rows, then up rows); output E4M3 [routes, inter] with logical scales
 * [routes, inter / 32].  shared_weight (one expert, with its scales) may be NULL. */
int mxfp6_array_gemm_w6a8_silu_mxfp8(uint8_t* output_dev, uint8_t* output_scales_dev,
                                     const uint8_t* activation_dev,
                                     const uint8_t* logical_scales_dev, int64_t activation_rows,
                                     const uint8_t* weight_dev, const uint8_t* weight_scales_dev,
                                     int experts, const uint8_t* shared_weight_dev,
                                     const uint8_t* shared_weight_scales_dev,
                                     const void* topk_ids_dev, int ids_are_int64, int64_t tokens,
                                     int topk, int include_shared, int64_t inter, int64_t k,
                                     void* stream);
/* torch.ops.mxfp6.array_gemm_w6a8_reduce_out and qwen35_w2_splitk_reduce_out (schemas
 * csrc/moe.cu:10058-10065, 10097-10103; hosts :6984-7393, :9120-9396): activation
 * [tokens * lanes, k] with lanes = topk + compute_shared;
 * output[t] = cast(sigmoid(gate[t]) * shared[t] + sum_l w[t, l] * cast(routed[t, l])), FP32,
 * shared term first, where the shared row is computed here (compute_shared), given
 * (shared_output_dev, [tokens, n] of the output type) or absent.  At most 9 lanes, k <= 2048.
 * routing_ready != 0: the caller vouches that topk_ids were complete before the kernel that
 * precedes this one on the stream let its dependents start (true behind
 * mxfp6_array_gemm_w6a8_silu_mxfp8, which waits for its own inputs first); the kernel then
 * fetches the experts' weights before its dependency wait.  0 is always safe. */
int mxfp6_array_gemm_w6a8_reduce(void* output_dev, int out_dtype, const uint8_t* activation_dev,
                                 const uint8_t* logical_scales_dev, const uint8_t* weight_dev,
                                 const uint8_t* weight_scales_dev, int experts,
                                 const uint8_t* shared_weight_dev,
                                 const uint8_t* shared_weight_scales_dev, const void* topk_ids_dev,
                                 int ids_are_int64, const float* topk_weights_dev,
                                 const void* shared_gate_dev, int gate_dtype, int gate_stride,
                                 const void* shared_output_dev, int compute_shared, int64_t tokens,
                                 int topk, int64_t n, int64_t k, int routing_ready, void* stream);
/* The decode schedule of python/mxfp6/qwen35.py:384-432 from given router logits, in two
 * launches: W1 over the routes (top-k + shared expert per token) with the softmax top-k and
 * the MXFP8 quantization of the hidden rows done inside every CTA (the arithmetic of
 * mxfp6_moe_topk_quant), then W2 with the weighted reduce and the gated shared row.  hidden
 * [tokens, hidden_size] and router_logits [tokens, logit_experts] are BF16; w1 is
 * [experts, 2 * inter, 3 * hidden_size / 4], w2 [experts, hidden_size, 3 * inter / 4], the last
 * matrix of both the shared expert unless the four shared_* pointers bring it; activation
 * [tokens * (topk + 1), inter] + activation_scales [.., inter / 32] are scratch; topk_ids /
 * topk_weights receive the selection; output [tokens, hidden_size].  w2_own_routing != 0: the
 * second launch repeats the selection for itself before its dependency wait and fetches
 * weights meanwhile; 0: it reads topk_ids / topk_weights once the first has completed (same
 * bytes either way).  _supported returns 1 when
 * the shapes fit (topk <= 8, inter <= 2048, at most 16 blocks of 128 hidden values per CTA of
 * the W1 launch); otherwise use the three entry points above.  _preferred returns 1 when this
 * form is also expected to be the faster one (measured: wherever it is supported). */
int mxfp6_moe_decode_layer_supported(int64_t tokens, int topk, int logit_experts,
                                     int64_t hidden_size, int64_t inter);
int mxfp6_moe_decode_layer_preferred(int64_t tokens, int topk, int logit_experts,
                                     int64_t hidden_size, int64_t inter);
int mxfp6_moe_decode_layer(void* output_dev, int out_dtype, const void* hidden_dev,
                           const void* router_logits_dev, const void* shared_gate_dev,
                           int gate_dtype, int gate_stride, const uint8_t* w1_dev,
                           const uint8_t* w1_scales_dev, const uint8_t* w2_dev,
                           const uint8_t* w2_scales_dev, int experts, const uint8_t* shared_w1_dev,
                           const uint8_t* shared_w1_scales_dev, const uint8_t* shared_w2_dev,
                           const uint8_t* shared_w2_scales_dev, uint8_t* activation_dev,
                           uint8_t* activation_scales_dev, int32_t* topk_ids_dev,
                           float* topk_weights_dev, int64_t tokens, int topk, int logit_experts,
                           int renormalize, int64_t hidden_size, int64_t inter, int w2_own_routing,
                           void* stream);
/* torch.ops.mxfp6.moe_reduce_array_out (schema csrc/moe.cu:10129-10131, kernel :8237-8282):
 * combined [tokens * (topk + 1), hidden], the shared row last of each token. */
int mxfp6_moe_reduce_array(void* output_dev, const void* combined_dev, int dtype,
                           const float* topk_weights_dev, const void* shared_gate_dev,
                           int gate_dtype, int gate_stride, int64_t tokens, int topk,
                           int64_t hidden_size, void* stream);
/* Router half of torch.ops.mxfp6.qwen35_router_quant_out (schema csrc/moe.cu:10066-10072, kernel
 * :237-511): routed_logits[b, e] = bf16(hidden[b] . gate[e]) in FP32 for e < routed_experts;
 * the shared expert's gate logit (row routed_experts of gate_weight when gate_rows says so,
 * else shared_gate_weight) goes to shared_gate[b].  All BF16. */
int mxfp6_moe_router_logits(const void* hidden_dev, const void* gate_weight_dev,
                            const void* shared_gate_weight_dev, void* routed_logits_dev,
                            void* shared_gate_dev, int64_t batch, int64_t k, int routed_experts,
                            int gate_rows, void* stream);
/* torch.ops.mxfp6.moe_reduce_out (csrc/moe.cu:7927-8082, host :8377-8531):
 * out[t] = cast(sigmoid(gate[t]) * shared[t] + sum_r w[t,r] * routed[inv[t,r]]), FP32.
 * shared / shared_gate may be NULL; gate dtype 0/1/2 = f16/bf16/f32; gate_stride is
 * the row length of the gate tensor (its last column is used). */
int mxfp6_moe_reduce(void* out_dev, const void* routed_dev, int dtype,
                     const float* topk_weights_dev, const int32_t* inverse_permutation_dev,
                     const void* shared_dev, const void* shared_gate_dev, int gate_dtype,
                     int gate_stride, int64_t tokens, int hidden_size, int topk,
                     int64_t routed_rows, void* stream);
/* torch.ops.mxfp6.moe_reduce_tp2_out (schema csrc/moe.cu:10124-10128, kernel :7698-7925) with
 * the reference's argument list: the reduce above (BF16) into this rank's data buffer, then
 * the sum over `world` ranks (2 in the reference, up to 8 here) in rank order, FP32, rounded
 * once.  signal_ptrs_host[r] / buffer_ptrs_host[r]: rank r's signal area (>= 64 bytes, zero
 * before the first call) and data buffer (>= tokens * hidden * 2 bytes), both valid on this
 * device.  Every wait is bounded (status 301); a closing handshake makes the single buffer
 * safe to rewrite when the call's last kernel has run. */
int mxfp6_moe_reduce_tp_pointers(void* out_dev, const void* routed_dev,
                                 const float* topk_weights_dev,
                                 const int32_t* inverse_permutation_dev, const void* shared_dev,
                                 const void* shared_gate_dev, int gate_dtype, int gate_stride,
                                 int64_t tokens, int hidden_size, int topk, int64_t routed_rows,
                                 const uint64_t* signal_ptrs_host,
                                 const uint64_t* buffer_ptrs_host, int world, int rank,
                                 void* stream);

/* ---- split-K workspace arena ----------------------------------------------
 * torch.ops.mxfp6.begin_workspace_planning / finalize_workspace_planning /
 * workspace_stats / workspace_barriers_zero (csrc/torch_extension.cu:1955-2116).
 * While planning, launches record the scratch they need and use a transient
 * stream-ordered allocation.  finalize freezes the capacity; afterwards each
 * stream gets one persistent lane on its first eager launch and a launch that
 * is being captured on a stream without a lane fails. */
int mxfp6_workspace_begin_planning(void);
int mxfp6_workspace_finalize_planning(void* stream, int64_t out_stats[10]);
/* stats, in the order of the reference's dictionary
 * (csrc/torch_extension.cu:1965-1991): [0] layouts, [1] max_reduction_bytes,
 * [2] max_barrier_bytes, [3] arena_bytes, [4] lanes, [5] total_arena_bytes,
 * [6] planning, [7] frozen, [8] persistent_launches, [9] fallback_launches */
int mxfp6_workspace_stats(int64_t out_stats[10]);
int mxfp6_workspace_barriers_zero(int* all_zero);
/* Drops every lane and returns the arena to its initial state (test helper). */
int mxfp6_workspace_reset(void);

#ifdef __cplusplus
}
#endif

#endif /* MXFP6_B200_H_ */
