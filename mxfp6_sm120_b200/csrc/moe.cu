// Routed-MoE support kernels: softmax top-k + MXFP8 quantization of the token rows,
// expert histogram / offsets, row permutation with grouped-packed scales, the
// unfused SiLU*mul + MXFP8 requantization, and the weighted reduce with the gated
// shared expert.
//
// Arithmetic follows the reference:
//   * top-k: FP32 softmax of BF16 logits (expf, max-subtracted, multiply by 1/sum,
//     non-finite -> 0), k rounds of arg-max with ties to the smaller expert id,
//     optional renormalisation w / sum(w)            (csrc/moe.cu:412-510);
//   * routing: counts -> exclusive prefix = expert_offsets, prefix of 128-padded
//     counts = scale_offsets, row order inside an expert is arrival order
//                                                     (csrc/moe.cu:4263-4446);
//   * SiLU path: g = bf16(a_g); u = bf16(a_u); s = bf16(g / (1 + expf(-g)));
//     v = bf16(s * u); MXFP8 quantization of v per 32   (csrc/moe.cu:5199-5205);
//   * reduce: out[t] = cast(sigmoid(gate_t) * shared[t] + sum_r w[t,r] * routed[inv[t,r]])
//     in FP32, shared term first, routes in order       (csrc/moe.cu:7972-7988).
// The launch shapes are new and generic in hidden size, expert count and k.
#include "common.cuh"

#include "topk.cuh"

#include <cuda_fp8.h>

#include <cstdlib>

namespace mx {
namespace {

constexpr int kMaxTopk = 16;
constexpr int kMaxExperts = 1024;

__device__ __forceinline__ uint32_t e4m3x4(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

// Softmax top-k of one token by one warp (topk.cuh), written to the token's rows.
__device__ __forceinline__ void warp_softmax_topk(const __nv_bfloat16* __restrict__ logits_row,
                                                  int experts, int topk, int renormalize,
                                                  float* __restrict__ weights_row,
                                                  int32_t* __restrict__ ids_row, int lane) {
  float weight;
  int id;
  warp_softmax_topk_any(logits_row, experts, topk, renormalize, lane, &weight, &id);
  if (lane < topk) {
    weights_row[lane] = weight;
    ids_row[lane] = id;
  }
}

// ---------------------------------------------------------------- top-k + quantize
// One CTA per `tokens_per_cta` tokens (1 for decode batches, 8 otherwise).  The first 256
// threads quantize the rows; then one warp per token does the softmax top-k.  A CTA of 288
// threads (one token per CTA) gives the top-k a warp of its own, beside the quantization.
constexpr int kQuantThreads = 256;

__global__ void __launch_bounds__(kQuantThreads + 32)
topk_quant_kernel(const __nv_bfloat16* __restrict__ hidden, const __nv_bfloat16* __restrict__ logits,
                  uint8_t* __restrict__ quantized, uint8_t* __restrict__ logical_scales,
                  uint8_t* __restrict__ dense_scales, float* __restrict__ topk_weights,
                  int32_t* __restrict__ topk_ids, int tokens, int tokens_per_cta, int hidden_size,
                  int experts, int topk, int renormalize) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");  // the rows may come from the kernel before
  const int first = blockIdx.x * tokens_per_cta;
  const int count = min(tokens_per_cta, tokens - first);
  const int groups = hidden_size / kScaleVec;
  const bool own_topk_warp = blockDim.x > kQuantThreads;
  if (quantized != nullptr && threadIdx.x < kQuantThreads) {
    const int row_chunks = hidden_size / 8;
    const int chunks = count * row_chunks;
    const int rounds = (chunks + kQuantThreads - 1) / kQuantThreads;
    // Four 16-byte loads per thread are in flight before the first one is used.
    constexpr int kUnroll = 4;
    const bool words = groups % 4 == 0 &&
                       (reinterpret_cast<uintptr_t>(logical_scales) & 3) == 0 &&
                       (reinterpret_cast<uintptr_t>(dense_scales) & 3) == 0;
    for (int it0 = 0; it0 < rounds; it0 += kUnroll) {
      uint4 raw[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int c = (it0 + u) * kQuantThreads + threadIdx.x;
        raw[u] = make_uint4(0u, 0u, 0u, 0u);
        if (c < chunks) {
          raw[u] = __ldg(reinterpret_cast<const uint4*>(hidden) + ((int64_t)first * row_chunks + c));
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int c = (it0 + u) * kQuantThreads + threadIdx.x;
        const bool valid = c < chunks;
        const int64_t gc = (int64_t)first * row_chunks + c;  // chunk index in the whole matrix
        float v[8];
        const uint32_t w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          v[2 * i] = __uint_as_float(w[i] << 16);
          v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        const uint32_t sbits = ue8m0_scale_bits(amax, 448.0f);
        const float inv = ue8m0_inverse(sbits);
        const uint32_t code = sbits >> 23;
        uint32_t word = code;
        word |= __shfl_down_sync(0xffffffffu, code, 4) << 8;
        word |= __shfl_down_sync(0xffffffffu, code, 8) << 16;
        word |= __shfl_down_sync(0xffffffffu, code, 12) << 24;
        if (valid) {
          reinterpret_cast<uint2*>(quantized)[gc] =
              make_uint2(e4m3x4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv),
                         e4m3x4(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv));
          const int token = first + c / row_chunks;
          const int g = (c % row_chunks) >> 2;
          if (words) {
            // 16 lanes = 4 groups of one row (a row holds a multiple of 16 chunks).
            if ((threadIdx.x & 15) == 0) {
              if (logical_scales != nullptr)
                *reinterpret_cast<uint32_t*>(logical_scales + (int64_t)token * groups + g) = word;
              if (dense_scales != nullptr)
                *reinterpret_cast<uint32_t*>(dense_scales +
                                             packed_scale_offset(token, g, groups)) = word;
            }
          } else if ((c & 3) == 0) {
            if (logical_scales != nullptr)
              logical_scales[(int64_t)token * groups + g] = static_cast<uint8_t>(code);
            if (dense_scales != nullptr)
              dense_scales[packed_scale_offset(token, g, groups)] = static_cast<uint8_t>(code);
          }
        }
      }
    }
  }
  if (topk_ids == nullptr) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (own_topk_warp) {
    if (warp == kQuantThreads / 32 && count > 0) {
      warp_softmax_topk(logits + (int64_t)first * experts, experts, topk, renormalize,
                        topk_weights + (int64_t)first * topk, topk_ids + (int64_t)first * topk, lane);
    }
    return;
  }
  for (int t = warp; t < count; t += blockDim.x >> 5) {
    const int token = first + t;
    warp_softmax_topk(logits + (int64_t)token * experts, experts, topk, renormalize,
                      topk_weights + (int64_t)token * topk, topk_ids + (int64_t)token * topk, lane);
  }
}

// ---------------------------------------------------------------- counts and offsets
__device__ __forceinline__ int local_expert(int64_t global, const int32_t* expert_map,
                                            int map_size, int local_experts) {
  if (global < 0) return -1;
  int local = static_cast<int>(global);
  if (expert_map != nullptr) {
    if (global >= map_size) return -1;
    local = expert_map[global];
  }
  return (local >= 0 && local < local_experts) ? local : -1;
}

// Single CTA: histogram of the routed expert ids, exclusive prefix sums.  With shared_rows > 0
// the last of the local_experts groups is the always-hit shared expert: no id selects it and
// it holds shared_rows rows (one per token), as in the reference's histogram
// (csrc/moe.cu:4486-4571).
template <class Id>
__global__ void __launch_bounds__(1024)
route_count_kernel(const Id* __restrict__ topk_ids, int64_t routes,
                   const int32_t* __restrict__ expert_map, int map_size, int local_experts,
                   int shared_rows, int64_t* __restrict__ expert_offsets,
                   int64_t* __restrict__ scale_offsets, int32_t* __restrict__ cursors) {
  __shared__ int counts[kMaxExperts];
  __shared__ int warp_sums[2][32];
  const int tid = threadIdx.x;
  for (int e = tid; e < kMaxExperts; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  const int routed_experts = local_experts - (shared_rows > 0 ? 1 : 0);
  for (int64_t i = tid; i < routes; i += blockDim.x) {
    const int e = local_expert(static_cast<int64_t>(topk_ids[i]), expert_map, map_size,
                               routed_experts);
    if (e >= 0) atomicAdd(&counts[e], 1);
  }
  if (shared_rows > 0 && tid == 0) counts[local_experts - 1] = shared_rows;  // no id reaches it
  __syncthreads();
  // Block-wide inclusive scans (one expert per thread) of counts and padded counts.
  const int c = tid < local_experts ? counts[tid] : 0;
  const int pc = (c + kAtomRows - 1) / kAtomRows * kAtomRows;
  int incl = c, pincl = pc;
  const int lane = tid & 31, warp = tid >> 5;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int a = __shfl_up_sync(0xffffffffu, incl, d);
    const int b = __shfl_up_sync(0xffffffffu, pincl, d);
    if (lane >= d) {
      incl += a;
      pincl += b;
    }
  }
  if (lane == 31) {
    warp_sums[0][warp] = incl;
    warp_sums[1][warp] = pincl;
  }
  __syncthreads();
  if (warp == 0) {
    int a = warp_sums[0][lane], b = warp_sums[1][lane];
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int ua = __shfl_up_sync(0xffffffffu, a, d);
      const int ub = __shfl_up_sync(0xffffffffu, b, d);
      if (lane >= d) {
        a += ua;
        b += ub;
      }
    }
    warp_sums[0][lane] = a;
    warp_sums[1][lane] = b;
  }
  __syncthreads();
  const int base = warp > 0 ? warp_sums[0][warp - 1] : 0;
  const int pbase = warp > 0 ? warp_sums[1][warp - 1] : 0;
  if (tid < local_experts) {
    expert_offsets[tid] = base + incl - c;
    scale_offsets[tid] = pbase + pincl - pc;
    if (cursors != nullptr) cursors[tid] = 0;
    if (tid == local_experts - 1) {
      expert_offsets[local_experts] = base + incl;
      scale_offsets[local_experts] = pbase + pincl;
    }
  }
}

// One warp per route: claim a row of its expert, copy the MXFP8 row and its scales.  Warps
// routes .. routes + shared_rows - 1 fill the trailing shared group: token t is its row t, and
// the inverse permutation (routed routes only) has no entry for it.
template <class Id>
__global__ void __launch_bounds__(256)
route_scatter_kernel(const uint8_t* __restrict__ activation,
                     const uint8_t* __restrict__ logical_scales, const Id* __restrict__ topk_ids,
                     int64_t routes, int topk, int hidden_size,
                     const int32_t* __restrict__ expert_map, int map_size, int local_experts,
                     int shared_rows, const int64_t* __restrict__ expert_offsets,
                     const int64_t* __restrict__ scale_offsets, int32_t* __restrict__ cursors,
                     uint8_t* __restrict__ permuted, uint8_t* __restrict__ grouped_scales,
                     int32_t* __restrict__ inverse_permutation,
                     int32_t* __restrict__ source_tokens) {
  // Lets a following GEMM start its prologue; it still waits for this grid to finish.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int lane = threadIdx.x & 31;
  const int64_t route = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (route >= routes + shared_rows) return;
  const bool shared = route >= routes;
  int e, local = 0;
  int64_t token;
  if (shared) {
    e = local_experts - 1;
    token = route - routes;
    local = static_cast<int>(token);
    if (lane == 0) atomicAdd(&cursors[e], 1);  // the cursors end as the group sizes
  } else {
    e = local_expert(static_cast<int64_t>(topk_ids[route]), expert_map, map_size,
                     local_experts - (shared_rows > 0 ? 1 : 0));
    if (e < 0) {
      if (lane == 0) inverse_permutation[route] = -1;  // dropped: the reducer skips it
      return;
    }
    if (lane == 0) local = atomicAdd(&cursors[e], 1);
    local = __shfl_sync(0xffffffffu, local, 0);
    token = route / topk;
  }
  const int64_t row = expert_offsets[e] + local;
  if (permuted != nullptr) {
    const uint4* src = reinterpret_cast<const uint4*>(activation + token * hidden_size);
    uint4* dst = reinterpret_cast<uint4*>(permuted + row * hidden_size);
    // four 16-byte loads in flight per lane before the first store
    const int chunks = hidden_size / 16;
    for (int i0 = lane; i0 < chunks; i0 += 128) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (i0 + 32 * u < chunks) v[u] = __ldg(src + i0 + 32 * u);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (i0 + 32 * u < chunks) dst[i0 + 32 * u] = v[u];
      }
    }
  }
  const int groups = hidden_size / kScaleVec;
  const int64_t srow = scale_offsets[e] + local;
  const uint8_t* scale_row = logical_scales + token * groups;
  if (groups % 4 == 0 && (reinterpret_cast<uintptr_t>(scale_row) & 3) == 0 &&
      (reinterpret_cast<uintptr_t>(grouped_scales) & 3) == 0) {
    // the four groups of a 128-K block are one word in both layouts
    for (int g = 4 * lane; g < groups; g += 128) {
      *reinterpret_cast<uint32_t*>(grouped_scales + packed_scale_offset(srow, g, groups)) =
          __ldg(reinterpret_cast<const uint32_t*>(scale_row + g));
    }
  } else {
    for (int g = lane; g < groups; g += 32) {
      grouped_scales[packed_scale_offset(srow, g, groups)] = __ldg(scale_row + g);
    }
  }
  if (lane == 0) {
    if (!shared) inverse_permutation[route] = static_cast<int32_t>(row);
    if (source_tokens != nullptr) source_tokens[row] = static_cast<int32_t>(token);
  }
}

// ---------------------------------------------------------------- small-batch fusion
// Decode-sized batches (tokens * topk <= 1024): one CTA does the whole front end of
// the layer - MXFP8 quantization of the rows, softmax top-k, expert histogram and
// offsets, row permutation - so that three kernel boundaries disappear.  The
// reference fuses the same steps with a cooperative launch (csrc/moe.cu:620-962).
constexpr int kFusedThreads = 1024;
constexpr int kFusedMaxRoutes = 1024;

__global__ void __launch_bounds__(kFusedThreads)
topk_quant_route_small_kernel(const __nv_bfloat16* __restrict__ hidden,
                              const __nv_bfloat16* __restrict__ logits,
                              uint8_t* __restrict__ quantized, uint8_t* __restrict__ logical_scales,
                              uint8_t* __restrict__ dense_scales, float* __restrict__ topk_weights,
                              int32_t* __restrict__ topk_ids, int tokens, int hidden_size,
                              int experts, int topk, int renormalize,
                              const int32_t* __restrict__ expert_map, int map_size,
                              int local_experts, int64_t* __restrict__ expert_offsets,
                              int64_t* __restrict__ scale_offsets, int32_t* __restrict__ cursors,
                              uint8_t* __restrict__ permuted, uint8_t* __restrict__ grouped_scales,
                              int32_t* __restrict__ inverse_permutation,
                              int32_t* __restrict__ source_tokens) {
  __shared__ int counts[kMaxExperts];
  __shared__ int starts[kMaxExperts];
  __shared__ int scale_starts[kMaxExperts];
  __shared__ int warp_sums[2][32];
  __shared__ int route_expert[kFusedMaxRoutes];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int groups = hidden_size / kScaleVec;
  for (int e = tid; e < kMaxExperts; e += kFusedThreads) counts[e] = 0;
  // ---- quantize every row (4 lanes per 32-value group)
  const int chunks = tokens * (hidden_size / 8);
  const int rounds = (chunks + kFusedThreads - 1) / kFusedThreads;
  for (int it = 0; it < rounds; ++it) {
    const int c = it * kFusedThreads + tid;
    const bool valid = c < chunks;
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (valid) {
      const uint4 raw = __ldg(reinterpret_cast<const uint4*>(hidden) + c);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
      }
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const uint32_t sbits = ue8m0_scale_bits(amax, 448.0f);
    const float inv = ue8m0_inverse(sbits);
    if (valid) {
      reinterpret_cast<uint2*>(quantized)[c] =
          make_uint2(e4m3x4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv),
                     e4m3x4(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv));
      if ((c & 3) == 0) {
        const int group = c >> 2;
        const int token = group / groups;
        const int g = group - token * groups;
        const uint8_t code = static_cast<uint8_t>(sbits >> 23);
        logical_scales[group] = code;
        if (dense_scales != nullptr) dense_scales[packed_scale_offset(token, g, groups)] = code;
      }
    }
  }
  // ---- top-k: one warp per token
  for (int token = warp; token < tokens; token += kFusedThreads / 32) {
    float weight;
    int id;
    warp_softmax_topk_regs<8>(logits + (int64_t)token * experts, experts, topk, renormalize, lane,
                              &weight, &id);
    if (lane < topk) {
      topk_weights[(int64_t)token * topk + lane] = weight;
      topk_ids[(int64_t)token * topk + lane] = id;
    }
  }
  __syncthreads();  // rows, scales and ids written by this CTA are visible to all its threads
  // ---- histogram of local experts
  const int routes = tokens * topk;
  for (int r = tid; r < routes; r += kFusedThreads) {
    const int e = local_expert(static_cast<int64_t>(topk_ids[r]), expert_map, map_size, local_experts);
    route_expert[r] = e;
    if (e >= 0) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  // ---- exclusive prefix sums of counts and 128-padded counts (one expert per thread)
  const int cnt = tid < local_experts ? counts[tid] : 0;
  const int pcnt = (cnt + kAtomRows - 1) / kAtomRows * kAtomRows;
  int incl = cnt, pincl = pcnt;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int a = __shfl_up_sync(0xffffffffu, incl, d);
    const int b = __shfl_up_sync(0xffffffffu, pincl, d);
    if (lane >= d) {
      incl += a;
      pincl += b;
    }
  }
  if (lane == 31) {
    warp_sums[0][warp] = incl;
    warp_sums[1][warp] = pincl;
  }
  __syncthreads();
  if (warp == 0) {
    int a = warp_sums[0][lane], b = warp_sums[1][lane];
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int ua = __shfl_up_sync(0xffffffffu, a, d);
      const int ub = __shfl_up_sync(0xffffffffu, b, d);
      if (lane >= d) {
        a += ua;
        b += ub;
      }
    }
    warp_sums[0][lane] = a;
    warp_sums[1][lane] = b;
  }
  __syncthreads();
  const int base = warp > 0 ? warp_sums[0][warp - 1] : 0;
  const int pbase = warp > 0 ? warp_sums[1][warp - 1] : 0;
  if (tid < local_experts) {
    starts[tid] = base + incl - cnt;
    scale_starts[tid] = pbase + pincl - pcnt;
    expert_offsets[tid] = base + incl - cnt;
    scale_offsets[tid] = pbase + pincl - pcnt;
    if (tid == local_experts - 1) {
      expert_offsets[local_experts] = base + incl;
      scale_offsets[local_experts] = pbase + pincl;
    }
    counts[tid] = 0;  // reused as the per-expert cursor
  }
  __syncthreads();
  // ---- permutation: one warp per route
  for (int route = warp; route < routes; route += kFusedThreads / 32) {
    const int e = route_expert[route];
    if (e < 0) {
      if (lane == 0) inverse_permutation[route] = -1;
      continue;
    }
    int local = 0;
    if (lane == 0) local = atomicAdd(&counts[e], 1);
    local = __shfl_sync(0xffffffffu, local, 0);
    const int row = starts[e] + local;
    const int token = route / topk;
    const uint4* src = reinterpret_cast<const uint4*>(quantized + (int64_t)token * hidden_size);
    uint4* dst = reinterpret_cast<uint4*>(permuted + (int64_t)row * hidden_size);
    for (int i = lane; i < hidden_size / 16; i += 32) dst[i] = src[i];
    const int srow = scale_starts[e] + local;
    for (int g = lane; g < groups; g += 32) {
      grouped_scales[packed_scale_offset(srow, g, groups)] = logical_scales[(int64_t)token * groups + g];
    }
    if (lane == 0) {
      inverse_permutation[route] = row;
      if (source_tokens != nullptr) source_tokens[row] = token;
    }
  }
  // The cursors end at the per-expert counts, as after the multi-kernel path.
  __syncthreads();
  if (cursors != nullptr && tid < local_experts) cursors[tid] = counts[tid];
}

// ---------------------------------------------------------------- SiLU * mul + MXFP8
// input [rows, 2I] (gate columns first), output [rows, I] E4M3 + scales.  Scale
// placement: logical [rows, I/32]; or packed with row -> scale row through
// expert/scale offsets (grouped) or identity (dense).
// One warp per row and 256 columns per pass (8 per lane): the row's expert is looked up once,
// in a shared-memory copy of expert_offsets, and four lanes' scale codes leave as one word
// when the layout allows it (a row of groups that is a multiple of four).
template <class T>
__global__ void __launch_bounds__(256)
silu_mul_quant_kernel(const T* __restrict__ input, uint8_t* __restrict__ output,
                      uint8_t* __restrict__ logical, uint8_t* __restrict__ packed, int64_t rows,
                      int inter, const int64_t* __restrict__ expert_offsets,
                      const int64_t* __restrict__ scale_offsets, int experts,
                      const uint16_t* __restrict__ silu_lut) {
  __shared__ int row_begin[kMaxExperts + 1];
  __shared__ int scale_begin[kMaxExperts + 1];
  const bool grouped = expert_offsets != nullptr;
  if (grouped) {
    for (int e = threadIdx.x; e <= experts; e += blockDim.x) {
      row_begin[e] = static_cast<int>(expert_offsets[e]);
      scale_begin[e] = static_cast<int>(scale_offsets[e]);
    }
    __syncthreads();
  }
  const int lane = threadIdx.x & 31;
  const int groups = inter / kScaleVec;
  const bool words = groups % 4 == 0 && (reinterpret_cast<uintptr_t>(logical) & 3) == 0 &&
                     (reinterpret_cast<uintptr_t>(packed) & 3) == 0;
  const int warps = static_cast<int>(gridDim.x) * (blockDim.x >> 5);
  const int first = static_cast<int>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  // A grouped buffer is sized for the worst case; only the rows the offsets cover are live
  // (an expert-parallel rank holds about 1 / world of the routes its buffer could take).
  const int64_t live = grouped ? min((int64_t)row_begin[experts], rows) : rows;
  for (int64_t row = first; row < live; row += warps) {
    int64_t srow = row;
    if (grouped) {
      int lo = 0, hi = experts;  // largest e with row_begin[e] <= row
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (row_begin[mid] <= row) lo = mid; else hi = mid;
      }
      srow = scale_begin[lo] + (row - row_begin[lo]);
    }
    const T* in_row = input + row * 2 * inter;
    for (int col0 = 0; col0 < inter; col0 += 256) {
      const int col = col0 + lane * 8;
      const bool valid = col < inter;
      float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (valid) {
        const uint4 graw = __ldg(reinterpret_cast<const uint4*>(in_row + col));
        const uint4 uraw = __ldg(reinterpret_cast<const uint4*>(in_row + inter + col));
        const T* gv = reinterpret_cast<const T*>(&graw);
        const T* uv = reinterpret_cast<const T*>(&uraw);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float g = round_bf16(to_float(gv[i]));
          const float u = round_bf16(to_float(uv[i]));
          const float sv = silu_bf16_lookup(silu_lut, g);  // = bf16(g / (1 + expf(-g)))
          v[i] = round_bf16(sv * u);
        }
      }
      float amax = 0.0f;
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      const uint32_t sbits = ue8m0_scale_bits(amax, 448.0f);
      const float inv = ue8m0_inverse(sbits);
      const uint32_t code = sbits >> 23;
      uint32_t word = code;
      word |= __shfl_down_sync(0xffffffffu, code, 4) << 8;
      word |= __shfl_down_sync(0xffffffffu, code, 8) << 16;
      word |= __shfl_down_sync(0xffffffffu, code, 12) << 24;
      if (valid) {
        *reinterpret_cast<uint2*>(output + row * inter + col) =
            make_uint2(e4m3x4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv),
                       e4m3x4(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv));
        const int g = col / kScaleVec;
        if (words) {
          if ((lane & 15) == 0) {
            if (logical != nullptr)
              *reinterpret_cast<uint32_t*>(logical + row * groups + g) = word;
            if (packed != nullptr)
              *reinterpret_cast<uint32_t*>(packed + packed_scale_offset(srow, g, groups)) = word;
          }
        } else if ((lane & 3) == 0) {
          if (logical != nullptr) logical[row * groups + g] = static_cast<uint8_t>(code);
          if (packed != nullptr)
            packed[packed_scale_offset(srow, g, groups)] = static_cast<uint8_t>(code);
        }
      }
    }
  }
}

// ---------------------------------------------------------------- weighted reduce
template <class T>
struct Pack8 {
  uint4 raw;
};

template <class T>
__device__ __forceinline__ void unpack8(const uint4& raw, float (&v)[8]) {
  const T* p = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = to_float(p[i]);
}

template <class T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <>
__device__ __forceinline__ __half from_float<__half>(float v) {
  return __float2half_rn(v);
}

// grid = (tokens, ceil(H / (8 * blockDim.x))); every thread owns 8 consecutive columns.
template <class T>
__global__ void __launch_bounds__(256)
moe_reduce_kernel(T* __restrict__ out, const T* __restrict__ routed,
                  const float* __restrict__ topk_weights,
                  const int32_t* __restrict__ inverse_permutation, const T* __restrict__ shared,
                  const void* __restrict__ shared_gate, int gate_dtype, int gate_stride,
                  int hidden_size, int topk, int64_t routed_rows) {
  const int token = blockIdx.x;
  const int col = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (col >= hidden_size) return;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (shared != nullptr) {
    float gate = 1.0f;
    if (shared_gate != nullptr) {
      const int64_t gi = (int64_t)token * gate_stride + (gate_stride - 1);
      float x;
      if (gate_dtype == kF32) x = static_cast<const float*>(shared_gate)[gi];
      else if (gate_dtype == kBF16) x = __bfloat162float(static_cast<const __nv_bfloat16*>(shared_gate)[gi]);
      else x = __half2float(static_cast<const __half*>(shared_gate)[gi]);
      gate = __fdiv_rn(1.0f, 1.0f + expf(-x));
    }
    float s[8];
    unpack8<T>(__ldg(reinterpret_cast<const uint4*>(shared + (int64_t)token * hidden_size + col)), s);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = gate * s[i];
  }
  for (int r = 0; r < topk; ++r) {
    const int32_t row = inverse_permutation[(int64_t)token * topk + r];
    if (row < 0 || row >= routed_rows) continue;
    const float w = topk_weights[(int64_t)token * topk + r];
    float v[8];
    unpack8<T>(__ldg(reinterpret_cast<const uint4*>(routed + (int64_t)row * hidden_size + col)), v);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(acc[i], __fmul_rn(w, v[i]));
  }
  uint4 packed;
  T* o = reinterpret_cast<T*>(&packed);
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = from_float<T>(acc[i]);
  *reinterpret_cast<uint4*>(out + (int64_t)token * hidden_size + col) = packed;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

int moe_topk_quant(const void* hidden, const void* logits, int64_t tokens, int hidden_size,
                   int experts, int topk, int renormalize, uint8_t* quantized,
                   uint8_t* logical_scales, uint8_t* dense_scales, float* topk_weights,
                   int32_t* topk_ids, cudaStream_t stream) {
  MX_REQUIRE(tokens > 0 && tokens <= INT32_MAX, "tokens must be positive");
  MX_REQUIRE(hidden_size > 0 && hidden_size % kScaleVec == 0, "hidden size must be a multiple of 32");
  MX_REQUIRE(quantized == nullptr || (hidden != nullptr && aligned16(hidden)),
             "hidden must be a 16-byte aligned device pointer");
  if (topk_ids != nullptr) {
    MX_REQUIRE(logits != nullptr && topk_weights != nullptr, "logits/topk_weights must not be null");
    MX_REQUIRE(experts > 0 && experts <= kMaxExperts, "experts must be in [1, %d]", kMaxExperts);
    MX_REQUIRE(topk > 0 && topk <= kMaxTopk && topk <= experts, "topk must be in [1, %d]", kMaxTopk);
  }
  // Up to one CTA per SM: one token per CTA, the top-k in a warp of its own beside the
  // quantization.  Above: eight tokens per CTA (measured at 4096 tokens: 16.0 us against 38.3 us
  // with one token per CTA, whose 4096 small CTAs cost more to launch than they save).
  const int tokens_per_cta = tokens <= 148 ? 1 : 8;
  const unsigned grid = (unsigned)((tokens + tokens_per_cta - 1) / tokens_per_cta);
  // One token per CTA: the top-k gets a warp of its own beside the 256 quantizing threads.
  const bool own_topk_warp = tokens_per_cta == 1 && topk_ids != nullptr && quantized != nullptr;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(grid);
  config.blockDim = dim3(own_topk_warp ? kQuantThreads + 32 : kQuantThreads);
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = grid <= 148 ? 1 : 0;  // the kernel opens with a dependency wait
  MX_CUDA(cudaLaunchKernelEx(&config, topk_quant_kernel, static_cast<const __nv_bfloat16*>(hidden),
                             static_cast<const __nv_bfloat16*>(logits), quantized, logical_scales,
                             dense_scales, topk_weights, topk_ids, (int)tokens, tokens_per_cta,
                             hidden_size, experts, topk, renormalize));
  return kOk;
}

int moe_route(const uint8_t* activation, const uint8_t* logical_scales, const void* topk_ids,
              int ids_are_int64, int64_t tokens, int topk, int hidden_size,
              const int32_t* expert_map, int map_size, int local_experts, int include_shared,
              int64_t* expert_offsets, int64_t* scale_offsets, int32_t* cursors,
              uint8_t* permuted, uint8_t* grouped_scales, int32_t* inverse_permutation,
              int32_t* source_tokens, cudaStream_t stream) {
  MX_REQUIRE(tokens > 0 && topk > 0, "tokens and topk must be positive");
  MX_REQUIRE(local_experts > (include_shared ? 1 : 0) && local_experts <= kMaxExperts,
             "local_experts must be in [1, %d] and count one trailing shared expert when "
             "include_shared is set",
             kMaxExperts);
  MX_REQUIRE(hidden_size > 0 && hidden_size % kScaleVec == 0 && hidden_size % 16 == 0,
             "hidden size must be a multiple of 32");
  MX_REQUIRE(topk_ids && expert_offsets && scale_offsets && cursors && grouped_scales &&
                 inverse_permutation && logical_scales,
             "routing buffers must not be null");
  MX_REQUIRE(permuted == nullptr || (activation != nullptr && aligned16(activation) && aligned16(permuted)),
             "activation / permuted rows must be 16-byte aligned");
  const int64_t routes = tokens * topk;
  MX_REQUIRE(routes + tokens <= INT32_MAX, "routed and shared rows must fit int32");
  const int shared_rows = include_shared ? static_cast<int>(tokens) : 0;
  const unsigned scatter_grid = (unsigned)((routes + shared_rows + 7) / 8);
  if (ids_are_int64) {
    const int64_t* ids = static_cast<const int64_t*>(topk_ids);
    route_count_kernel<int64_t><<<1, 1024, 0, stream>>>(ids, routes, expert_map, map_size,
                                                        local_experts, shared_rows, expert_offsets,
                                                        scale_offsets, cursors);
    route_scatter_kernel<int64_t><<<scatter_grid, 256, 0, stream>>>(
        activation, logical_scales, ids, routes, topk, hidden_size, expert_map, map_size,
        local_experts, shared_rows, expert_offsets, scale_offsets, cursors, permuted,
        grouped_scales, inverse_permutation, source_tokens);
  } else {
    const int32_t* ids = static_cast<const int32_t*>(topk_ids);
    route_count_kernel<int32_t><<<1, 1024, 0, stream>>>(ids, routes, expert_map, map_size,
                                                        local_experts, shared_rows, expert_offsets,
                                                        scale_offsets, cursors);
    route_scatter_kernel<int32_t><<<scatter_grid, 256, 0, stream>>>(
        activation, logical_scales, ids, routes, topk, hidden_size, expert_map, map_size,
        local_experts, shared_rows, expert_offsets, scale_offsets, cursors, permuted,
        grouped_scales, inverse_permutation, source_tokens);
  }
  MX_CUDA(cudaGetLastError());
  return kOk;
}

int moe_topk_quant_route(const void* hidden, const void* logits, int64_t tokens, int hidden_size,
                         int experts, int topk, int renormalize, uint8_t* quantized,
                         uint8_t* logical_scales, uint8_t* dense_scales, float* topk_weights,
                         int32_t* topk_ids, const int32_t* expert_map, int map_size,
                         int local_experts, int64_t* expert_offsets, int64_t* scale_offsets,
                         int32_t* cursors, uint8_t* permuted, uint8_t* grouped_scales,
                         int32_t* inverse_permutation, int32_t* source_tokens,
                         cudaStream_t stream) {
  MX_REQUIRE(tokens > 0 && topk > 0, "tokens and topk must be positive");
  // One CTA copies every routed row, so the fusion only pays for a handful of tokens.
  // (the single-CTA kernel keeps eight logits per lane in registers: up to 256 experts)
  const bool small = tokens * topk <= kFusedMaxRoutes && tokens <= 8 && experts <= 256;
  if (!small) {
    if (int rc = moe_topk_quant(hidden, logits, tokens, hidden_size, experts, topk, renormalize,
                                quantized, logical_scales, dense_scales, topk_weights, topk_ids,
                                stream))
      return rc;
    return moe_route(quantized, logical_scales, topk_ids, 0, tokens, topk, hidden_size, expert_map,
                     map_size, local_experts, /*include_shared=*/0, expert_offsets, scale_offsets,
                     cursors, permuted, grouped_scales, inverse_permutation, source_tokens, stream);
  }
  MX_REQUIRE(hidden && logits && quantized && logical_scales && topk_weights && topk_ids &&
                 expert_offsets && scale_offsets && permuted && grouped_scales &&
                 inverse_permutation,
             "routing buffers must not be null");
  MX_REQUIRE(hidden_size > 0 && hidden_size % kScaleVec == 0, "hidden size must be a multiple of 32");
  MX_REQUIRE(experts > 0 && experts <= kMaxExperts && local_experts > 0 &&
                 local_experts <= kMaxExperts,
             "experts must be in [1, %d]", kMaxExperts);
  MX_REQUIRE(topk <= kMaxTopk && topk <= experts, "topk must be in [1, %d]", kMaxTopk);
  MX_REQUIRE(aligned16(hidden) && aligned16(quantized) && aligned16(permuted),
             "row buffers must be 16-byte aligned");
  topk_quant_route_small_kernel<<<1, kFusedThreads, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(hidden), static_cast<const __nv_bfloat16*>(logits),
      quantized, logical_scales, dense_scales, topk_weights, topk_ids, (int)tokens, hidden_size,
      experts, topk, renormalize, expert_map, map_size, local_experts, expert_offsets,
      scale_offsets, cursors, permuted, grouped_scales, inverse_permutation, source_tokens);
  MX_CUDA(cudaGetLastError());
  return kOk;
}

int silu_mul_quant(const void* input, int dtype, int64_t rows, int inter, uint8_t* output,
                   uint8_t* logical, uint8_t* packed, const int64_t* expert_offsets,
                   const int64_t* scale_offsets, int experts, cudaStream_t stream) {
  MX_REQUIRE(input != nullptr && output != nullptr, "pointers must not be null");
  MX_REQUIRE(dtype == kF16 || dtype == kBF16, "input must be float16 or bfloat16");
  MX_REQUIRE(rows > 0 && inter > 0 && inter % kScaleVec == 0,
             "input must be [M, 2K] with K divisible by 32");
  MX_REQUIRE(aligned16(input) && (reinterpret_cast<uintptr_t>(output) & 7) == 0,
             "input/output must be 16/8-byte aligned");
  MX_REQUIRE(logical != nullptr || packed != nullptr, "one scale output is required");
  MX_REQUIRE((expert_offsets == nullptr) == (scale_offsets == nullptr),
             "expert_offsets and scale_offsets go together");
  MX_REQUIRE(expert_offsets == nullptr || (experts > 0 && experts <= kMaxExperts),
             "experts must be in [1, %d]", kMaxExperts);
  const uint16_t* silu_lut = nullptr;
  if (int rc = silu_table(stream, &silu_lut)) return rc;
  int64_t blocks = (rows + 7) / 8;  // one warp per row, eight warps per CTA
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (dtype == kBF16) {
    silu_mul_quant_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(input), output, logical, packed, rows, inter,
        expert_offsets, scale_offsets, experts, silu_lut);
  } else {
    silu_mul_quant_kernel<__half><<<(unsigned)blocks, 256, 0, stream>>>(
        static_cast<const __half*>(input), output, logical, packed, rows, inter, expert_offsets,
        scale_offsets, experts, silu_lut);
  }
  MX_CUDA(cudaGetLastError());
  return kOk;
}

int moe_reduce(void* out, const void* routed, int dtype, const float* topk_weights,
               const int32_t* inverse_permutation, const void* shared, const void* shared_gate,
               int gate_dtype, int gate_stride, int64_t tokens, int hidden_size, int topk,
               int64_t routed_rows, cudaStream_t stream) {
  MX_REQUIRE(out && routed && topk_weights && inverse_permutation, "pointers must not be null");
  MX_REQUIRE(dtype == kF16 || dtype == kBF16, "routed_output must be float16 or bfloat16");
  MX_REQUIRE(tokens > 0 && topk > 0 && hidden_size > 0 && hidden_size % 8 == 0,
             "hidden size must be a multiple of 8");
  MX_REQUIRE(aligned16(out) && aligned16(routed) && (shared == nullptr || aligned16(shared)),
             "row buffers must be 16-byte aligned");
  MX_REQUIRE(shared_gate == nullptr || shared != nullptr, "shared_gate requires shared_output");
  MX_REQUIRE(gate_stride >= 1, "gate stride must be positive");
  const int threads = hidden_size / 8 < 256 ? ((hidden_size / 8 + 31) / 32 * 32) : 256;
  const dim3 grid((unsigned)tokens, (unsigned)((hidden_size / 8 + threads - 1) / threads));
  if (dtype == kBF16) {
    moe_reduce_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(
        static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(routed), topk_weights,
        inverse_permutation, static_cast<const __nv_bfloat16*>(shared), shared_gate, gate_dtype,
        gate_stride, hidden_size, topk, routed_rows);
  } else {
    moe_reduce_kernel<__half><<<grid, threads, 0, stream>>>(
        static_cast<__half*>(out), static_cast<const __half*>(routed), topk_weights,
        inverse_permutation, static_cast<const __half*>(shared), shared_gate, gate_dtype,
        gate_stride, hidden_size, topk, routed_rows);
  }
  MX_CUDA(cudaGetLastError());
  return kOk;
}

}  // namespace mx
