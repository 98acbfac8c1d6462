// Softmax top-k of one token by one warp, shared by the routing kernels.
#pragma once

#include <cuda_bf16.h>

#include <cstdint>

namespace mx {

// Order-preserving map of a float onto an unsigned integer (and back), for warp reductions.
__device__ __forceinline__ uint32_t ordered_bits(float v) {
  const uint32_t u = __float_as_uint(v);
  return (u & 0x80000000u) != 0u ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float from_ordered_bits(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) != 0u ? (k & 0x7fffffffu) : ~k);
}

// FP32 softmax of one token's BF16 logits and k rounds of arg-max (ties to the smaller id),
// by one full warp; lane l owns experts l, l + 32, ...  On return lane r < topk holds the
// r-th selected expert and its weight (renormalised over the selection if asked); the
// reference's rule, csrc/moe.cu:440-511: probabilities in FP32 with the maximum subtracted,
// non-finite probabilities count as 0, a selected probability is replaced by -10000.
template <int kPerLane>
__device__ __forceinline__ void warp_softmax_topk_regs(const __nv_bfloat16* __restrict__ logits_row,
                                                       int experts, int topk, int renormalize,
                                                       int lane, float* weight_out, int* id_out) {
  float p[kPerLane];
  float vmax = -INFINITY;
  const int per_lane = (experts + 31) / 32;
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    p[i] = -INFINITY;
    const int e = lane + 32 * i;
    if (i < per_lane && e < experts) {
      p[i] = __bfloat162float(logits_row[e]);
      vmax = fmaxf(vmax, p[i]);
    }
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, d));
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    const int e = lane + 32 * i;
    if (i < per_lane && e < experts) {
      p[i] = expf(p[i] - vmax);
      sum += p[i];
    } else {
      p[i] = -1.0f;  // never selected
    }
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
  const float inv_sum = 1.0f / sum;
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    if (p[i] >= 0.0f) {
      float q = p[i] * inv_sum;
      if (!isfinite(q)) q = 0.0f;
      p[i] = q;
    }
  }
  float weight_sum = 0.0f;
  float my_weight = 0.0f;  // lane r keeps the r-th selected weight
  int my_id = 0;
  // Every lane keeps the best of its own values; a round is then two warp reductions (the
  // largest value, then the smallest id among the lanes that hold it) and a rescan in the one
  // lane that lost its value.
  float best = -2.0f;
  int best_id = 0x7fffffff;
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    if (p[i] > best) {  // ascending ids inside a lane: first maximum is the smallest id
      best = p[i];
      best_id = lane + 32 * i;
    }
  }
  for (int r = 0; r < topk; ++r) {
    const uint32_t top = __reduce_max_sync(0xffffffffu, ordered_bits(best));
    const int winner = __reduce_min_sync(0xffffffffu, ordered_bits(best) == top ? best_id : 0x7fffffff);
    const float value = from_ordered_bits(top);
    if (lane == (winner & 31)) {
      best = -2.0f;
      best_id = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < kPerLane; ++i) {
        if (lane + 32 * i == winner) p[i] = -10000.0f;
        if (p[i] > best) {
          best = p[i];
          best_id = lane + 32 * i;
        }
      }
    }
    if (lane == r) {
      my_weight = value;
      my_id = winner;
    }
    weight_sum += value;
  }
  if (renormalize) my_weight = weight_sum > 0.0f ? my_weight / weight_sum : 0.0f;
  *weight_out = my_weight;
  *id_out = my_id;
}

// Up to 256 experts need 8 values per lane; the general case (up to 1024) 32.
__device__ __forceinline__ void warp_softmax_topk_any(const __nv_bfloat16* __restrict__ logits_row,
                                                      int experts, int topk, int renormalize,
                                                      int lane, float* weight_out, int* id_out) {
  if (experts <= 256) {
    warp_softmax_topk_regs<8>(logits_row, experts, topk, renormalize, lane, weight_out, id_out);
  } else {
    warp_softmax_topk_regs<32>(logits_row, experts, topk, renormalize, lane, weight_out, id_out);
  }
}

}  // namespace mx
