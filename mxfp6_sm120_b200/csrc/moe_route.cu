// Decode-batch MoE without permutation: one single-row W6A8 GEMM per route.
//
// The reference serves batches of up to eight tokens with "array" and split-K kernels that
// read each route's activation row and its expert's weights in place (route r = token *
// lanes + lane; the expert is topk_ids[token, lane], or the always-on shared expert for the
// lane after the last routed one): route_w6a8_kernel / route_w6a8_silu_mxfp8_kernel /
// route_w6a8_reduce_kernel and the cooperative qwen35_w1_splitk / qwen35_w2_splitk kernels
// (csrc/moe.cu:1306-1481, 1882-2286, 2689-2960, 2977-3270, 3272-3629; host entry points
// :6713-7393).  Here that is three tcgen05 kernels built like the weight-streaming GEMM
// (gemm_stream.cu): under half an SM's shared memory per CTA, programmatic launch, bounded
// waits, cluster push reductions through distributed shared memory.
//
//   route_gemm_kernel<store | swiglu>   one (route, 128-feature tile) per cluster; the CTAs
//       of the cluster split K and push their FP32 partial row to rank 0.  Store mode
//       writes the BF16/FP16 row; SwiGLU mode reads the gate tile and the matching up tile
//       and writes MXFP8 codes with logical UE8M0 scales (the reference's five BF16
//       roundings, csrc/moe.cu:2226-2235).
//   route_w2_reduce_kernel               one (token, 128-feature tile) per cluster; the
//       CTAs split the token's lanes, every lane accumulates into tensor-memory columns of
//       its own, every weighted term w_l * routed_l (routed_l rounded to the output type)
//       is pushed to rank 0, and rank 0 adds sigmoid(gate) * shared and the terms one by one
//       in lane order (csrc/moe.cu:3228-3265, 7972-7988): the bytes equal those of the
//       store kernel followed by moe_reduce_array_kernel, and no routed output reaches
//       global memory.
//
//   route_w1_front_kernel                the W1 (SwiGLU) kernel of the decode schedule with the
//       layer's front end inside: every CTA runs the softmax top-k of its token and quantizes
//       its K slice of the token's BF16 row into the shared-memory operand, so the schedule is
//       two launches (moe_decode_layer) and depends on nothing but the layer's inputs.
//
// A route's activation is one row.  It is MMA operand B with N = 16 (row 0 real, rows 1..15
// whatever follows it in memory or zero fill: their accumulator columns are never read).
// Its scales come as LOGICAL bytes [rows, K/32] (the reference's array ops take them so):
// four consecutive bytes are the four scale groups of a 128-K block, exactly the first
// word of the 512-byte atom that tcgen05.cp moves to tensor memory, so a warp writes one
// word per block into shared memory, 16 bytes apart, and the copy of block j starts at
// byte 16 * j: what it reads beyond the first word belongs to other blocks and lands in
// the scale rows of tokens that do not exist.
#include "gemm.cuh"
#include "ptx.cuh"
#include "topk.cuh"
#include "wait.cuh"

#include <cuda.h>
#include <cuda_fp8.h>

#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <unordered_map>

namespace mx {

int make_tensor_map_2d(CUtensorMap* out, int type, const void* base, uint64_t inner, uint64_t rows,
                       uint64_t stride, uint32_t box_rows);

namespace {

constexpr int kTileF = 128;    // output features per tile (MMA M)
constexpr int kTileK = 128;    // K values per pipeline stage
constexpr int kMmaK = 32;      // K values per tcgen05.mma
constexpr int kRows = 16;      // MMA N: the route's row and fifteen rows of padding
constexpr int kThreads = 192;  // warp 0 TMA, warp 1 MMA, warps 2..5 epilogue
constexpr uint32_t kWTileBytes = kTileF * kTileK;
constexpr uint32_t kWTileTxBytes = kWTileBytes / 4 * 3;  // 16U6_ALIGN16B counts packed bytes
constexpr uint32_t kATileBytes = kRows * kTileK;
constexpr uint32_t kAtomBytes = 512;
constexpr int kMaxKBlocks = 64;   // K <= 8192
constexpr int kMaxCluster = 4;      // K split of the route GEMM (its reduction buffer holds four ranks)
constexpr int kMaxLaneCluster = 5;  // lane split of the reduce kernel: two lanes per CTA at most
constexpr int kMaxLanes = 9;      // routes of one token in the reduce kernel (top-8 + shared)

enum RouteMode : int { kRouteStore = 0, kRouteSwiglu = 1 };

struct RouteArgs {
  const uint8_t* w_scales;         // packed scales of the expert stack
  const uint8_t* shared_w_scales;  // packed scales of a separate shared expert, or null
  const uint8_t* act_scales;       // logical [act_rows, K / 32]
  const void* topk_ids;            // [tokens, topk] int32 or int64
  const float* topk_weights;       // reduce kernel: [tokens, topk]
  const void* shared_gate;         // reduce kernel: one logit per token (last column of a row)
  const void* shared_output;       // reduce kernel: precomputed shared rows [tokens, n], or null
  void* out;
  uint8_t* out_scales;             // SwiGLU mode: logical [routes, n / 32]
  int* status;
  const uint16_t* silu_lut;
  int ids_are_int64;
  int gate_dtype;
  int gate_stride;
  int tokens;
  int topk;
  int lanes;            // routes per token that this launch computes (topk, or topk + 1)
  int act_per_route;    // 1: activation rows = tokens * lanes; 0: one row per token
  int num_experts;      // experts in the stack
  int separate_shared;  // 1: the shared lane reads the second tensor map
  int n;                // output features per route (SwiGLU: the intermediate size)
  int w_rows;           // weight rows per expert (SwiGLU: 2 * n)
  int k_blocks;
  int tiles;            // n / 128
  int cluster;          // CTAs per cluster (K split, or lane split in the reduce kernel)
  int out_dtype;
  int routing_ready;    // reduce kernel: ids were complete before the preceding kernel's dependents started
  // front kernel / reduce kernel with the routing done inside the CTA
  const void* hidden;      // BF16 [tokens, K]: quantized by the front kernel itself
  const void* logits;      // BF16 [tokens, logit_experts]: softmax top-k per CTA
  int32_t* ids_out;        // front kernel: [tokens, topk], written once per token
  float* weights_out;      // front kernel: [tokens, topk]
  int logit_experts;
  int renormalize;
};

__device__ __forceinline__ int read_expert(const RouteArgs& a, int token, int lane) {
  if (lane >= a.topk) return a.separate_shared != 0 ? -2 : a.num_experts - 1;  // shared lane
  const int64_t at = (int64_t)token * a.topk + lane;
  const int64_t id = a.ids_are_int64 != 0 ? static_cast<const int64_t*>(a.topk_ids)[at]
                                           : static_cast<const int32_t*>(a.topk_ids)[at];
  return (id < 0 || id >= a.num_experts) ? -1 : (int)id;
}

template <int MODE>
struct RCfg {
  static constexpr int kWTiles = MODE == kRouteSwiglu ? 2 : 1;
  static constexpr uint32_t kStageBytes = kWTiles * (kWTileBytes + kAtomBytes) + kATileBytes;
  // activation scale words, 16 bytes apart, plus the tail the last copy reads
  static constexpr uint32_t kSfbBytes = kMaxKBlocks * 16 + kAtomBytes;
  // partial rows pushed to rank 0: [rank][warp][tile][32 floats]
  static constexpr uint32_t kRedBytes = kMaxCluster * 4 * kWTiles * 128;
  static constexpr size_t kBudget = 233472 / 2 - 1024;
  static constexpr int kStages = (int)((kBudget - 2048 - kSfbBytes - kRedBytes) / kStageBytes);
  static_assert(kStages >= 3, "the ring needs a few stages");
  static constexpr size_t kSmemBytes =
      1024 + (size_t)kStages * kStageBytes + kSfbBytes + kRedBytes + 1024;
  static_assert(kSmemBytes <= kBudget, "two CTAs must fit one SM");
  static constexpr int kSfSets = 4;
  static constexpr int kSfSetCols = 4 * kWTiles + 4;
  static constexpr int kSfCol = kWTiles * kRows;
  static constexpr int kTmemCols = 128;
  static_assert(kSfCol + kSfSets * kSfSetCols <= kTmemCols, "tensor memory layout");
};

// ------------------------------------------------------------------------------------
// One (route, feature tile) per cluster; K split over the cluster's CTAs.
template <int MODE>
__global__ void __launch_bounds__(kThreads, 2)
route_gemm_kernel(const __grid_constant__ CUtensorMap tm_w,
                  const __grid_constant__ CUtensorMap tm_shared,
                  const __grid_constant__ CUtensorMap tm_a, const RouteArgs args) {
  using C = RCfg<MODE>;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* w_tiles = smem;                                                   // [S][T][16 KB]
  uint8_t* a_tiles = w_tiles + (size_t)C::kStages * C::kWTiles * kWTileBytes;  // [S][2 KB]
  uint8_t* sfa_tiles = a_tiles + (size_t)C::kStages * kATileBytes;           // [S][T][512]
  uint8_t* sfb = sfa_tiles + (size_t)C::kStages * C::kWTiles * kAtomBytes;
  float* red = reinterpret_cast<float*>(sfb + C::kSfbBytes);
  uint8_t* fixed = reinterpret_cast<uint8_t*>(red) + C::kRedBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(fixed);  // full[S], empty[S], tfull, sfb, red
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(fixed + 8 * (2 * C::kStages + 3));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t full0 = ptx::smem_u32(bars);
  const uint32_t empty0 = full0 + 8 * C::kStages;
  const uint32_t tfull = empty0 + 8 * C::kStages;
  const uint32_t sfb_bar = tfull + 8;
  const uint32_t red_full = sfb_bar + 8;

  const int ck = args.cluster;
  const int rank = ck > 1 ? (int)ptx::cluster_ctarank() : 0;
  const int unit = (int)blockIdx.x / ck;
  const int route = unit / args.tiles;
  const int tile = unit - route * args.tiles;
  const int token = route / args.lanes;
  const int route_lane = route - token * args.lanes;
  const int src_row = args.act_per_route != 0 ? route : token;
  const int kb0 = (rank * args.k_blocks) / ck;
  const int kb1 = ((rank + 1) * args.k_blocks) / ck;
  const uint32_t tx_stage = C::kWTiles * (kWTileTxBytes + kAtomBytes) + kATileBytes;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < C::kStages; ++s) {
      ptx::mbar_init(full0 + 8 * s, 1);
      ptx::mbar_init(empty0 + 8 * s, 1);
    }
    ptx::mbar_init(tfull, 1);
    ptx::mbar_init(sfb_bar, 1);
    ptx::mbar_init(red_full, 1);
    if (ck > 1 && rank == 0) {
      // every rank sends each of its four epilogue warps' kWTiles x 128 bytes
      ptx::mbar_arrive_expect_tx(red_full, (uint32_t)(ck * 4 * C::kWTiles * 128));
    }
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tm_w);
    ptx::prefetch_tensormap(&tm_a);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), C::kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (ck > 1) ptx::cluster_sync_all();
  bool cluster_arrived = false;

  // Expert ids, activations and their scales come from the kernel before this one.  The
  // kernel after this one starts only now, so that it may read that routing data before
  // its own dependency wait (route_w2_reduce_kernel fetches its weights that early).
  ptx::grid_dependency_wait();
  ptx::grid_launch_dependents();
  const int expert = read_expert(args, token, route_lane);  // -1: no such expert, -2: separate shared
  const bool live = expert != -1;
  const CUtensorMap* wmap = expert == -2 ? &tm_shared : &tm_w;
  const uint8_t* wsc = expert == -2 ? args.shared_w_scales : args.w_scales;
  const int w_row0 = (expert < 0 ? 0 : expert) * args.w_rows + tile * kTileF;  // gate rows (or the only tile)

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    int stage = 0;
    uint32_t phase = 0;
    bool ok = live;
    for (int kb = kb0; ok && kb < kb1; ++kb) {
      ok = __all_sync(0xffffffffu, bounded_wait(empty0 + 8 * stage, phase ^ 1u, abort_flag,
                                                args.status, 121));
      if (!ok) break;
      if (ptx::elect_one()) {
        const uint32_t bar = full0 + 8 * stage;
        ptx::mbar_arrive_expect_tx(bar, tx_stage);
#pragma unroll
        for (int t = 0; t < C::kWTiles; ++t) {
          const int w_row = w_row0 + t * args.n;  // tile 1: the up rows, n rows further down
          ptx::tma_load_2d(
              ptx::smem_u32(w_tiles + (size_t)(stage * C::kWTiles + t) * kWTileBytes), wmap,
              kb * kTileK, w_row, bar);
          ptx::bulk_load(ptx::smem_u32(sfa_tiles + (size_t)(stage * C::kWTiles + t) * kAtomBytes),
                         wsc + ((int64_t)(w_row / kAtomRows) * args.k_blocks + kb) * kAtomBytes,
                         kAtomBytes, bar);
        }
        ptx::tma_load_2d(ptx::smem_u32(a_tiles + (size_t)stage * kATileBytes), &tm_a, kb * kTileK,
                         src_row, bar);
      }
      __syncwarp();
      if (++stage == C::kStages) {
        stage = 0;
        phase ^= 1u;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    constexpr uint32_t kIdesc = (4u << 7) | (0u << 10) | ((uint32_t)(kRows >> 3) << 17) | (1u << 23) |
                                ((uint32_t)(kTileF >> 4) << 24);
    int stage = 0;
    uint32_t phase = 0;
    uint32_t sf_set = 0;
    bool ok = live && __all_sync(0xffffffffu, bounded_wait(sfb_bar, 0u, abort_flag, args.status, 122));
    for (int kb = kb0; ok && kb < kb1; ++kb) {
      ok = __all_sync(0xffffffffu,
                      bounded_wait(full0 + 8 * stage, phase, abort_flag, args.status, 123));
      if (!ok) break;
      ptx::tc_fence_after();
      if (ptx::elect_one()) {
        const uint32_t sfa_t = tmem_base + C::kSfCol + sf_set * C::kSfSetCols;
        const uint32_t sfb_t = sfa_t + 4 * C::kWTiles;
#pragma unroll
        for (int t = 0; t < C::kWTiles; ++t) {
          ptx::tc_cp_32x128b_warpx4(sfa_t + 4 * t, ptx::smem_desc_scale_atom(ptx::smem_u32(
                                                       sfa_tiles + (size_t)(stage * C::kWTiles + t) * kAtomBytes)));
        }
        ptx::tc_cp_32x128b_warpx4(sfb_t, ptx::smem_desc_scale_atom(ptx::smem_u32(sfb + (kb - kb0) * 16)));
        const uint64_t b_desc = ptx::smem_desc_sw128(ptx::smem_u32(a_tiles + (size_t)stage * kATileBytes));
#pragma unroll
        for (int t = 0; t < C::kWTiles; ++t) {
          const uint64_t a_desc = ptx::smem_desc_sw128(
              ptx::smem_u32(w_tiles + (size_t)(stage * C::kWTiles + t) * kWTileBytes));
#pragma unroll
          for (int ks = 0; ks < kTileK / kMmaK; ++ks) {
            const uint32_t idesc = kIdesc | ((uint32_t)ks << 4) | ((uint32_t)ks << 29);
            ptx::tc_mma_mxf8f6f4(tmem_base + t * kRows, a_desc + 2 * ks, b_desc + 2 * ks, idesc,
                                 sfa_t + 4 * t, sfb_t, (kb > kb0 || ks > 0) ? 1u : 0u);
          }
        }
        ptx::tc_commit(empty0 + 8 * stage);
      }
      __syncwarp();
      sf_set = (sf_set + 1u) % C::kSfSets;
      if (++stage == C::kStages) {
        stage = 0;
        phase ^= 1u;
      }
    }
    if (ok) {
      if (ptx::elect_one()) ptx::tc_commit(tfull);
      __syncwarp();
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int quarter = warp & 3;
    if (warp == 2 && live) {
      // This CTA's share of the route's activation scales, one word per 128-K block.
      const uint32_t* words = reinterpret_cast<const uint32_t*>(
          args.act_scales + (int64_t)src_row * (args.k_blocks * 4));
      for (int j = lane; j < kb1 - kb0; j += 32) {
        *reinterpret_cast<uint32_t*>(sfb + j * 16) = words[kb0 + j];
      }
      ptx::fence_proxy_async();  // tcgen05.cp reads them through the async proxy
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(sfb_bar);
    }
    bool ok = live && bounded_wait(tfull, 0u, abort_flag, args.status, 124);
    float acc[C::kWTiles];
#pragma unroll
    for (int t = 0; t < C::kWTiles; ++t) acc[t] = 0.0f;
    if (ok) {
      ptx::tc_fence_after();
      const uint32_t t_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll
      for (int t = 0; t < C::kWTiles; ++t) {
        uint32_t r[16];
        ptx::tmem_ld_x16(t_addr + t * kRows, r);
        ptx::tmem_ld_wait();
        acc[t] = __uint_as_float(r[0]);  // column 0: the route's row
      }
    }
    if (ck > 1) {
      // Partial row -> rank 0, which adds the ranks in order.  Layout [rank][warp][tile][32].
      float* send = reinterpret_cast<float*>(w_tiles) + (quarter * C::kWTiles) * 32;  // ring is idle
      if (ok) {
#pragma unroll
        for (int t = 0; t < C::kWTiles; ++t) send[t * 32 + lane] = acc[t];
        ptx::fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          ptx::bulk_copy_to_peer(
              ptx::mapa(ptx::smem_u32(red + ((rank * 4 + quarter) * C::kWTiles) * 32), 0u),
              ptx::smem_u32(send), (uint32_t)(C::kWTiles * 128), ptx::mapa(red_full, 0u));
        }
      }
      if (rank == 0 && ok) {
        ok = bounded_wait_cluster(red_full, 0u, abort_flag, args.status, 126);
        if (ok) {
#pragma unroll
          for (int t = 0; t < C::kWTiles; ++t) {
            float sum = 0.0f;
            for (int src = 0; src < ck; ++src) sum += red[((src * 4 + quarter) * C::kWTiles + t) * 32 + lane];
            acc[t] = sum;
          }
        }
      }
      ptx::cluster_arrive_relaxed();  // rank 0: after its rows have landed; the others: at once
      cluster_arrived = true;
    }
    if (ok && rank == 0) {
      const int f = tile * kTileF + quarter * 32 + lane;
      if constexpr (MODE == kRouteSwiglu) {
        // bf16 gate, bf16 up, bf16 silu(gate), bf16 product; MXFP8 over the warp's 32 features
        const float g = round_bf16(acc[0]);
        const float u = round_bf16(acc[1]);
        const float v = round_bf16(silu_bf16_lookup(args.silu_lut, g) * u);
        float amax = fabsf(v);
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
        const uint32_t sbits = ue8m0_scale_bits(amax, 448.0f);
        const uint32_t code = __nv_cvt_float2_to_fp8x2(make_float2(v * ue8m0_inverse(sbits), 0.0f),
                                                       __NV_SATFINITE, __NV_E4M3) & 0xffu;
        static_cast<uint8_t*>(args.out)[(int64_t)route * args.n + f] = (uint8_t)code;
        if (lane == 0) {
          args.out_scales[(int64_t)route * (args.n / kScaleVec) + f / kScaleVec] = (uint8_t)(sbits >> 23);
        }
      } else {
        if (args.out_dtype == kBF16) {
          static_cast<__nv_bfloat16*>(args.out)[(int64_t)route * args.n + f] = __float2bfloat16_rn(acc[0]);
        } else {
          static_cast<__half*>(args.out)[(int64_t)route * args.n + f] = __float2half_rn(acc[0]);
        }
      }
    }
  }

  // ---------------- teardown ----------------
  ptx::tc_fence_before();
  __syncthreads();
  if (ck > 1) {
    if (!cluster_arrived) ptx::cluster_arrive_relaxed();
    ptx::cluster_wait();
  }
  if (*abort_flag != 0) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ------------------------------------------------------------------------------------
// One (token, feature tile) per cluster; the token's lanes split over the cluster's CTAs.
struct WCfg {
  static constexpr uint32_t kStageBytes = kWTileBytes + kAtomBytes + kATileBytes;
  static constexpr uint32_t kSfbBytes = kMaxLanes * 16 * 16 + kAtomBytes;  // K <= 2048 per lane
  static constexpr int kMaxKBlocksPerLane = 16;
  static constexpr uint32_t kRedBytes = kMaxLanes * 4 * 128;  // one term per lane and feature
  static constexpr size_t kBudget = 233472 / 2 - 1024;
  static constexpr int kStages = (int)((kBudget - 2048 - kSfbBytes - kRedBytes) / kStageBytes);
  static constexpr size_t kSmemBytes =
      1024 + (size_t)kStages * kStageBytes + kSfbBytes + kRedBytes + 1024;
  static_assert(kSmemBytes <= kBudget, "two CTAs must fit one SM");
  static constexpr int kSfCol = kMaxLanes * kRows;  // one accumulator per lane
  static constexpr int kSfSets = 4;
  static constexpr int kTmemCols = 256;
  static_assert(kSfCol + kSfSets * 8 <= kTmemCols, "tensor memory layout");
};

__device__ __forceinline__ float gate_of(const RouteArgs& a, int token) {
  const int64_t gi = (int64_t)token * a.gate_stride + (a.gate_stride - 1);
  float x;
  if (a.gate_dtype == kF32) x = static_cast<const float*>(a.shared_gate)[gi];
  else if (a.gate_dtype == kBF16) x = __bfloat162float(static_cast<const __nv_bfloat16*>(a.shared_gate)[gi]);
  else x = __half2float(static_cast<const __half*>(a.shared_gate)[gi]);
  return __fdiv_rn(1.0f, 1.0f + expf(-x));
}

__global__ void __launch_bounds__(kThreads, 2)
route_w2_reduce_kernel(const __grid_constant__ CUtensorMap tm_w,
                       const __grid_constant__ CUtensorMap tm_shared,
                       const __grid_constant__ CUtensorMap tm_a, const RouteArgs args) {
  using C = WCfg;
  ptx::grid_launch_dependents();

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* w_tiles = smem;
  uint8_t* a_tiles = w_tiles + (size_t)C::kStages * kWTileBytes;
  uint8_t* sfa_tiles = a_tiles + (size_t)C::kStages * kATileBytes;
  uint8_t* sfb = sfa_tiles + (size_t)C::kStages * kAtomBytes;
  float* red = reinterpret_cast<float*>(sfb + C::kSfbBytes);
  uint8_t* fixed = reinterpret_cast<uint8_t*>(red) + C::kRedBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(fixed);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(fixed + 8 * (2 * C::kStages + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* own_ids = reinterpret_cast<volatile int*>(tmem_slot + 4);        // [16]
  volatile float* own_weights = reinterpret_cast<volatile float*>(tmem_slot + 20);  // [16]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t full0 = ptx::smem_u32(bars);
  const uint32_t empty0 = full0 + 8 * C::kStages;
  const uint32_t tfull = empty0 + 8 * C::kStages;
  const uint32_t sfb_bar = tfull + 8;
  const uint32_t red_full = sfb_bar + 8;
  const uint32_t ids_bar = red_full + 8;
  // With the logits given, every CTA selects the experts of its token itself (one warp, before
  // the dependency wait: the logits are older than the kernel in front) instead of reading
  // the ids and weights another kernel wrote.
  const bool own_routing = args.logits != nullptr;

  const int cr = args.cluster;
  const int rank = cr > 1 ? (int)ptx::cluster_ctarank() : 0;
  const int unit = (int)blockIdx.x / cr;
  const int token = unit / args.tiles;
  const int tile = unit - token * args.tiles;
  // Lanes in the order of the sum: the shared lane (the last one) first, then 0, 1, ...
  // Position p of that order is lane (p == 0 && shared computed) ? lanes - 1 : p - shared.
  const int shared_first = args.lanes > args.topk ? 1 : 0;
  const int p0 = (rank * args.lanes) / cr;
  const int p1 = ((rank + 1) * args.lanes) / cr;
  const int kbn = args.k_blocks;
  const uint32_t tx_stage = kWTileTxBytes + kAtomBytes + kATileBytes;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < C::kStages; ++s) {
      ptx::mbar_init(full0 + 8 * s, 1);
      ptx::mbar_init(empty0 + 8 * s, 1);
    }
    ptx::mbar_init(tfull, 1);
    ptx::mbar_init(sfb_bar, 1);
    ptx::mbar_init(red_full, 1);
    ptx::mbar_init(ids_bar, 1);
    if (cr > 1 && rank == 0) {
      // terms of the other ranks' lanes: 128 bytes per lane and epilogue warp
      ptx::mbar_arrive_expect_tx(red_full, (uint32_t)(args.lanes - args.lanes / cr) * 4u * 128u);
    }
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tm_w);
    ptx::prefetch_tensormap(&tm_a);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), C::kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (cr > 1) ptx::cluster_sync_all();
  bool cluster_arrived = false;

  // Every warp needs the experts of this CTA's lanes: each reads them for itself (a few words).
  auto lane_of = [&](int p) { return shared_first != 0 ? (p == 0 ? args.lanes - 1 : p - 1) : p; };
  auto expert_of = [&](int l) -> int {
    if (!own_routing) return read_expert(args, token, l);
    if (l >= args.topk) return args.separate_shared != 0 ? -2 : args.num_experts - 1;
    return own_ids[l];
  };

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    // Weights and their scales depend on the routing data only.  Where the caller vouches
    // that this data was complete before the preceding kernel let this one start, the ring
    // is filled with them before the dependency wait; the activation tiles follow after it.
    auto load_weights = [&](int stage, int expert, int kb) {
      const CUtensorMap* wmap = expert == -2 ? &tm_shared : &tm_w;
      const uint8_t* wsc = expert == -2 ? args.shared_w_scales : args.w_scales;
      const int w_row = (expert < 0 ? 0 : expert) * args.w_rows + tile * kTileF;
      const uint32_t bar = full0 + 8 * stage;
      ptx::mbar_arrive_expect_tx(bar, tx_stage);
      ptx::tma_load_2d(ptx::smem_u32(w_tiles + (size_t)stage * kWTileBytes), wmap, kb * kTileK, w_row, bar);
      ptx::bulk_load(ptx::smem_u32(sfa_tiles + (size_t)stage * kAtomBytes),
                     wsc + ((int64_t)(w_row / kAtomRows) * kbn + kb) * kAtomBytes, kAtomBytes, bar);
    };
    int ahead = 0;  // blocks whose weights are already on their way
    bool routed = true;
    if (own_routing) {
      routed = __all_sync(0xffffffffu, bounded_wait(ids_bar, 0u, abort_flag, args.status, 137));
    }
    if (routed && (args.routing_ready != 0 || own_routing)) {
      for (int p = p0; p < p1 && ahead < C::kStages; ++p) {
        const int expert = expert_of(lane_of(p));
        if (expert == -1) continue;
        for (int kb = 0; kb < kbn && ahead < C::kStages; ++kb) {
          if (ptx::elect_one()) load_weights(ahead, expert, kb);
          __syncwarp();
          ++ahead;
        }
      }
    }
    ptx::grid_dependency_wait();
    int stage = 0;
    uint32_t phase = 0;
    int block = 0;
    bool ok = routed;
    for (int p = p0; ok && p < p1; ++p) {
      const int l = lane_of(p);
      const int expert = expert_of(l);
      if (expert == -1) continue;
      const int src_row = token * args.lanes + l;
      for (int kb = 0; ok && kb < kbn; ++kb, ++block) {
        if (block >= ahead) {
          ok = __all_sync(0xffffffffu, bounded_wait(empty0 + 8 * stage, phase ^ 1u, abort_flag,
                                                    args.status, 131));
          if (!ok) break;
        }
        if (ptx::elect_one()) {
          if (block >= ahead) load_weights(stage, expert, kb);
          ptx::tma_load_2d(ptx::smem_u32(a_tiles + (size_t)stage * kATileBytes), &tm_a, kb * kTileK,
                           src_row, full0 + 8 * stage);
        }
        __syncwarp();
        if (++stage == C::kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    constexpr uint32_t kIdesc = (4u << 7) | (0u << 10) | ((uint32_t)(kRows >> 3) << 17) | (1u << 23) |
                                ((uint32_t)(kTileF >> 4) << 24);
    int stage = 0;
    uint32_t phase = 0;
    uint32_t sf_set = 0;
    ptx::grid_dependency_wait();
    bool ok = __all_sync(0xffffffffu, bounded_wait(sfb_bar, 0u, abort_flag, args.status, 132));
    for (int p = p0; ok && p < p1; ++p) {
      const int l = lane_of(p);
      if (!own_routing && read_expert(args, token, l) == -1) continue;
      const uint32_t d_t = tmem_base + (p - p0) * kRows;
      for (int kb = 0; ok && kb < kbn; ++kb) {
        ok = __all_sync(0xffffffffu,
                        bounded_wait(full0 + 8 * stage, phase, abort_flag, args.status, 133));
        if (!ok) break;
        ptx::tc_fence_after();
        if (ptx::elect_one()) {
          const uint32_t sfa_t = tmem_base + C::kSfCol + sf_set * 8;
          const uint32_t sfb_t = sfa_t + 4;
          ptx::tc_cp_32x128b_warpx4(sfa_t, ptx::smem_desc_scale_atom(
                                               ptx::smem_u32(sfa_tiles + (size_t)stage * kAtomBytes)));
          ptx::tc_cp_32x128b_warpx4(sfb_t, ptx::smem_desc_scale_atom(ptx::smem_u32(
                                               sfb + ((p - p0) * C::kMaxKBlocksPerLane + kb) * 16)));
          const uint64_t a_desc = ptx::smem_desc_sw128(ptx::smem_u32(w_tiles + (size_t)stage * kWTileBytes));
          const uint64_t b_desc = ptx::smem_desc_sw128(ptx::smem_u32(a_tiles + (size_t)stage * kATileBytes));
#pragma unroll
          for (int ks = 0; ks < kTileK / kMmaK; ++ks) {
            const uint32_t idesc = kIdesc | ((uint32_t)ks << 4) | ((uint32_t)ks << 29);
            ptx::tc_mma_mxf8f6f4(d_t, a_desc + 2 * ks, b_desc + 2 * ks, idesc, sfa_t, sfb_t,
                                 (kb > 0 || ks > 0) ? 1u : 0u);
          }
          ptx::tc_commit(empty0 + 8 * stage);
        }
        __syncwarp();
        sf_set = (sf_set + 1u) % C::kSfSets;
        if (++stage == C::kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
    if (ok) {
      if (ptx::elect_one()) ptx::tc_commit(tfull);
      __syncwarp();
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int quarter = warp & 3;
    if (own_routing && warp == 2) {
      float weight;
      int id;
      warp_softmax_topk_any(static_cast<const __nv_bfloat16*>(args.logits) +
                                (int64_t)token * args.logit_experts,
                            args.logit_experts, args.topk, args.renormalize, lane, &weight, &id);
      if (lane < args.topk) {
        own_ids[lane] = id;
        own_weights[lane] = weight;
      }
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(ids_bar);
    }
    ptx::grid_dependency_wait();
    if (warp == 2) {
      // activation scale words of this CTA's lanes: lane position q, block kb -> word at
      // (q * 16 + kb) * 16 bytes
      const int count = (p1 - p0) * kbn;
      for (int j = lane; j < count; j += 32) {
        const int q = j / kbn, kb = j - q * kbn;
        const int l = lane_of(p0 + q);
        const uint32_t* words = reinterpret_cast<const uint32_t*>(
            args.act_scales + (int64_t)(token * args.lanes + l) * (kbn * 4));
        *reinterpret_cast<uint32_t*>(sfb + (q * C::kMaxKBlocksPerLane + kb) * 16) = words[kb];
      }
      ptx::fence_proxy_async();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(sfb_bar);
    }
    // Weights of this CTA's lanes (0 for a lane without an expert) and the gate: fetched
    // while the tensor cores work.
    float weight_of[kMaxLanes];
    bool live_lane[kMaxLanes];
    if (own_routing) bounded_wait(ids_bar, 0u, abort_flag, args.status, 138);
#pragma unroll
    for (int q = 0; q < kMaxLanes; ++q) {
      weight_of[q] = 0.0f;
      live_lane[q] = false;
      if (p0 + q < p1) {
        const int l = lane_of(p0 + q);
        live_lane[q] = expert_of(l) != -1;
        weight_of[q] = l >= args.topk ? gate_of(args, token)
                       : own_routing  ? own_weights[l]
                                      : args.topk_weights[(int64_t)token * args.topk + l];
      }
    }
    const int f = tile * kTileF + quarter * 32 + lane;
    const bool bf16_out = args.out_dtype == kBF16;
    float external = 0.0f;
    if (rank == 0 && args.shared_output != nullptr) {
      // a shared row computed elsewhere comes first in the sum, gated
      const int64_t at = (int64_t)token * args.n + f;
      const float s = bf16_out ? __bfloat162float(static_cast<const __nv_bfloat16*>(args.shared_output)[at])
                               : __half2float(static_cast<const __half*>(args.shared_output)[at]);
      external = __fmul_rn(gate_of(args, token), s);
    }
    bool ok = bounded_wait(tfull, 0u, abort_flag, args.status, 134);
    // Every lane's weighted term goes to the owner (rank 0), which adds them one by one in
    // the order of the unfused reduce, so the sum does not depend on the cluster size.
    // terms[quarter][position][32]: the owner's own terms are written in place.
    float* terms = (rank == 0 ? red : reinterpret_cast<float*>(w_tiles)) + quarter * (kMaxLanes * 32);
    if (ok) {
      ptx::tc_fence_after();
      const uint32_t t_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll
      for (int q = 0; q < kMaxLanes; ++q) {
        if (p0 + q < p1) {
          float term = 0.0f;
          if (live_lane[q]) {
            uint32_t r[16];
            ptx::tmem_ld_x16(t_addr + q * kRows, r);
            ptx::tmem_ld_wait();
            // The routed row as the GEMM would have stored it: rounded to the output type.
            const float raw = __uint_as_float(r[0]);
            const float v = bf16_out ? __bfloat162float(__float2bfloat16_rn(raw))
                                     : __half2float(__float2half_rn(raw));
            term = __fmul_rn(weight_of[q], v);
          }
          terms[(p0 + q) * 32 + lane] = term;
        }
      }
    }
    if (cr > 1) {
      if (ok && rank != 0 && p1 > p0) {
        ptx::fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          ptx::bulk_copy_to_peer(
              ptx::mapa(ptx::smem_u32(red + (quarter * kMaxLanes + p0) * 32), 0u),
              ptx::smem_u32(terms + p0 * 32), (uint32_t)(p1 - p0) * 128u, ptx::mapa(red_full, 0u));
        }
      }
      if (rank == 0 && ok) ok = bounded_wait_cluster(red_full, 0u, abort_flag, args.status, 136);
      ptx::cluster_arrive_relaxed();
      cluster_arrived = true;
    }
    if (ok && rank == 0) {
      const int64_t at = (int64_t)token * args.n + f;
      float acc = external;
      int p = 0;
      if (args.shared_output == nullptr) {
        acc = terms[lane];
        p = 1;
      }
      for (; p < args.lanes; ++p) acc = __fadd_rn(acc, terms[p * 32 + lane]);
      if (bf16_out) static_cast<__nv_bfloat16*>(args.out)[at] = __float2bfloat16_rn(acc);
      else static_cast<__half*>(args.out)[at] = __float2half_rn(acc);
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (cr > 1) {
    if (!cluster_arrived) ptx::cluster_arrive_relaxed();
    ptx::cluster_wait();
  }
  if (*abort_flag != 0) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, C::kTmemCols);
  }
}


// ------------------------------------------------------------------------------------
// W1 of the decode schedule with its front end inside: every CTA selects the experts of its
// token itself (softmax top-k of the token's logits by one warp) and quantizes its K slice of
// the token's BF16 row straight into the MMA's shared-memory operand, so the layer needs no
// top-k / quantization kernel in front and this kernel depends on nothing but the layer's
// inputs.  One (route, 128-feature tile) per cluster, K split over the cluster, SwiGLU + MXFP8
// epilogue as route_gemm_kernel<swiglu>; the bytes equal those of topk_quant_kernel followed
// by that kernel (same top-k code, same quantizer arithmetic).
//
// The route's activation: 128 codes per K block at the start of a 1 KB slot (row 0 of a
// 128-byte-swizzled 8-row atom; rows 1..7 and the second atom, which is the next block's slot,
// are never-read padding of the N = 16 operand).  The ring holds ONE weight tile per stage
// (gate and up tiles of a K block alternate), which leaves room for 17 such slots.
struct FCfg {
  static constexpr int kMaxBlocks = 16;                                  // K blocks per CTA
  static constexpr uint32_t kStageBytes = kWTileBytes + kAtomBytes;       // one weight tile
  static constexpr uint32_t kABytes = (kMaxBlocks + 1) * 1024;
  static constexpr uint32_t kSfbBytes = kMaxBlocks * 16 + kAtomBytes;
  static constexpr uint32_t kRedBytes = kMaxCluster * 4 * 2 * 128;
  static constexpr size_t kBudget = 233472 / 2 - 1024;
  static constexpr int kStages = (int)((kBudget - 2048 - kABytes - kSfbBytes - kRedBytes) / kStageBytes);
  static_assert(kStages >= 4, "the ring needs a few stages");
  static constexpr size_t kSmemBytes =
      1024 + (size_t)kStages * kStageBytes + kABytes + kSfbBytes + kRedBytes + 1024;
  static_assert(kSmemBytes <= kBudget, "two CTAs must fit one SM");
  static constexpr int kSfSets = 4;
  static constexpr int kSfaCol = 2 * kRows;                  // behind the two accumulators
  static constexpr int kSfbCol = kSfaCol + kSfSets * 4;
  static constexpr int kTmemCols = 128;
  static_assert(kSfbCol + kSfSets * 4 <= kTmemCols, "tensor memory layout");
};

__device__ __forceinline__ uint32_t e4m3x4_codes(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

__global__ void __launch_bounds__(kThreads, 2)
route_w1_front_kernel(const __grid_constant__ CUtensorMap tm_w,
                      const __grid_constant__ CUtensorMap tm_shared, const RouteArgs args) {
  using C = FCfg;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* w_tiles = smem;                                             // [S][16 KB]
  uint8_t* a_buf = w_tiles + (size_t)C::kStages * kWTileBytes;         // [blocks + 1][1 KB]
  uint8_t* sfa_tiles = a_buf + C::kABytes;                             // [S][512]
  uint8_t* sfb = sfa_tiles + (size_t)C::kStages * kAtomBytes;
  float* red = reinterpret_cast<float*>(sfb + C::kSfbBytes);
  uint8_t* fixed = reinterpret_cast<uint8_t*>(red) + C::kRedBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(fixed);  // full[S], empty[S], tfull, act, ids, red
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(fixed + 8 * (2 * C::kStages + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* expert_slot = reinterpret_cast<volatile int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t full0 = ptx::smem_u32(bars);
  const uint32_t empty0 = full0 + 8 * C::kStages;
  const uint32_t tfull = empty0 + 8 * C::kStages;
  const uint32_t act_bar = tfull + 8;
  const uint32_t ids_bar = act_bar + 8;
  const uint32_t red_full = ids_bar + 8;

  const int ck = args.cluster;
  const int rank = ck > 1 ? (int)ptx::cluster_ctarank() : 0;
  const int unit = (int)blockIdx.x / ck;
  const int route = unit / args.tiles;
  const int tile = unit - route * args.tiles;
  const int token = route / args.lanes;
  const int route_lane = route - token * args.lanes;
  const int kb0 = (rank * args.k_blocks) / ck;
  const int kb1 = ((rank + 1) * args.k_blocks) / ck;
  const uint32_t tx_stage = kWTileTxBytes + kAtomBytes;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < C::kStages; ++s) {
      ptx::mbar_init(full0 + 8 * s, 1);
      ptx::mbar_init(empty0 + 8 * s, 1);
    }
    ptx::mbar_init(tfull, 1);
    ptx::mbar_init(act_bar, 3);   // the three quantizing warps
    ptx::mbar_init(ids_bar, 1);
    ptx::mbar_init(red_full, 1);
    if (ck > 1 && rank == 0) ptx::mbar_arrive_expect_tx(red_full, (uint32_t)(ck * 4 * 2 * 128));
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tm_w);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), C::kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (ck > 1) ptx::cluster_sync_all();
  bool cluster_arrived = false;

  // The hidden rows and the logits come from the kernel before this one.  The kernel after
  // this one starts only now: it may read the logits before its own dependency wait.
  ptx::grid_dependency_wait();
  ptx::grid_launch_dependents();

  if (warp == 0) {
    // ---------------- TMA producer: needs the expert, then streams its two tiles per block ----
    bool ok = __all_sync(0xffffffffu, bounded_wait(ids_bar, 0u, abort_flag, args.status, 141));
    const int expert = ok ? *expert_slot : 0;
    const CUtensorMap* wmap = expert == -2 ? &tm_shared : &tm_w;
    const uint8_t* wsc = expert == -2 ? args.shared_w_scales : args.w_scales;
    const int w_row0 = (expert < 0 ? 0 : expert) * args.w_rows + tile * kTileF;
    int stage = 0;
    uint32_t phase = 0;
    for (int kb = kb0; ok && kb < kb1; ++kb) {
      for (int t = 0; ok && t < 2; ++t) {
        ok = __all_sync(0xffffffffu, bounded_wait(empty0 + 8 * stage, phase ^ 1u, abort_flag,
                                                  args.status, 142));
        if (!ok) break;
        if (ptx::elect_one()) {
          const uint32_t bar = full0 + 8 * stage;
          const int w_row = w_row0 + t * args.n;  // t = 1: the up rows, n rows further down
          ptx::mbar_arrive_expect_tx(bar, tx_stage);
          ptx::tma_load_2d(ptx::smem_u32(w_tiles + (size_t)stage * kWTileBytes), wmap, kb * kTileK,
                           w_row, bar);
          ptx::bulk_load(ptx::smem_u32(sfa_tiles + (size_t)stage * kAtomBytes),
                         wsc + ((int64_t)(w_row / kAtomRows) * args.k_blocks + kb) * kAtomBytes,
                         kAtomBytes, bar);
        }
        __syncwarp();
        if (++stage == C::kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    constexpr uint32_t kIdesc = (4u << 7) | (0u << 10) | ((uint32_t)(kRows >> 3) << 17) | (1u << 23) |
                                ((uint32_t)(kTileF >> 4) << 24);
    int stage = 0;
    uint32_t phase = 0;
    uint32_t set = 0;
    bool ok = __all_sync(0xffffffffu, bounded_wait(act_bar, 0u, abort_flag, args.status, 143));
    for (int kb = kb0; ok && kb < kb1; ++kb) {
      const uint32_t sfb_t = tmem_base + C::kSfbCol + (uint32_t)((kb - kb0) % C::kSfSets) * 4;
      for (int t = 0; ok && t < 2; ++t) {
        ok = __all_sync(0xffffffffu,
                        bounded_wait(full0 + 8 * stage, phase, abort_flag, args.status, 144));
        if (!ok) break;
        ptx::tc_fence_after();
        if (ptx::elect_one()) {
          const uint32_t sfa_t = tmem_base + C::kSfaCol + set * 4;
          ptx::tc_cp_32x128b_warpx4(sfa_t, ptx::smem_desc_scale_atom(
                                               ptx::smem_u32(sfa_tiles + (size_t)stage * kAtomBytes)));
          if (t == 0) {
            ptx::tc_cp_32x128b_warpx4(sfb_t, ptx::smem_desc_scale_atom(ptx::smem_u32(sfb + (kb - kb0) * 16)));
          }
          const uint64_t a_desc = ptx::smem_desc_sw128(ptx::smem_u32(w_tiles + (size_t)stage * kWTileBytes));
          const uint64_t b_desc = ptx::smem_desc_sw128(ptx::smem_u32(a_buf + (size_t)(kb - kb0) * 1024));
#pragma unroll
          for (int ks = 0; ks < kTileK / kMmaK; ++ks) {
            const uint32_t idesc = kIdesc | ((uint32_t)ks << 4) | ((uint32_t)ks << 29);
            ptx::tc_mma_mxf8f6f4(tmem_base + t * kRows, a_desc + 2 * ks, b_desc + 2 * ks, idesc, sfa_t,
                                 sfb_t, (kb > kb0 || ks > 0) ? 1u : 0u);
          }
          ptx::tc_commit(empty0 + 8 * stage);
        }
        __syncwarp();
        set = (set + 1u) % C::kSfSets;
        if (++stage == C::kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
    if (ok) {
      if (ptx::elect_one()) ptx::tc_commit(tfull);
      __syncwarp();
    }
  } else {
    // ---------------- warps 2..5: front end, then the epilogue ----------------
    const int quarter = warp & 3;
    if (warp == 2) {
      // routing of this CTA's token: the route's expert, and once per token the ids and weights
      int expert = args.separate_shared != 0 ? -2 : args.num_experts - 1;  // the shared lane
      if (route_lane < args.topk) {
        float weight;
        int id;
        warp_softmax_topk_any(static_cast<const __nv_bfloat16*>(args.logits) +
                                  (int64_t)token * args.logit_experts,
                              args.logit_experts, args.topk, args.renormalize, lane, &weight, &id);
        expert = __shfl_sync(0xffffffffu, id, route_lane);
        if (route_lane == 0 && tile == 0 && rank == 0 && lane < args.topk) {
          args.ids_out[(int64_t)token * args.topk + lane] = id;
          args.weights_out[(int64_t)token * args.topk + lane] = weight;
        }
      }
      if (lane == 0) {
        *expert_slot = expert;
        ptx::mbar_arrive(ids_bar);
      }
    } else {
      // MXFP8 of this CTA's K slice of the token's row: 8 values per thread, 4 threads per
      // scale group, the arithmetic of the activation quantizer (quantize.cu)
      const int t96 = (int)threadIdx.x - 96;
      const int chunks = (kb1 - kb0) * 16;
      const uint4* row = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(args.hidden) +
                                                        (int64_t)token * args.k_blocks * kTileK +
                                                        (int64_t)kb0 * kTileK);
      for (int c0 = 0; c0 < chunks; c0 += 96) {
        const int c = c0 + t96;
        const bool valid = c < chunks;
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        if (valid) raw = __ldg(row + c);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        float v[8];
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
          *reinterpret_cast<uint2*>(a_buf + (size_t)(c >> 4) * 1024 + (c & 15) * 8) =
              make_uint2(e4m3x4_codes(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv),
                         e4m3x4_codes(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv));
          if ((c & 15) == 0) *reinterpret_cast<uint32_t*>(sfb + (c >> 4) * 16) = word;
        }
      }
      ptx::fence_proxy_async();  // the MMA and tcgen05.cp read these through the async proxy
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(act_bar);
    }
    bool ok = bounded_wait(tfull, 0u, abort_flag, args.status, 145);
    float acc[2] = {0.0f, 0.0f};
    if (ok) {
      ptx::tc_fence_after();
      const uint32_t t_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        uint32_t r[16];
        ptx::tmem_ld_x16(t_addr + t * kRows, r);
        ptx::tmem_ld_wait();
        acc[t] = __uint_as_float(r[0]);  // column 0: the route's row
      }
    }
    if (ck > 1) {
      float* send = reinterpret_cast<float*>(w_tiles) + (quarter * 2) * 32;  // the ring is idle
      if (ok) {
        send[lane] = acc[0];
        send[32 + lane] = acc[1];
        ptx::fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          ptx::bulk_copy_to_peer(ptx::mapa(ptx::smem_u32(red + ((rank * 4 + quarter) * 2) * 32), 0u),
                                 ptx::smem_u32(send), 256u, ptx::mapa(red_full, 0u));
        }
      }
      if (rank == 0 && ok) {
        ok = bounded_wait_cluster(red_full, 0u, abort_flag, args.status, 146);
        if (ok) {
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            float sum = 0.0f;
            for (int src = 0; src < ck; ++src) sum += red[((src * 4 + quarter) * 2 + t) * 32 + lane];
            acc[t] = sum;
          }
        }
      }
      ptx::cluster_arrive_relaxed();
      cluster_arrived = true;
    }
    if (ok && rank == 0) {
      const int f = tile * kTileF + quarter * 32 + lane;
      const float g = round_bf16(acc[0]);
      const float u = round_bf16(acc[1]);
      const float v = round_bf16(silu_bf16_lookup(args.silu_lut, g) * u);
      float amax = fabsf(v);
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
      const uint32_t sbits = ue8m0_scale_bits(amax, 448.0f);
      const uint32_t code = __nv_cvt_float2_to_fp8x2(make_float2(v * ue8m0_inverse(sbits), 0.0f),
                                                     __NV_SATFINITE, __NV_E4M3) & 0xffu;
      static_cast<uint8_t*>(args.out)[(int64_t)route * args.n + f] = (uint8_t)code;
      if (lane == 0) {
        args.out_scales[(int64_t)route * (args.n / kScaleVec) + f / kScaleVec] = (uint8_t)(sbits >> 23);
      }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (ck > 1) {
    if (!cluster_arrived) ptx::cluster_arrive_relaxed();
    ptx::cluster_wait();
  }
  if (*abort_flag != 0) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <class T>
__device__ __forceinline__ T round_to(float v);
template <>
__device__ __forceinline__ __nv_bfloat16 round_to<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <>
__device__ __forceinline__ __half round_to<__half>(float v) {
  return __float2half_rn(v);
}

// out[t] = sigmoid(gate_t) * combined[t * (topk + 1) + topk] + sum_l w[t, l] * combined[t * (topk + 1) + l]
template <class T>
__global__ void __launch_bounds__(256)
moe_reduce_array_kernel(T* __restrict__ out, const T* __restrict__ combined,
                        const float* __restrict__ topk_weights, RouteArgs args) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int token = blockIdx.x;
  const int lanes = args.topk + 1;
  const float gate = gate_of(args, token);
  for (int f = threadIdx.x; f < args.n; f += blockDim.x) {
    const T* rows = combined + (int64_t)token * lanes * args.n + f;
    float acc = __fmul_rn(gate, to_float<T>(rows[(int64_t)args.topk * args.n]));
    for (int l = 0; l < args.topk; ++l) {
      acc = __fadd_rn(acc, __fmul_rn(topk_weights[(int64_t)token * args.topk + l],
                                     to_float<T>(rows[(int64_t)l * args.n])));
    }
    out[(int64_t)token * args.n + f] = round_to<T>(acc);
  }
}

// logits[b, e] = bf16(sum_k hidden[b, k] * gate[e, k]) in FP32, one CTA per gate row; rows
// beyond `routed` (the shared expert's gate row) go to shared_gate[b].
__global__ void __launch_bounds__(256)
router_logits_kernel(const __nv_bfloat16* __restrict__ hidden, const __nv_bfloat16* __restrict__ gate,
                     const __nv_bfloat16* __restrict__ shared_gate_row, __nv_bfloat16* __restrict__ logits,
                     __nv_bfloat16* __restrict__ shared_gate, int batch, int k, int routed) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  constexpr int kTokens = 8;  // tokens per pass over the gate row
  __shared__ float warp_sums[kTokens][8];
  const int e = blockIdx.x;
  const __nv_bfloat16* row = e < routed ? gate + (int64_t)e * k
                                        : (shared_gate_row != nullptr ? shared_gate_row : gate + (int64_t)e * k);
  // Per token the sum runs in one fixed order (a thread's strided elements, a shuffle tree, the
  // warps in turn), whatever the batch size: a token's logits do not depend on its neighbours.
  for (int b0 = 0; b0 < batch; b0 += kTokens) {
    float acc[kTokens];
#pragma unroll
    for (int t = 0; t < kTokens; ++t) acc[t] = 0.0f;
    for (int i = threadIdx.x * 8; i < k; i += blockDim.x * 8) {
      const uint4 w = __ldg(reinterpret_cast<const uint4*>(row + i));
      const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
      for (int t = 0; t < kTokens; ++t) {
        if (b0 + t < batch) {
          const uint4 x = __ldg(reinterpret_cast<const uint4*>(hidden + (int64_t)(b0 + t) * k + i));
          const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 wf = __bfloat1622float2(wp[j]);
            const float2 xf = __bfloat1622float2(xp[j]);
            acc[t] = fmaf(wf.x, xf.x, acc[t]);
            acc[t] = fmaf(wf.y, xf.y, acc[t]);
          }
        }
      }
    }
#pragma unroll
    for (int t = 0; t < kTokens; ++t) {
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) acc[t] += __shfl_xor_sync(0xffffffffu, acc[t], d);
      if ((threadIdx.x & 31) == 0) warp_sums[t][threadIdx.x >> 5] = acc[t];
    }
    __syncthreads();
    if (threadIdx.x < kTokens && b0 + (int)threadIdx.x < batch) {
      const int b = b0 + (int)threadIdx.x;
      float total = 0.0f;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) total += warp_sums[threadIdx.x][w];
      if (e < routed) logits[(int64_t)b * routed + e] = __float2bfloat16_rn(total);
      else shared_gate[b] = __float2bfloat16_rn(total);
    }
    __syncthreads();
  }
}

bool use_pdl() {
  static const bool enabled = []() {
    const char* env = std::getenv("MXFP6_B200_PDL");
    return env == nullptr || env[0] != '0';
  }();
  return enabled;
}

template <class Kernel>
int launch_route(Kernel kernel, size_t smem, int grid, int cluster, cudaStream_t stream,
                 const CUtensorMap& tm_w, const CUtensorMap& tm_shared, const CUtensorMap& tm_a,
                 const RouteArgs& args) {
  // One attribute call per kernel and device.
  static std::mutex mutex;
  static std::unordered_map<const void*, unsigned long long> configured;
  int device = 0;
  MX_CUDA(cudaGetDevice(&device));
  {
    std::lock_guard<std::mutex> lock(mutex);
    unsigned long long& mask = configured[reinterpret_cast<const void*>(kernel)];
    if (device < 64 && (mask >> device & 1ull) == 0) {
      MX_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      MX_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                   cudaSharedmemCarveoutMaxShared));
      mask |= 1ull << device;
    }
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((unsigned)grid);
  config.blockDim = dim3(kThreads);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  int count = 0;
  if (cluster > 1) {
    attribute[count].id = cudaLaunchAttributeClusterDimension;
    attribute[count].val.clusterDim.x = (unsigned)cluster;
    attribute[count].val.clusterDim.y = 1;
    attribute[count].val.clusterDim.z = 1;
    ++count;
  }
  if (use_pdl()) {
    attribute[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[count].val.programmaticStreamSerializationAllowed = 1;
    ++count;
  }
  config.attrs = attribute;
  config.numAttrs = count;
  MX_CUDA(cudaLaunchKernelEx(&config, kernel, tm_w, tm_shared, tm_a, args));
  return kOk;
}

int common_checks(const uint8_t* activation, const uint8_t* act_scales, const uint8_t* weight,
                  const uint8_t* weight_scales, const void* topk_ids, int64_t tokens, int topk,
                  int num_experts, int64_t n, int64_t k) {
  MX_REQUIRE(activation && act_scales && weight && weight_scales && topk_ids,
             "operand pointers must not be null");
  MX_REQUIRE(tokens > 0 && tokens <= (1 << 20) && topk > 0 && topk <= 64,
             "tokens and topk must be positive");
  MX_REQUIRE(num_experts >= 1, "the weight stack holds at least one expert");
  MX_REQUIRE(n > 0 && n % 128 == 0 && n <= INT32_MAX, "N must be a multiple of 128; got %lld",
             (long long)n);
  MX_REQUIRE(k > 0 && k % 128 == 0 && k / 128 <= kMaxKBlocks,
             "K must be a multiple of 128 and at most %d; got %lld", kMaxKBlocks * 128, (long long)k);
  MX_REQUIRE((reinterpret_cast<uintptr_t>(activation) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(weight) & 31) == 0 &&
                 (reinterpret_cast<uintptr_t>(weight_scales) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(act_scales) & 3) == 0,
             "activation 16-byte, weights 32-byte, weight scales 16-byte, logical scales 4-byte aligned");
  return kOk;
}

int sm_count();

// Lanes of a token per CTA of the reduce kernel: two where the launch stays inside the GPU's
// CTA slots, then three, then half of them, then all (clusters of more than two CTAs stop at
// 240 CTAs).  Returns the cluster size.
int lane_cluster(int64_t units, int lanes) {
  const int64_t slots = 2 * (int64_t)sm_count() - 8;
  const int64_t wide_slots = slots - slots / 6;
  const int choices[3] = {(lanes + 1) / 2, (lanes + 2) / 3, 2};
  for (int c : choices) {
    if (c >= 2 && c <= kMaxLaneCluster && c <= lanes && units * c <= (c > 2 ? wide_slots : slots)) {
      return c;
    }
  }
  return 1;
}

int sm_count() {
  static int count = []() {
    int device = 0, sms = 148;
    if (cudaGetDevice(&device) == cudaSuccess) {
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    }
    return sms > 0 ? sms : 148;
  }();
  return count;
}

}  // namespace

// torch.ops.mxfp6.array_gemm_w6a8_out / array_gemm_w6a8_silu_mxfp8_out and the W1 half of the
// split-K decode schedule (csrc/moe.cu:6713-6982, 8648-8916): swiglu != 0 -> weight rows per
// expert = 2 * n (gate rows, then up rows), out = E4M3 [routes, n] + logical scales.
int moe_route_gemm(void* out, uint8_t* out_scales, int out_dtype, int swiglu,
                   const uint8_t* activation, const uint8_t* act_scales, int64_t act_rows,
                   const uint8_t* weight, const uint8_t* weight_scales, int num_experts,
                   const uint8_t* shared_weight, const uint8_t* shared_weight_scales,
                   const void* topk_ids, int ids_are_int64, int64_t tokens, int topk,
                   int include_shared, int64_t n, int64_t k, cudaStream_t stream) {
  if (int rc = common_checks(activation, act_scales, weight, weight_scales, topk_ids, tokens, topk,
                             num_experts, n, k))
    return rc;
  MX_REQUIRE(out != nullptr, "output must not be null");
  MX_REQUIRE(swiglu == 0 || out_scales != nullptr, "the SwiGLU form needs a scale output");
  MX_REQUIRE(swiglu != 0 || out_dtype == kBF16 || out_dtype == kF16, "out_dtype must be float16 or bfloat16");
  MX_REQUIRE((shared_weight == nullptr) == (shared_weight_scales == nullptr),
             "shared_weight and shared_weight_scales go together");
  MX_REQUIRE(shared_weight == nullptr || include_shared != 0, "a shared weight needs include_shared");
  MX_REQUIRE(include_shared == 0 || shared_weight != nullptr || num_experts >= 2,
             "include_shared requires one trailing shared expert");
  const int lanes = topk + (include_shared != 0 ? 1 : 0);
  const int64_t routes = tokens * lanes;
  MX_REQUIRE(act_rows == tokens || act_rows == routes,
             "activation rows must equal tokens or all routed/shared rows");
  const int w_rows = (int)n * (swiglu != 0 ? 2 : 1);
  CUtensorMap tm_w, tm_shared, tm_a;
  if (int rc = make_tensor_map_2d(&tm_w, (int)CU_TENSOR_MAP_DATA_TYPE_16U6_ALIGN16B, weight,
                                  (uint64_t)k, (uint64_t)num_experts * w_rows, (uint64_t)k * 3 / 4, kTileF))
    return rc;
  tm_shared = tm_w;
  if (shared_weight != nullptr) {
    MX_REQUIRE((reinterpret_cast<uintptr_t>(shared_weight) & 31) == 0, "shared weight must be 32-byte aligned");
    if (int rc = make_tensor_map_2d(&tm_shared, (int)CU_TENSOR_MAP_DATA_TYPE_16U6_ALIGN16B, shared_weight,
                                    (uint64_t)k, (uint64_t)w_rows, (uint64_t)k * 3 / 4, kTileF))
      return rc;
  }
  if (int rc = make_tensor_map_2d(&tm_a, (int)CU_TENSOR_MAP_DATA_TYPE_UINT8, activation, (uint64_t)k,
                                  (uint64_t)act_rows, (uint64_t)k, kRows))
    return rc;
  int device = 0;
  MX_CUDA(cudaGetDevice(&device));
  RouteArgs args = {};
  args.w_scales = weight_scales;
  args.shared_w_scales = shared_weight_scales;
  args.act_scales = act_scales;
  args.topk_ids = topk_ids;
  args.ids_are_int64 = ids_are_int64;
  args.out = out;
  args.out_scales = out_scales;
  args.status = device_status_word(device);
  if (args.status == nullptr) return kCudaError;
  args.tokens = (int)tokens;
  args.topk = topk;
  args.lanes = lanes;
  args.act_per_route = act_rows == routes ? 1 : 0;
  args.num_experts = num_experts;
  args.separate_shared = shared_weight != nullptr ? 1 : 0;
  args.n = (int)n;
  args.w_rows = w_rows;
  args.k_blocks = (int)(k / kTileK);
  args.tiles = (int)(n / kTileF);
  args.out_dtype = out_dtype;
  // Split K while the launch stays inside the GPU's CTA slots (two per SM); every CTA keeps
  // at least two K blocks.  Clusters of more than two CTAs do not fill the last slots of
  // the GPU, so such a launch stops at 240 CTAs.
  const int64_t units = routes * args.tiles;
  const int64_t slots = 2 * (int64_t)sm_count() - 8;
  const int64_t wide_slots = slots - slots / 6;
  int ck = (int)std::min<int64_t>({(int64_t)kMaxCluster, wide_slots / units, (int64_t)args.k_blocks / 2});
  if (ck < 2 && units * 2 <= slots && args.k_blocks >= 4) ck = 2;
  if (ck < 1) ck = 1;
  args.cluster = ck;
  MX_REQUIRE(units * ck <= INT32_MAX, "too many routes");
  if (swiglu != 0) {
    if (int rc = silu_table(stream, &args.silu_lut)) return rc;
    return launch_route(route_gemm_kernel<kRouteSwiglu>, RCfg<kRouteSwiglu>::kSmemBytes,
                        (int)(units * ck), ck, stream, tm_w, tm_shared, tm_a, args);
  }
  return launch_route(route_gemm_kernel<kRouteStore>, RCfg<kRouteStore>::kSmemBytes, (int)(units * ck),
                      ck, stream, tm_w, tm_shared, tm_a, args);
}

// torch.ops.mxfp6.array_gemm_w6a8_reduce_out and the W2 half of the split-K decode schedule
// (csrc/moe.cu:6984-7393, 9120-9396): activation [tokens * lanes, K] with lanes = topk + 1
// (the shared row is computed here) or topk (shared_output given, or no shared expert).
int moe_route_w2_reduce(void* out, int out_dtype, const uint8_t* activation,
                        const uint8_t* act_scales, const uint8_t* weight,
                        const uint8_t* weight_scales, int num_experts,
                        const uint8_t* shared_weight, const uint8_t* shared_weight_scales,
                        const void* topk_ids, int ids_are_int64, const float* topk_weights,
                        const void* shared_gate, int gate_dtype, int gate_stride,
                        const void* shared_output, int compute_shared, int64_t tokens, int topk,
                        int64_t n, int64_t k, int routing_ready, const void* logits,
                        int logit_experts, int renormalize, cudaStream_t stream) {
  if (int rc = common_checks(activation, act_scales, weight, weight_scales, topk_ids, tokens, topk,
                             num_experts, n, k))
    return rc;
  MX_REQUIRE(out != nullptr && topk_weights != nullptr, "output and topk_weights must not be null");
  MX_REQUIRE(out_dtype == kBF16 || out_dtype == kF16, "out_dtype must be float16 or bfloat16");
  MX_REQUIRE(!(shared_output != nullptr && compute_shared != 0),
             "a precomputed shared row and a shared lane exclude each other");
  MX_REQUIRE((shared_output == nullptr && compute_shared == 0) || shared_gate != nullptr,
             "the shared expert needs its gate");
  MX_REQUIRE(gate_stride >= 1, "gate stride must be positive");
  MX_REQUIRE((shared_weight == nullptr) == (shared_weight_scales == nullptr),
             "shared_weight and shared_weight_scales go together");
  MX_REQUIRE(shared_weight == nullptr || compute_shared != 0, "a shared weight needs the shared lane");
  const int lanes = topk + (compute_shared != 0 ? 1 : 0);
  MX_REQUIRE(lanes <= kMaxLanes, "at most %d routes per token", kMaxLanes);
  MX_REQUIRE(k / 128 <= WCfg::kMaxKBlocksPerLane, "K of the down projection must be at most %d",
             WCfg::kMaxKBlocksPerLane * 128);
  const int64_t routes = tokens * lanes;
  CUtensorMap tm_w, tm_shared, tm_a;
  if (int rc = make_tensor_map_2d(&tm_w, (int)CU_TENSOR_MAP_DATA_TYPE_16U6_ALIGN16B, weight,
                                  (uint64_t)k, (uint64_t)num_experts * n, (uint64_t)k * 3 / 4, kTileF))
    return rc;
  tm_shared = tm_w;
  if (shared_weight != nullptr) {
    MX_REQUIRE((reinterpret_cast<uintptr_t>(shared_weight) & 31) == 0, "shared weight must be 32-byte aligned");
    if (int rc = make_tensor_map_2d(&tm_shared, (int)CU_TENSOR_MAP_DATA_TYPE_16U6_ALIGN16B, shared_weight,
                                    (uint64_t)k, (uint64_t)n, (uint64_t)k * 3 / 4, kTileF))
      return rc;
  }
  if (int rc = make_tensor_map_2d(&tm_a, (int)CU_TENSOR_MAP_DATA_TYPE_UINT8, activation, (uint64_t)k,
                                  (uint64_t)routes, (uint64_t)k, kRows))
    return rc;
  int device = 0;
  MX_CUDA(cudaGetDevice(&device));
  RouteArgs args = {};
  args.w_scales = weight_scales;
  args.shared_w_scales = shared_weight_scales;
  args.act_scales = act_scales;
  args.topk_ids = topk_ids;
  args.ids_are_int64 = ids_are_int64;
  args.topk_weights = topk_weights;
  args.shared_gate = shared_gate;
  args.gate_dtype = gate_dtype;
  args.gate_stride = gate_stride;
  args.shared_output = shared_output;
  args.out = out;
  args.status = device_status_word(device);
  if (args.status == nullptr) return kCudaError;
  args.tokens = (int)tokens;
  args.topk = topk;
  args.lanes = lanes;
  args.act_per_route = 1;
  args.num_experts = num_experts;
  args.separate_shared = shared_weight != nullptr ? 1 : 0;
  args.n = (int)n;
  args.w_rows = (int)n;
  args.k_blocks = (int)(k / kTileK);
  args.tiles = (int)(n / kTileF);
  args.out_dtype = out_dtype;
  args.routing_ready = routing_ready != 0 ? 1 : 0;
  if (logits != nullptr) {
    MX_REQUIRE(logit_experts >= topk && logit_experts <= 1024 && topk <= 16,
               "in-kernel routing takes up to 1024 experts and top-16");
    MX_REQUIRE(shared_weight != nullptr ? logit_experts <= num_experts : logit_experts < num_experts + (compute_shared != 0 ? 0 : 1),
               "the logits name more experts than the weight stack holds");
    args.logits = logits;
    args.logit_experts = logit_experts;
    args.renormalize = renormalize != 0 ? 1 : 0;
  }
  // Lanes per CTA: two where the launch stays inside the GPU's CTA slots, then three, then
  // half of them, then all (clusters of more than two CTAs stop at 240 CTAs, as above).
  const int64_t units = tokens * args.tiles;
  const int cr = lane_cluster(units, lanes);
  args.cluster = cr;
  return launch_route(route_w2_reduce_kernel, WCfg::kSmemBytes, (int)(units * cr), cr, stream, tm_w,
                      tm_shared, tm_a, args);
}

namespace {
// K split of a W1 launch over `units` (route, tile) pairs (two CTA slots per SM; every CTA keeps
// at least two K blocks; clusters of more than two CTAs stop at 240 CTAs).
int w1_cluster(int64_t units, int k_blocks) {
  const int64_t slots = 2 * (int64_t)sm_count() - 8;
  const int64_t wide_slots = slots - slots / 6;
  int ck = (int)std::min<int64_t>({(int64_t)kMaxCluster, wide_slots / units, (int64_t)k_blocks / 2});
  if (ck < 2 && units * 2 <= slots && k_blocks >= 4) ck = 2;
  return ck < 1 ? 1 : ck;
}
}  // namespace

// Whether moe_decode_layer takes the problem: at most 9 routes per token, a down projection of
// at most 2048 inputs, and at most 16 K blocks of the hidden size per CTA of the W1 launch.
int moe_decode_layer_supported(int64_t tokens, int topk, int logit_experts, int64_t hidden_size,
                               int64_t inter) {
  if (tokens <= 0 || topk <= 0 || topk + 1 > kMaxLanes || logit_experts < topk || logit_experts > 1024)
    return 0;
  if (hidden_size <= 0 || hidden_size % 128 != 0 || inter <= 0 || inter % 128 != 0) return 0;
  if (inter / 128 > WCfg::kMaxKBlocksPerLane) return 0;
  const int k_blocks = (int)(hidden_size / kTileK);
  const int ck = w1_cluster(tokens * (topk + 1) * (inter / kTileF), k_blocks);
  return (k_blocks + ck - 1) / ck <= FCfg::kMaxBlocks ? 1 : 0;
}

// Whether the two-launch form is expected to beat top-k kernel + W1 + W2: wherever it is
// supported.  Measured on the named shape (hidden 2048, intermediate 512, 256 experts, top-8;
// warm, us per layer; three launches / two with W2 selecting again / two with W2 reading the
// ids W1 wrote): 16.5 / 16.6 / 16.5 at 1 token, 19.0 / 20.9 / 18.5 at 2, 26.5 / 26.1 / 24.7 at 4,
// 39.0 / 38.2 / 37.1 at 8, 61.0 / 60.3 / 59.4 at 16, 110.8 / 112.3 / 110.6 at 32.  W2 repeating the
// selection pays only while its CTAs sit beside W1's (1 token); reading the ids is never worse.
int moe_decode_layer_preferred(int64_t tokens, int topk, int logit_experts, int64_t hidden_size,
                               int64_t inter) {
  return moe_decode_layer_supported(tokens, topk, logit_experts, hidden_size, inter);
}

// The decode schedule of one routed-MoE layer in two launches (the reference's three-kernel
// schedule, python/mxfp6/qwen35.py:384-432, without the kernel in front): W1 over routes with
// top-k selection and activation quantization inside every CTA, then W2 with the weighted
// reduce, which selects the experts again for itself while W1 runs.  hidden / logits BF16;
// activation [tokens * (topk + 1), inter] and its logical scales are scratch between the two;
// topk_ids / topk_weights receive the selection.
int moe_decode_layer(void* out, int out_dtype, const void* hidden, const void* logits,
                     const void* shared_gate, int gate_dtype, int gate_stride, const uint8_t* w1,
                     const uint8_t* w1_scales, const uint8_t* w2, const uint8_t* w2_scales,
                     int num_experts, const uint8_t* shared_w1, const uint8_t* shared_w1_scales,
                     const uint8_t* shared_w2, const uint8_t* shared_w2_scales, uint8_t* activation,
                     uint8_t* activation_scales, int32_t* topk_ids, float* topk_weights,
                     int64_t tokens, int topk, int logit_experts, int renormalize,
                     int64_t hidden_size, int64_t inter, int w2_own_routing, cudaStream_t stream) {
  MX_REQUIRE(out && hidden && logits && shared_gate && w1 && w1_scales && w2 && w2_scales &&
                 activation && activation_scales && topk_ids && topk_weights,
             "pointers must not be null");
  MX_REQUIRE(moe_decode_layer_supported(tokens, topk, logit_experts, hidden_size, inter) != 0,
             "the two-launch decode schedule does not take %lld tokens, top-%d, hidden %lld, "
             "intermediate %lld", (long long)tokens, topk, (long long)hidden_size, (long long)inter);
  MX_REQUIRE((shared_w1 == nullptr) == (shared_w1_scales == nullptr) &&
                 (shared_w1 == nullptr) == (shared_w2 == nullptr) &&
                 (shared_w1 == nullptr) == (shared_w2_scales == nullptr),
             "the separate shared expert comes as four pointers or none");
  MX_REQUIRE(shared_w1 != nullptr ? logit_experts <= num_experts : logit_experts < num_experts,
             "the logits name more experts than the weight stack holds");
  MX_REQUIRE((reinterpret_cast<uintptr_t>(hidden) & 15) == 0 && (reinterpret_cast<uintptr_t>(w1) & 31) == 0 &&
                 (reinterpret_cast<uintptr_t>(w1_scales) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(activation_scales) & 3) == 0,
             "hidden 16-byte, weights 32-byte, weight scales 16-byte, activation scales 4-byte aligned");
  const int lanes = topk + 1;
  const int w_rows = (int)inter * 2;
  CUtensorMap tm_w, tm_shared;
  if (int rc = make_tensor_map_2d(&tm_w, (int)CU_TENSOR_MAP_DATA_TYPE_16U6_ALIGN16B, w1,
                                  (uint64_t)hidden_size, (uint64_t)num_experts * w_rows,
                                  (uint64_t)hidden_size * 3 / 4, kTileF))
    return rc;
  tm_shared = tm_w;
  if (shared_w1 != nullptr) {
    MX_REQUIRE((reinterpret_cast<uintptr_t>(shared_w1) & 31) == 0, "shared weight must be 32-byte aligned");
    if (int rc = make_tensor_map_2d(&tm_shared, (int)CU_TENSOR_MAP_DATA_TYPE_16U6_ALIGN16B, shared_w1,
                                    (uint64_t)hidden_size, (uint64_t)w_rows,
                                    (uint64_t)hidden_size * 3 / 4, kTileF))
      return rc;
  }
  int device = 0;
  MX_CUDA(cudaGetDevice(&device));
  RouteArgs args = {};
  args.w_scales = w1_scales;
  args.shared_w_scales = shared_w1_scales;
  args.out = activation;
  args.out_scales = activation_scales;
  args.status = device_status_word(device);
  if (args.status == nullptr) return kCudaError;
  args.tokens = (int)tokens;
  args.topk = topk;
  args.lanes = lanes;
  args.num_experts = num_experts;
  args.separate_shared = shared_w1 != nullptr ? 1 : 0;
  args.n = (int)inter;
  args.w_rows = w_rows;
  args.k_blocks = (int)(hidden_size / kTileK);
  args.tiles = (int)(inter / kTileF);
  args.hidden = hidden;
  args.logits = logits;
  args.ids_out = topk_ids;
  args.weights_out = topk_weights;
  args.logit_experts = logit_experts;
  args.renormalize = renormalize != 0 ? 1 : 0;
  const int64_t units = tokens * lanes * args.tiles;
  args.cluster = w1_cluster(units, args.k_blocks);
  if (int rc = silu_table(stream, &args.silu_lut)) return rc;
  {
    // One attribute call per device.
    static std::mutex mutex;
    static unsigned long long configured = 0;
    std::lock_guard<std::mutex> lock(mutex);
    if (device < 64 && (configured >> device & 1ull) == 0) {
      MX_CUDA(cudaFuncSetAttribute(route_w1_front_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)FCfg::kSmemBytes));
      MX_CUDA(cudaFuncSetAttribute(route_w1_front_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                   cudaSharedmemCarveoutMaxShared));
      configured |= 1ull << device;
    }
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((unsigned)(units * args.cluster));
  config.blockDim = dim3(kThreads);
  config.dynamicSmemBytes = FCfg::kSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  int count = 0;
  if (args.cluster > 1) {
    attribute[count].id = cudaLaunchAttributeClusterDimension;
    attribute[count].val.clusterDim.x = (unsigned)args.cluster;
    attribute[count].val.clusterDim.y = 1;
    attribute[count].val.clusterDim.z = 1;
    ++count;
  }
  if (use_pdl()) {
    attribute[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[count].val.programmaticStreamSerializationAllowed = 1;
    ++count;
  }
  config.attrs = attribute;
  config.numAttrs = count;
  MX_CUDA(cudaLaunchKernelEx(&config, route_w1_front_kernel, tm_w, tm_shared, args));
  // W2 either repeats the selection for itself before its dependency wait (and fills its ring
  // with weights meanwhile), or reads the ids and weights W1 wrote once W1 has completed.
  return moe_route_w2_reduce(out, out_dtype, activation, activation_scales, w2, w2_scales, num_experts,
                             shared_w2, shared_w2_scales, topk_ids, 0, topk_weights, shared_gate,
                             gate_dtype, gate_stride, nullptr, 1, tokens, topk, hidden_size, inter, 0,
                             w2_own_routing != 0 ? logits : nullptr, logit_experts, renormalize, stream);
}

// Router half of torch.ops.mxfp6.qwen35_router_quant_out (csrc/moe.cu:237-511): the BF16 gate
// matrix times the hidden rows; top-k and quantization follow as moe_topk_quant.
int moe_router_logits(const void* hidden, const void* gate_weight, const void* shared_gate_weight,
                      void* routed_logits, void* shared_gate, int64_t batch, int64_t k, int routed,
                      int gate_rows, cudaStream_t stream) {
  MX_REQUIRE(hidden && gate_weight && routed_logits, "pointers must not be null");
  MX_REQUIRE(batch > 0 && batch <= 4096 && k > 0 && k % 8 == 0, "batch and k out of range");
  MX_REQUIRE(routed > 0 && gate_rows >= routed && gate_rows <= routed + 1, "gate rows out of range");
  const int rows = routed + ((shared_gate != nullptr) ? 1 : 0);
  MX_REQUIRE(shared_gate == nullptr || shared_gate_weight != nullptr || gate_rows == routed + 1,
             "the shared gate needs a gate row");
  MX_REQUIRE((reinterpret_cast<uintptr_t>(hidden) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(gate_weight) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(shared_gate_weight) & 15) == 0,
             "hidden and gate weights must be 16-byte aligned");
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((unsigned)rows);
  config.blockDim = dim3(256);
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = use_pdl() ? 1 : 0;
  MX_CUDA(cudaLaunchKernelEx(&config, router_logits_kernel, static_cast<const __nv_bfloat16*>(hidden),
                             static_cast<const __nv_bfloat16*>(gate_weight),
                             static_cast<const __nv_bfloat16*>(shared_gate_weight),
                             static_cast<__nv_bfloat16*>(routed_logits),
                             static_cast<__nv_bfloat16*>(shared_gate), (int)batch, (int)k, routed));
  return kOk;
}

// torch.ops.mxfp6.moe_reduce_array_out (csrc/moe.cu:8237-8282, host :8284-8375).
int moe_reduce_array(void* out, const void* combined, int dtype, const float* topk_weights,
                     const void* shared_gate, int gate_dtype, int gate_stride, int64_t tokens,
                     int topk, int64_t n, cudaStream_t stream) {
  MX_REQUIRE(out && combined && topk_weights && shared_gate, "pointers must not be null");
  MX_REQUIRE(tokens > 0 && tokens <= INT32_MAX && topk > 0 && n > 0 && n <= INT32_MAX,
             "tokens, topk and n must be positive");
  MX_REQUIRE(dtype == kBF16 || dtype == kF16, "dtype must be float16 or bfloat16");
  MX_REQUIRE(gate_stride >= 1, "gate stride must be positive");
  RouteArgs args = {};
  args.shared_gate = shared_gate;
  args.gate_dtype = gate_dtype;
  args.gate_stride = gate_stride;
  args.topk = topk;
  args.n = (int)n;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((unsigned)tokens);
  config.blockDim = dim3(256);
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = use_pdl() ? 1 : 0;
  if (dtype == kBF16) {
    MX_CUDA(cudaLaunchKernelEx(&config, moe_reduce_array_kernel<__nv_bfloat16>,
                               static_cast<__nv_bfloat16*>(out),
                               static_cast<const __nv_bfloat16*>(combined), topk_weights, args));
  } else {
    MX_CUDA(cudaLaunchKernelEx(&config, moe_reduce_array_kernel<__half>, static_cast<__half*>(out),
                               static_cast<const __half*>(combined), topk_weights, args));
  }
  return kOk;
}

}  // namespace mx
