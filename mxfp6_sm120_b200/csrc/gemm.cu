// W6A8 block-scaled GEMM for sm_100a: out[m, f] = alpha * sum_k A8[m,k] * W6[f,k]
// with one UE8M0 scale per 32 K values on both operands.
//
// Replaces the reference's CUTLASS SM120 instantiations
// (csrc/include/mxfp6_gemm/kernel_normal.hpp:94-184, kernel_swapped.hpp:98-317)
// and its grouped kernels (csrc/moe.cu:1483-1692) with ONE persistent,
// warp-specialised tcgen05 kernel:
//   * the weight tile (128 output features x 128 K) is MMA operand A.  TMA reads
//     the packed 6-bit rows with the 16U6_ALIGN16B tensor-map type, which expands
//     every 12 packed bytes to a 16-byte shared-memory segment, the form
//     tcgen05.mma kind::mxf8f6f4 consumes;
//   * the activation tile (TN rows x 128 K, E4M3 bytes) is operand B, so a decode
//     batch of 1..32 rows costs one narrow MMA N instead of a padded 128-row M;
//   * scale atoms (512 bytes = 128 rows x 4 k-groups) are bulk-copied to shared
//     memory and moved to tensor memory with tcgen05.cp; the per-MMA k-group is
//     selected through the scale-id fields of the instruction descriptor;
//   * FP32 accumulators live in tensor memory, double buffered, so the epilogue
//     of tile i overlaps the main loop of tile i+1;
//   * split-K writes FP32 partial tiles to a caller-provided scratch arena and the
//     last-arriving CTA of a tile reduces them in split order (deterministic) and
//     resets the tile counter, so the arena needs zeroing only once.
// Every wait is bounded: on expiry the CTA records a code in the device status
// word, lets its copies drain, frees tensor memory and returns.
#include "gemm.cuh"
#include "ptx.cuh"
#include "wait.cuh"

#include <cuda_fp8.h>

#include <cuda.h>
#include <mutex>
#include <unordered_map>
#include <cstring>
#include <cstdlib>

namespace mx {
namespace {

constexpr int kTileF = 128;         // output features per tile (MMA M)
constexpr int kTileK = 128;         // K values per pipeline stage
constexpr int kMmaK = 32;           // K values per tcgen05.mma
constexpr int kThreads = 192;       // warp 0 TMA, warp 1 MMA, warps 2..5 epilogue
constexpr int kMaxGroups = 512;
constexpr uint32_t kWTileBytes = kTileF * kTileK;  // padded 6-bit rows: 128 B per row
// The mbarrier transaction count of a 16U6_ALIGN16B load is the PACKED byte count
// read from global memory (12 of every 16 shared-memory bytes), measured on B200.
constexpr uint32_t kWTileTxBytes = kWTileBytes / 4 * 3;
constexpr uint32_t kAtomBytes = 512;

struct KernelArgs {
  const uint8_t* w_scales;
  const uint8_t* a_scales;
  const int64_t* expert_offsets;
  const int64_t* scale_offsets;
  void* out;
  float* partials;
  uint32_t* counters;
  int* status;
  int64_t m_total;
  int groups;
  int n;
  int k_blocks;       // k / 128
  int n_tiles;        // ceil(n / 128)
  int splits;
  int out_dtype;
  float alpha;
  int a_scale_row_blocks;  // 128-row blocks present in the activation scale buffer
  // SwiGLU mode: weight matrices hold 2 * n rows (gate rows first, then up rows);
  // the output is E4M3 [m_total, n] with UE8M0 scales per 32 features, logical
  // [m_total, n / 32] and/or packed (row r of group g -> packed row
  // out_scale_offsets[g] + r - expert_offsets[g]; identity when null).
  int w_rows_per_group;
  // > 1: the CTAs of a thread-block cluster split K among themselves and reduce
  // their FP32 partial tiles through distributed shared memory (args.splits == cluster_k).
  int cluster_k;
  uint8_t* out_packed_scales;
  uint8_t* out_logical_scales;
  const int64_t* out_scale_offsets;
  const uint16_t* silu_lut;  // SwiGLU mode: bf16(silu(g)) for every BF16 g (silu_table.cu)
};

constexpr int kModeStore = 0;   // out = cast(alpha * acc)
constexpr int kModeSwiglu = 1;  // out = MXFP8(bf16(silu(bf16 gate)) * bf16 up)

template <int TN, int MODE, int CL>
struct Cfg {
  static constexpr int kWTiles = MODE == kModeSwiglu ? 2 : 1;  // weight tiles per K block
  static constexpr int kSfbAtoms = TN <= 128 ? 1 : 2;
  // 128-K blocks per pipeline stage.  Narrow tiles are bound by the per-stage cost
  // of the issuing warps (barrier wait, fence, commit), so they take more K per stage.
  static constexpr int kSubs =
      MODE == kModeSwiglu ? (TN <= 32 ? 2 : 1) : (TN <= 96 ? 2 : 1);
  // Scale columns rotate through several sets so that the tcgen05.cp of a block
  // never overwrites scales an earlier, still running MMA reads.
  static constexpr int kSfSets = 4;
  static constexpr int kSfSetCols = 4 * kWTiles + 4 * kSfbAtoms;
  static constexpr int kAccCols = kWTiles * TN;  // accumulator columns per buffer
  static constexpr int kAcc = (2 * kAccCols + kSfSets * kSfSetCols <= 512) ? 2 : 1;
  static constexpr int kSfaCol = kAcc * kAccCols;
  static constexpr int kSfbCol = kSfaCol + 4 * kWTiles;
  static constexpr int kColsUsed = kSfaCol + kSfSets * kSfSetCols;
  static_assert(kColsUsed <= 512, "tile does not fit tensor memory");
  static constexpr int kTmemCols =
      kColsUsed <= 32 ? 32 : kColsUsed <= 64 ? 64 : kColsUsed <= 128 ? 128 : kColsUsed <= 256 ? 256 : 512;
  static constexpr uint32_t kATileBytes = TN * kTileK;
  static constexpr uint32_t kStageBytes = kSubs * (kWTiles * kWTileBytes + kATileBytes);
  static constexpr uint32_t kSfStageBytes = kSubs * kAtomBytes * (kWTiles + kSfbAtoms);
  // Per-warp staging of the epilogue: 32 rows x 33 floats (SwiGLU) or 32 x 32 halves.
  static constexpr uint32_t kEpiWarpBytes = MODE == kModeSwiglu ? 32 * 33 * 4 + 128 : 2048;
  static constexpr uint32_t kFixedBytes =
      1024 /*align slack*/ + 8192 /*barriers + tables*/ + 4 * kEpiWarpBytes;
  // Cluster split-K: every CTA parks its FP32 partial tile here for its peers.
  static constexpr bool kClusterOk = CL != 0;
  static_assert(!kClusterOk || TN <= 96, "cluster split-K is for narrow tiles");
  static constexpr uint32_t kRedBytes = kClusterOk ? kAccCols * kTileF * 4 : 0;
  static constexpr int kStagesRaw =
      (int)((232448u - kFixedBytes - kRedBytes) / (kStageBytes + kSfStageBytes));
  static constexpr int kStages = kStagesRaw > 12 ? 12 : kStagesRaw;
  static constexpr size_t kSmemBytes =
      kFixedBytes + kRedBytes + (size_t)kStages * (kStageBytes + kSfStageBytes);
};

struct Work {
  int group, n_tile, m_tile, split, tile_id;
  int64_t row0;        // first activation row of the tile
  int rows;            // valid rows in the tile
  int64_t scale_row0;  // packed-scale row of row0
};

// tile_prefix[g] = number of row tiles of groups < g.
template <int TN>
__device__ __forceinline__ bool decode_work(int w, const KernelArgs& a, const int* tile_prefix,
                                            Work* out) {
  const int total_row_tiles = tile_prefix[a.groups];
  const int total = total_row_tiles * a.n_tiles * a.splits;
  if (w >= total) return false;
  // The issuing warps run this at every tile switch and share their schedulers with
  // polling warps: the common cases (no K split, one row tile per group) avoid divisions.
  int rest = w;
  out->split = 0;
  if (a.splits > 1) {
    rest = w / a.splits;
    out->split = w - rest * a.splits;
  }
  out->tile_id = rest;
  // Largest g with n_tiles * tile_prefix[g] <= rest.
  int lo = 0, hi = a.groups;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (tile_prefix[mid] * a.n_tiles <= rest) lo = mid; else hi = mid;
  }
  // Skip empty groups that share the same prefix value.
  while (lo + 1 < a.groups && tile_prefix[lo + 1] * a.n_tiles <= rest) ++lo;
  out->group = lo;
  const int local = rest - tile_prefix[lo] * a.n_tiles;
  const int mt = tile_prefix[lo + 1] - tile_prefix[lo];
  if (mt == 1) {
    out->m_tile = 0;
    out->n_tile = local;
  } else {
    out->n_tile = local / mt;
    out->m_tile = local - out->n_tile * mt;
  }
  // Group extents were copied to shared memory in the prologue.
  const int* row_begin = tile_prefix + (kMaxGroups + 1);
  const int* scale_begin = row_begin + (kMaxGroups + 1);
  const int first = row_begin[lo] + out->m_tile * TN;  // rows fit 32 bits (checked on the host)
  const int left = row_begin[lo + 1] - first;
  out->row0 = first;
  out->rows = left < TN ? left : TN;
  out->scale_row0 = scale_begin[lo] + out->m_tile * TN;
  return true;
}

// Final value(s) of one (token row, feature) element -> global memory.  In SwiGLU
// mode all 32 lanes of the warp must call together (the scale group is the warp).
template <int MODE>
__device__ __forceinline__ void emit_element(const KernelArgs& args, int64_t row, int f, bool ok,
                                             int lane, float main_acc, float up_acc,
                                             int64_t scale_row) {
  if constexpr (MODE == kModeSwiglu) {
    const int groups = args.n / kScaleVec;
    const float g = round_bf16(main_acc);
    const float u = round_bf16(up_acc);
    const float sv = silu_bf16_lookup(args.silu_lut, g);  // = bf16(g / (1 + expf(-g)))
    const float v = round_bf16(sv * u);
    float amax = fabsf(v);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
    const uint32_t sbits = ue8m0_scale_bits(amax, 448.0f);
    const float inv = ue8m0_inverse(sbits);
    const uint32_t code =
        __nv_cvt_float2_to_fp8x2(make_float2(v * inv, 0.0f), __NV_SATFINITE, __NV_E4M3) & 0xffu;
    if (ok) {
      static_cast<uint8_t*>(args.out)[row * args.n + f] = (uint8_t)code;
      if (lane == 0) {
        const uint8_t sc = (uint8_t)(sbits >> 23);
        const int g_index = f / kScaleVec;
        if (args.out_logical_scales != nullptr) args.out_logical_scales[row * groups + g_index] = sc;
        if (args.out_packed_scales != nullptr)
          args.out_packed_scales[packed_scale_offset(scale_row, g_index, groups)] = sc;
      }
    }
  } else {
    if (ok) {
      if (args.out_dtype == kBF16) {
        static_cast<__nv_bfloat16*>(args.out)[row * args.n + f] =
            __float2bfloat16_rn(args.alpha * main_acc);
      } else {
        static_cast<__half*>(args.out)[row * args.n + f] = __float2half_rn(args.alpha * main_acc);
      }
    }
  }
}

// Cluster split-K reduce of this CTA's share of the token rows: ROWS rows per round, all
// their loads from the (up to RANKS) partial tiles issued before any is used.
template <int TN, int MODE, int ROWS, int RANKS>
__device__ __forceinline__ void cluster_reduce_rows(const KernelArgs& args, const float* red,
                                                    const Work& wk, int my_rank, int cluster_k,
                                                    int f, bool f_ok, int fl, int lane,
                                                    int64_t srow0) {
#pragma unroll 1
  for (int t0 = my_rank; t0 < wk.rows; t0 += ROWS * cluster_k) {
    float vm[ROWS][RANKS], vu[ROWS][RANKS];
#pragma unroll
    for (int j = 0; j < ROWS; ++j) {
      const int t = t0 + j * cluster_k;
      const uint32_t local = ptx::smem_u32(red + t * kTileF + fl);
#pragma unroll
      for (int r = 0; r < RANKS; ++r) {
        vm[j][r] = 0.0f;
        vu[j][r] = 0.0f;
        if (t < wk.rows && r < cluster_k) {
          const uint32_t remote = ptx::mapa(local, (uint32_t)r);
          vm[j][r] = ptx::ld_dsmem_f32(remote);
          if (MODE == kModeSwiglu) vu[j][r] = ptx::ld_dsmem_f32(remote + TN * kTileF * 4);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < ROWS; ++j) {
      const int t = t0 + j * cluster_k;
      float main_acc = 0.0f, up_acc = 0.0f;
#pragma unroll
      for (int r = 0; r < RANKS; ++r) {
        if (r < cluster_k) {
          main_acc += vm[j][r];
          up_acc += vu[j][r];
        }
      }
      if (t < wk.rows) {  // warp-uniform: every lane of the warp has the same t
        emit_element<MODE>(args, wk.row0 + t, f, f_ok, lane, main_acc, up_acc, srow0 + t);
      }
    }
  }
}

template <int TN, int MODE, int CL>
__global__ void __launch_bounds__(kThreads, 1)
w6a8_gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_a,
                 const KernelArgs args) {
  using C = Cfg<TN, MODE, CL>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* w_tiles = smem;
  uint8_t* a_tiles = w_tiles + (size_t)C::kStages * C::kSubs * C::kWTiles * kWTileBytes;
  uint8_t* sf_tiles = a_tiles + (size_t)C::kStages * C::kSubs * C::kATileBytes;
  uint8_t* fixed = sf_tiles + (size_t)C::kStages * C::kSfStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(fixed);  // full[S], empty[S], tfull[2], tempty[2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(fixed + 8 * (2 * C::kStages + 6));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* last_flag = reinterpret_cast<volatile int*>(tmem_slot + 2);
  // Three tables of kMaxGroups + 1 ints: row-tile prefix, first row, first scale row.
  int* tile_prefix = reinterpret_cast<int*>(fixed + 1024);
  uint8_t* epi_stage = fixed + 8192;                          // 4 x kEpiWarpBytes
  float* red = reinterpret_cast<float*>(fixed + 8192 + 4 * C::kEpiWarpBytes);  // cluster partial tile

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t full0 = ptx::smem_u32(bars);
  const uint32_t empty0 = full0 + 8 * C::kStages;
  const uint32_t tfull0 = empty0 + 8 * C::kStages;
  const uint32_t tempty0 = tfull0 + 16;
  const uint32_t red_full = tempty0 + 16;   // all partial tiles of the cluster are written
  const uint32_t red_empty = red_full + 8;  // all peers have read this CTA's partial tile
  const int cluster_k = CL != 0 ? args.cluster_k : 1;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    *last_flag = 0;
    for (int s = 0; s < C::kStages; ++s) {
      ptx::mbar_init(full0 + 8 * s, 1);
      ptx::mbar_init(empty0 + 8 * s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(tfull0 + 8 * i, 1);
      ptx::mbar_init(tempty0 + 8 * i, 4);
    }
    ptx::mbar_init(red_full, 4 * (cluster_k > 1 ? cluster_k : 1));
    ptx::mbar_init(red_empty, 4 * (cluster_k > 1 ? cluster_k : 1));
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tm_w);
    ptx::prefetch_tensormap(&tm_a);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), C::kTmemCols);
    ptx::tmem_relinquish();
  }
  // Touch every 64-byte line of the kernel parameters now, so that the constant-cache
  // misses of a fresh launch overlap the previous kernel instead of the first copies.
  if (threadIdx.x >= 64 && threadIdx.x < 64 + (int)((sizeof(KernelArgs) + 63) / 64)) {
    const uint32_t word = reinterpret_cast<const uint32_t*>(&args)[(threadIdx.x - 64) * 16];
    asm volatile("" ::"r"(word));
  }
  // Row-tile prefix table (one entry per group).
  int* row_begin_tab = tile_prefix + (kMaxGroups + 1);
  int* scale_begin_tab = row_begin_tab + (kMaxGroups + 1);
  const bool dense = args.expert_offsets == nullptr;
  if (dense) {
    // A dense launch needs nothing from earlier kernels for its table or for the cluster
    // handshake: both happen before the wait, off the critical path of a decode chain.
    if (threadIdx.x == 0) {
      tile_prefix[0] = 0;
      tile_prefix[1] = (int)((args.m_total + TN - 1) / TN);
      row_begin_tab[0] = 0;
      row_begin_tab[1] = (int)args.m_total;
      scale_begin_tab[0] = 0;
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    if (cluster_k > 1) ptx::cluster_sync_all();
  }
  // Everything above is independent of earlier kernels; from here on global memory
  // written by them is read, so wait for them, then let the next kernel's prologue start.
  ptx::grid_dependency_wait();
  ptx::grid_launch_dependents();
  if (!dense) {
    for (int g = threadIdx.x; g <= args.groups; g += kThreads) {
      const int64_t first = args.expert_offsets[g];
      row_begin_tab[g] = (int)first;
      scale_begin_tab[g] = (int)args.scale_offsets[g];
      if (g < args.groups) {
        const int64_t rows = args.expert_offsets[g + 1] - first;
        tile_prefix[g + 1] = (int)((rows + TN - 1) / TN);
      }
    }
    __syncthreads();
    if (warp == 0) {
      int carry = 0;
      for (int base = 0; base < args.groups; base += 32) {
        const int g = base + lane;
        const int v = g < args.groups ? tile_prefix[g + 1] : 0;
        int incl = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const int up = __shfl_up_sync(0xffffffffu, incl, d);
          if (lane >= d) incl += up;
        }
        if (g < args.groups) tile_prefix[g + 1] = carry + incl;
        carry += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (lane == 0) tile_prefix[0] = 0;
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    // Peers must see this CTA's barriers initialised before they arrive on them.
    if (cluster_k > 1) ptx::cluster_sync_all();
  }
  const uint32_t tmem_base = *tmem_slot;

  const int kb_total = args.k_blocks;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    // The whole warp runs the loop (so that addresses stay warp-uniform) and one
    // elected lane issues the copies.
    {
      int stage = 0;
      uint32_t phase = 0;
      const uint32_t tx_sub = C::kWTiles * kWTileTxBytes + C::kATileBytes +
                              kAtomBytes * (C::kWTiles + C::kSfbAtoms);
      const int atoms_per_rb = kb_total;  // k/128 atoms per 128-row block
      Work wk;
      bool ok = true;
      for (int w = blockIdx.x; ok && decode_work<TN>(w, args, tile_prefix, &wk); w += gridDim.x) {
        const int kb0 = args.splits > 1 ? (wk.split * kb_total) / args.splits : 0;
        const int kb1 = args.splits > 1 ? ((wk.split + 1) * kb_total) / args.splits : kb_total;
        const int w_row = wk.group * args.w_rows_per_group + wk.n_tile * kTileF;
        const int sfb_rb0 = (int)(wk.scale_row0 / kAtomRows);
        for (int kb = kb0; kb < kb1; kb += C::kSubs) {
          const int nsub = (kb1 - kb) < C::kSubs ? (kb1 - kb) : C::kSubs;
          ok = __all_sync(0xffffffffu, bounded_wait(empty0 + 8 * stage, phase ^ 1u, abort_flag,
                                                    args.status, 101));
          if (!ok) break;
          const uint32_t bar = full0 + 8 * stage;
          if (ptx::elect_one()) {
            ptx::mbar_arrive_expect_tx(bar, tx_sub * nsub);
            for (int sub = 0; sub < nsub; ++sub) {
#pragma unroll
              for (int t = 0; t < C::kWTiles; ++t) {
                // tile 0: gate rows (or the only tile); tile 1: up rows, n rows further down
                ptx::tma_load_2d(
                    ptx::smem_u32(w_tiles + (size_t)((stage * C::kSubs + sub) * C::kWTiles + t) *
                                                kWTileBytes),
                    &tm_w, (kb + sub) * kTileK, w_row + t * args.n, bar);
              }
              ptx::tma_load_2d(
                  ptx::smem_u32(a_tiles + (size_t)(stage * C::kSubs + sub) * C::kATileBytes),
                  &tm_a, (kb + sub) * kTileK, (int)wk.row0, bar);
            }
            // Scale atoms of consecutive K blocks are adjacent in memory: one bulk
            // copy per operand row block covers the whole stage.
            uint8_t* sf = sf_tiles + (size_t)stage * C::kSfStageBytes;
#pragma unroll
            for (int t = 0; t < C::kWTiles; ++t) {
              const uint8_t* sfa_src =
                  args.w_scales +
                  ((int64_t)((w_row + t * args.n) / kAtomRows) * atoms_per_rb + kb) * kAtomBytes;
              ptx::bulk_load(ptx::smem_u32(sf + kAtomBytes * C::kSubs * t), sfa_src,
                             kAtomBytes * nsub, bar);
            }
#pragma unroll
            for (int j = 0; j < C::kSfbAtoms; ++j) {
              // A tile that ends inside the last row block re-reads that block for
              // the rows it does not have; those accumulator rows are never stored.
              int rb = sfb_rb0 + j;
              if (rb >= args.a_scale_row_blocks) rb = args.a_scale_row_blocks - 1;
              ptx::bulk_load(ptx::smem_u32(sf + kAtomBytes * C::kSubs * (C::kWTiles + j)),
                             args.a_scales + ((int64_t)rb * atoms_per_rb + kb) * kAtomBytes,
                             kAtomBytes * nsub, bar);
            }
          }
          __syncwarp();
          if (++stage == C::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      // E3M2 weights (A, format 4) x E4M3 activations (B, format 0), both K-major,
      // UE8M0 scales, M = 128, N = TN.
      constexpr uint32_t kIdesc = (4u << 7) | (0u << 10) | ((uint32_t)(TN >> 3) << 17) |
                                  (1u << 23) | ((uint32_t)(kTileF >> 4) << 24);
      uint32_t sf_set = 0;
      Work wk;
      bool ok = true;
      for (int w = blockIdx.x; ok && decode_work<TN>(w, args, tile_prefix, &wk); w += gridDim.x) {
        const int kb0 = args.splits > 1 ? (wk.split * kb_total) / args.splits : 0;
        const int kb1 = args.splits > 1 ? ((wk.split + 1) * kb_total) / args.splits : kb_total;
        if (!__all_sync(0xffffffffu, bounded_wait(tempty0 + 8 * acc, acc_phase ^ 1u, abort_flag,
                                                  args.status, 102)))
          break;
        ptx::tc_fence_after();
        const uint32_t d_t = tmem_base + acc * C::kAccCols;
        const uint32_t sfb_sub = (uint32_t)((wk.scale_row0 % kAtomRows) / 32);
        for (int kb = kb0; kb < kb1; kb += C::kSubs) {
          const int nsub = (kb1 - kb) < C::kSubs ? (kb1 - kb) : C::kSubs;
          ok = __all_sync(0xffffffffu,
                          bounded_wait(full0 + 8 * stage, phase, abort_flag, args.status, 103));
          if (!ok) break;
          ptx::tc_fence_after();
          if (ptx::elect_one()) {
            const uint32_t sf = ptx::smem_u32(sf_tiles + (size_t)stage * C::kSfStageBytes);
            for (int sub = 0; sub < nsub; ++sub) {
              const uint32_t sfa_t = tmem_base + C::kSfaCol + sf_set * C::kSfSetCols;
              const uint32_t sfb_base = tmem_base + C::kSfbCol + sf_set * C::kSfSetCols;
              const uint32_t sfb_t = sfb_base + sfb_sub;
              sf_set = (sf_set + 1u) % C::kSfSets;
#pragma unroll
              for (int t = 0; t < C::kWTiles; ++t) {
                ptx::tc_cp_32x128b_warpx4(
                    sfa_t + 4 * t, ptx::smem_desc_scale_atom(sf + kAtomBytes * (C::kSubs * t + sub)));
              }
#pragma unroll
              for (int j = 0; j < C::kSfbAtoms; ++j) {
                ptx::tc_cp_32x128b_warpx4(
                    sfb_base + 4 * j,
                    ptx::smem_desc_scale_atom(sf + kAtomBytes * (C::kSubs * (C::kWTiles + j) + sub)));
              }
              const uint64_t b_desc = ptx::smem_desc_sw128(
                  ptx::smem_u32(a_tiles + (size_t)(stage * C::kSubs + sub) * C::kATileBytes));
#pragma unroll
              for (int t = 0; t < C::kWTiles; ++t) {
                const uint64_t a_desc = ptx::smem_desc_sw128(ptx::smem_u32(
                    w_tiles + (size_t)((stage * C::kSubs + sub) * C::kWTiles + t) * kWTileBytes));
#pragma unroll
                for (int ks = 0; ks < kTileK / kMmaK; ++ks) {
                  const uint32_t idesc = kIdesc | ((uint32_t)ks << 4) | ((uint32_t)ks << 29);
                  // 32 K values = 32 bytes = 2 descriptor address units.
                  ptx::tc_mma_mxf8f6f4(d_t + t * TN, a_desc + 2 * ks, b_desc + 2 * ks, idesc,
                                       sfa_t + 4 * t, sfb_t, (kb + sub > kb0 || ks > 0) ? 1u : 0u);
                }
              }
            }
            ptx::tc_commit(empty0 + 8 * stage);
          }
          __syncwarp();
          if (++stage == C::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        if (ptx::elect_one()) ptx::tc_commit(tfull0 + 8 * acc);
        __syncwarp();
        if (++acc == C::kAcc) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int quarter = warp & 3;  // tensor-memory lane quarter this warp may read
    const int fl = quarter * 32 + lane;
    const int etid = threadIdx.x - 64;  // 0..127
    int acc = 0;
    uint32_t acc_phase = 0;
    uint32_t red_phase = 0;
    bool red_used = false;
    const uint32_t my_rank = cluster_k > 1 ? ptx::cluster_ctarank() : 0u;
    Work wk;
    for (int w = blockIdx.x; decode_work<TN>(w, args, tile_prefix, &wk); w += gridDim.x) {
      bool ready = bounded_wait(tfull0 + 8 * acc, acc_phase, abort_flag, args.status, 104);
      if constexpr (C::kClusterOk) {
        if (cluster_k > 1) {
          // ---- cluster split-K: partial tile -> own shared memory -> peers reduce ----
          if (!ready) break;
          ptx::tc_fence_after();
          const uint32_t t_addr0 =
              tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * C::kAccCols;
          // Peers must have finished reading the partial tile of the previous round.
          if (!bounded_wait_cluster(red_empty, red_phase ^ 1u, abort_flag, args.status, 105)) break;
#pragma unroll 1
          for (int c0 = 0; c0 < wk.rows; c0 += 16) {
#pragma unroll
            for (int t = 0; t < C::kWTiles; ++t) {
              uint32_t r[16];
              ptx::tmem_ld_x16(t_addr0 + t * TN + c0, r);
              ptx::tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                if (c0 + j < wk.rows) red[(t * TN + c0 + j) * kTileF + fl] = __uint_as_float(r[j]);
              }
            }
          }
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(tempty0 + 8 * acc);
          if (++acc == C::kAcc) {
            acc = 0;
            acc_phase ^= 1u;
          }
          // One arrival per epilogue warp on every CTA of the cluster (release).
          if (lane < cluster_k) ptx::mbar_arrive_remote(ptx::mapa(red_full, (uint32_t)lane));
          red_used = true;
          if (!bounded_wait_cluster(red_full, red_phase, abort_flag, args.status, 106)) break;
          const int f = wk.n_tile * kTileF + fl;
          const bool f_ok = f < args.n;
          const int64_t srow0 = args.out_scale_offsets != nullptr ? wk.scale_row0 : wk.row0;
          // Token rows are dealt round-robin to the CTAs; the sum runs over the ranks
          // in order, so the result does not depend on timing.  A round keeps 32 remote
          // loads in flight per lane: the fewer the ranks, the more rows per round.
          if (cluster_k <= 2) {
            cluster_reduce_rows<TN, MODE, 16, 2>(args, red, wk, (int)my_rank, cluster_k, f, f_ok,
                                                 fl, lane, srow0);
          } else if (cluster_k <= 4) {
            cluster_reduce_rows<TN, MODE, 8, 4>(args, red, wk, (int)my_rank, cluster_k, f, f_ok, fl,
                                                lane, srow0);
          } else {
            cluster_reduce_rows<TN, MODE, 4, 8>(args, red, wk, (int)my_rank, cluster_k, f, f_ok, fl,
                                                lane, srow0);
          }
          __syncwarp();
          // Nothing is published by this arrival (the peers' tiles were only read, and the
          // values have been used), so it needs no release fence.
          if (lane < cluster_k)
            ptx::mbar_arrive_remote_relaxed(ptx::mapa(red_empty, (uint32_t)lane));
          red_phase ^= 1u;
          continue;
        }
      }
      if (args.splits > 1) {
        // The split-K path below uses a 128-thread named barrier, so the four
        // epilogue warps must agree on whether to go on.
        uint32_t all;
        asm volatile(
            "{\n\t.reg .pred p, q;\n\t"
            "setp.ne.b32 p, %1, 0;\n\t"
            "bar.red.and.pred q, 1, 128, p;\n\t"
            "selp.u32 %0, 1, 0, q;\n\t}"
            : "=r"(all)
            : "r"((uint32_t)ready)
            : "memory");
        ready = all != 0;
      }
      if (!ready) break;
      ptx::tc_fence_after();
      const int f = wk.n_tile * kTileF + fl;
      const bool f_ok = f < args.n;
      const uint32_t t_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * C::kAccCols;
      float* part = nullptr;
      if (args.splits > 1) {
        part = args.partials + ((size_t)wk.tile_id * args.splits + wk.split) * (TN * kTileF);
      }
      // Lane = feature, column = token row in tensor memory; global memory wants
      // the features of a row next to each other.  Each warp turns 32 columns at a
      // time through its own slice of shared memory and then writes whole row
      // segments with 16-byte stores.  Columns at or beyond wk.rows are skipped.
      constexpr int kChunk = TN >= 32 ? 32 : 16;
      uint8_t* stage_bytes = epi_stage + quarter * C::kEpiWarpBytes;
      const int f0 = wk.n_tile * kTileF + quarter * 32;  // first feature of this warp
      if constexpr (MODE == kModeSwiglu) {
        float* stage = reinterpret_cast<float*>(stage_bytes);  // [kChunk][33]
        const int groups = args.n / kScaleVec;
        const int g_index = f0 / kScaleVec;
        // Output scales of a grouped launch share the activation's scale rows.
        const int64_t srow0 = args.out_scale_offsets != nullptr ? wk.scale_row0 : wk.row0;
#pragma unroll 1
        for (int c0 = 0; c0 < wk.rows; c0 += kChunk) {
          uint32_t rg[kChunk], ru[kChunk];
          ptx::tmem_ld_chunk<kChunk>(t_addr + c0, rg);
          ptx::tmem_ld_chunk<kChunk>(t_addr + TN + c0, ru);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < kChunk; ++j) {
            const float g = round_bf16(__uint_as_float(rg[j]));
            const float u = round_bf16(__uint_as_float(ru[j]));
            const float sv = silu_bf16_lookup(args.silu_lut, g);  // = bf16(g / (1 + expf(-g)))
            stage[j * 33 + lane] = round_bf16(sv * u);
          }
          __syncwarp();
          // Now lane = token row: its 32 features are one scale group.
          if (lane < kChunk) {
            float v[32];
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              v[i] = stage[lane * 33 + i];
              amax = fmaxf(amax, fabsf(v[i]));
            }
            const uint32_t sbits = ue8m0_scale_bits(amax, 448.0f);
            const float inv = ue8m0_inverse(sbits);
            uint32_t w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const uint32_t lo = __nv_cvt_float2_to_fp8x2(
                  make_float2(v[4 * i] * inv, v[4 * i + 1] * inv), __NV_SATFINITE, __NV_E4M3);
              const uint32_t hi = __nv_cvt_float2_to_fp8x2(
                  make_float2(v[4 * i + 2] * inv, v[4 * i + 3] * inv), __NV_SATFINITE, __NV_E4M3);
              w[i] = lo | (hi << 16);
            }
            const int t = c0 + lane;
            if (t < wk.rows && f0 < args.n) {
              const int64_t row = wk.row0 + t;
              uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(args.out) + row * args.n + f0);
              dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
              dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
              const uint8_t sc = (uint8_t)(sbits >> 23);
              if (args.out_logical_scales != nullptr)
                args.out_logical_scales[row * groups + g_index] = sc;
              if (args.out_packed_scales != nullptr)
                args.out_packed_scales[packed_scale_offset(srow0 + t, g_index, groups)] = sc;
            }
          }
          __syncwarp();
        }
      } else if (args.splits > 1) {
#pragma unroll 1
        for (int c0 = 0; c0 < wk.rows; c0 += 16) {
          uint32_t r[16];
          ptx::tmem_ld_x16(t_addr + c0, r);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (c0 + j < wk.rows) __stcg(part + (c0 + j) * kTileF + fl, __uint_as_float(r[j]));
          }
        }
      } else {
        uint16_t* stage = reinterpret_cast<uint16_t*>(stage_bytes);  // [kChunk][32] halves
        const bool bf16_out = args.out_dtype == kBF16;
#pragma unroll 1
        for (int c0 = 0; c0 < wk.rows; c0 += kChunk) {
          uint32_t r[kChunk];
          ptx::tmem_ld_chunk<kChunk>(t_addr + c0, r);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < kChunk; ++j) {
            const float v = args.alpha * __uint_as_float(r[j]);
            stage[j * 32 + lane] = bf16_out ? __bfloat16_as_ushort(__float2bfloat16_rn(v))
                                            : __half_as_ushort(__float2half_rn(v));
          }
          __syncwarp();
          // 4 lanes cover one 64-byte row segment; a warp writes 8 rows per pass.
          const int seg = lane & 3;
          const int fseg = f0 + seg * 8;
#pragma unroll
          for (int pass = 0; pass < kChunk / 8; ++pass) {
            const int rr = (lane >> 2) + 8 * pass;
            const int t = c0 + rr;
            if (t < wk.rows && fseg < args.n) {
              const uint4 v = *reinterpret_cast<const uint4*>(stage + rr * 32 + seg * 8);
              *reinterpret_cast<uint4*>(static_cast<uint16_t*>(args.out) +
                                        (wk.row0 + t) * args.n + fseg) = v;
            }
          }
          __syncwarp();
        }
      }
      // Accumulator buffer is free for the next tile.
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(tempty0 + 8 * acc);
      if (++acc == C::kAcc) {
        acc = 0;
        acc_phase ^= 1u;
      }
      if (args.splits > 1) {
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (etid == 0) {
          const uint32_t old = atomicAdd(args.counters + wk.tile_id, 1u);
          *last_flag = (old == (uint32_t)(args.splits - 1)) ? 1 : 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const bool last = *last_flag != 0;
        if (last) {
          __threadfence();
          const float* base = args.partials + (size_t)wk.tile_id * args.splits * (TN * kTileF);
          // Eight rows at a time so that 8 x splits independent loads are in
          // flight per thread; the sum over splits stays in split order.
          for (int t0 = 0; t0 < wk.rows; t0 += 8) {
            float sum[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) sum[j] = 0.0f;
            for (int s = 0; s < args.splits; ++s) {
              const float* src = base + ((size_t)s * TN + t0) * kTileF + fl;
              float v[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] = (t0 + j < wk.rows) ? __ldcg(src + j * kTileF) : 0.0f;
#pragma unroll
              for (int j = 0; j < 8; ++j) sum[j] += v[j];
            }
            if (f_ok) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                if (t0 + j < wk.rows) {
                  const int64_t idx = (wk.row0 + t0 + j) * args.n + f;
                  if (args.out_dtype == kBF16) {
                    static_cast<__nv_bfloat16*>(args.out)[idx] =
                        __float2bfloat16_rn(args.alpha * sum[j]);
                  } else {
                    static_cast<__half*>(args.out)[idx] = __float2half_rn(args.alpha * sum[j]);
                  }
                }
              }
            }
          }
          if (etid == 0) args.counters[wk.tile_id] = 0u;  // self-reset for the next launch
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
    }
    // A CTA of a cluster must not exit while peers may still read its partial tile.
    if (cluster_k > 1 && red_used) {
      bounded_wait_cluster(red_empty, red_phase ^ 1u, abort_flag, args.status, 107);
    }
  }

  // ---------------- teardown ----------------
  ptx::tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0) {
    // Give copies and MMAs still in flight time to land before the CTA's shared
    // and tensor memory are handed back.
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ------------------------------------------------------------------ host side

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                              const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                              const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = []() -> EncodeFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) !=
            cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      return nullptr;
    }
    return reinterpret_cast<EncodeFn>(p);
  }();
  return fn;
}

int make_map(CUtensorMap* map, CUtensorMapDataType type, const void* base, uint64_t inner,
             uint64_t rows, uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_rows) {
  EncodeFn fn = encode_fn();
  if (fn == nullptr) {
    set_error("cuTensorMapEncodeTiled is not available from the CUDA driver");
    return kCudaError;
  }
  const cuuint64_t dims[2] = {inner, rows};
  const cuuint64_t strides[1] = {row_stride_bytes};
  const cuuint32_t box[2] = {box_inner, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  // 32-bit maps describe rows of packed scale atoms (512 bytes each), copied unswizzled.
  const CUresult rc = fn(map, type, 2, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE,
                         type == CU_TENSOR_MAP_DATA_TYPE_UINT32 ? CU_TENSOR_MAP_SWIZZLE_NONE
                                                                : CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (inner=%llu rows=%llu stride=%llu)",
              (int)rc, (unsigned long long)inner, (unsigned long long)rows,
              (unsigned long long)row_stride_bytes);
    return kCudaError;
  }
  return kOk;
}

// Tensor maps are pure functions of (pointer, extents, box); encoding costs a
// few microseconds, so a small per-process cache keeps it off the decode path.
struct MapKey {
  const void* base;
  uint64_t inner, rows;
  uint32_t box_rows;
  int type;
  bool operator==(const MapKey& o) const {
    return base == o.base && inner == o.inner && rows == o.rows && box_rows == o.box_rows &&
           type == o.type;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.base);
    h = h * 1000003u ^ k.inner;
    h = h * 1000003u ^ k.rows;
    h = h * 1000003u ^ k.box_rows;
    h = h * 1000003u ^ (size_t)k.type;
    return h;
  }
};
std::mutex g_map_mutex;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;

int cached_map(CUtensorMap* out, CUtensorMapDataType type, const void* base, uint64_t inner,
               uint64_t rows, uint64_t stride, uint32_t box_rows) {
  const MapKey key{base, inner, rows, box_rows, (int)type};
  {
    std::lock_guard<std::mutex> lock(g_map_mutex);
    auto it = g_maps.find(key);
    if (it != g_maps.end()) {
      *out = it->second;
      return kOk;
    }
  }
  CUtensorMap map;
  if (int rc = make_map(&map, type, base, inner, rows, stride, kTileK, box_rows)) return rc;
  {
    std::lock_guard<std::mutex> lock(g_map_mutex);
    if (g_maps.size() > 4096) g_maps.clear();
    g_maps.emplace(key, map);
  }
  *out = map;
  return kOk;
}

int g_split_mode = 1;

bool use_pdl() {
  static const bool enabled = []() {
    const char* env = std::getenv("MXFP6_B200_PDL");
    return env == nullptr || env[0] != '0';
  }();
  return enabled;
}

template <int TN, int MODE, int CL>
int launch_variant(const CUtensorMap& tm_w, const CUtensorMap& tm_a, const KernelArgs& args,
                   const GemmPlan& plan, cudaStream_t stream) {
  using C = Cfg<TN, MODE, CL>;
  static bool configured[64] = {};
  int device = 0;
  MX_CUDA(cudaGetDevice(&device));
  if (device < 64 && !configured[device]) {
    MX_CUDA(cudaFuncSetAttribute(w6a8_gemm_kernel<TN, MODE, CL>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)C::kSmemBytes));
    configured[device] = true;
  }
  // Programmatic dependent launch: the prologue (barriers, tensor memory, tensor-map
  // prefetch) may run while the previous kernel on the stream drains; the kernel
  // itself waits (griddepcontrol.wait) before it touches global memory.
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((unsigned)plan.grid);
  config.blockDim = dim3(kThreads);
  config.dynamicSmemBytes = C::kSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  int count = 0;
  if (CL != 0) {
    attribute[count].id = cudaLaunchAttributeClusterDimension;
    attribute[count].val.clusterDim.x = (unsigned)plan.cluster_k;
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
  if (CL != 0) {
    // Never launch more clusters than can be resident: the persistent loop covers the rest.
    static int max_clusters[64][9] = {};
    if (device < 64 && max_clusters[device][plan.cluster_k] == 0) {
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, w6a8_gemm_kernel<TN, MODE, CL>, &config) !=
              cudaSuccess ||
          n < 1) {
        (void)cudaGetLastError();
        n = 1;
      }
      max_clusters[device][plan.cluster_k] = n;
    }
    const int resident = device < 64 ? max_clusters[device][plan.cluster_k] : 1;
    if (plan.grid / plan.cluster_k > resident) {
      config.gridDim = dim3((unsigned)(resident * plan.cluster_k));
    }
  }
  MX_CUDA(cudaLaunchKernelEx(&config, w6a8_gemm_kernel<TN, MODE, CL>, tm_w, tm_a, args));
  return kOk;
}

template <int TN, int MODE>
int launch_tn(const CUtensorMap& tm_w, const CUtensorMap& tm_a, const KernelArgs& args,
              const GemmPlan& plan, cudaStream_t stream) {
  if (plan.cluster_k > 1) {
    if constexpr (TN <= 96) {
      return launch_variant<TN, MODE, 1>(tm_w, tm_a, args, plan, stream);
    } else {
      set_error("tile_tokens %d cannot use cluster split-K", TN);
      return kInvalidArgument;
    }
  }
  return launch_variant<TN, MODE, 0>(tm_w, tm_a, args, plan, stream);
}

template <int TN, int MODE>
void fill_plan(GemmPlan* plan) {
  plan->stages = Cfg<TN, MODE, 0>::kStages;
  plan->smem_bytes = Cfg<TN, MODE, 0>::kSmemBytes;
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

// Cached 2-D tensor map (128-byte swizzle, 128-element inner box) for other
// translation units of the library.
int make_tensor_map_2d(CUtensorMap* out, int type, const void* base, uint64_t inner, uint64_t rows,
                       uint64_t stride, uint32_t box_rows) {
  return cached_map(out, (CUtensorMapDataType)type, base, inner, rows, stride, box_rows);
}

bool stream_kernel_applies(const GemmProblem& p);
int plan_w6a8_stream(const GemmProblem& p, int sms, GemmPlan* plan);
int launch_w6a8_stream(const GemmProblem& p, const GemmPlan& plan, cudaStream_t stream);
bool pair_kernel_applies(const GemmProblem& p, int tile_tokens);
int plan_w6a8_pair(const GemmProblem& p, int sms, GemmPlan* plan);
int launch_w6a8_pair(const GemmProblem& p, const GemmPlan& plan, cudaStream_t stream);
static int g_pair_mode = -1;  // -1: read MXFP6_B200_PAIR once; 0 off; 1 on
void set_cta_pair_mode(int enabled) { g_pair_mode = enabled != 0 ? 1 : 0; }
int cta_pair_mode() {
  if (g_pair_mode < 0) {
    const char* env = std::getenv("MXFP6_B200_PAIR");
    g_pair_mode = (env != nullptr && env[0] == '0') ? 0 : 1;
  }
  return g_pair_mode;
}

int plan_w6a8(const GemmProblem& p, GemmPlan* plan) {
  MX_REQUIRE(p.m_total > 0, "m must be positive; got %lld", (long long)p.m_total);
  MX_REQUIRE(p.m_total <= (int64_t)INT32_MAX - 1024, "m must fit 32 bits; got %lld",
             (long long)p.m_total);
  MX_REQUIRE(p.n > 0 && p.n % 8 == 0, "n must be a positive multiple of 8; got %d", p.n);
  MX_REQUIRE(p.k > 0 && p.k % 128 == 0, "k must be a positive multiple of 128; got %d", p.k);
  MX_REQUIRE(p.groups >= 1 && p.groups <= kMaxGroups, "groups must be in [1, %d]", kMaxGroups);
  MX_REQUIRE(p.groups == 1 || p.n % 128 == 0, "grouped weights need n %% 128 == 0");
  const bool grouped = p.expert_offsets != nullptr;
  if (p.force_kernel == kKernelStream) {
    MX_REQUIRE(stream_kernel_applies(p),
               "the weight-streaming kernel takes dense launches of at most 64 rows with "
               "tile_tokens 16, 32 or 64 and no scratch split");
    return plan_w6a8_stream(p, sm_count(), plan);
  }
  if (p.force_kernel == kKernelPair) {
    MX_REQUIRE(p.splits <= 1 && p.cluster_k <= 1 && pair_kernel_applies(p, p.tile_tokens),
               "the CTA-pair kernel takes dense launches with m > 128, n %% 128 == 0, n >= 256 and "
               "tile_tokens 128, 192 or 256");
    return plan_w6a8_pair(p, sm_count(), plan);
  }
  if (p.force_kernel < 0 && stream_kernel_mode() == 1 && stream_kernel_applies(p)) {
    if (int rc = plan_w6a8_stream(p, sm_count(), plan)) return rc;
    // 64-row tiles leave that kernel a ring of three stages: enough when a cluster shares a
    // tile, but a launch with a tile per CTA streams 3 % faster through the deep ring of
    // the persistent kernel (27.4 against 26.6 us at 64 x 34816 x 5120).
    if (!(plan->tile_tokens == 64 && plan->cluster_k == 1)) return kOk;
    *plan = GemmPlan{};
  }
  if (p.force_kernel < 0 && p.splits <= 1 && p.cluster_k <= 1 && cta_pair_mode() == 1 &&
      pair_kernel_applies(p, p.tile_tokens)) {
    return plan_w6a8_pair(p, sm_count(), plan);
  }
  int tn = p.tile_tokens;
  if (tn == 0) {
    // Rows per group that a tile should cover.
    const int64_t rows = grouped ? (p.m_total + p.groups - 1) / p.groups : p.m_total;
    if (grouped) {
      // Group sizes are device data; the mean is all the host knows.  A tile somewhat
      // wider than the mean lets most groups finish in one row tile (measured with 256
      // experts, top-8: 87 us at 192 against 117 us at 128 for a mean of 128 rows).
      tn = rows <= 48 ? 64 : rows <= 96 ? 128 : 192;
    } else if (rows <= 16) tn = 16;
    else if (rows <= 32) tn = 32;
    else if (rows <= 64) tn = 64;
    else if (rows <= 128) {
      // 65..128 rows: two 64-row tiles per feature tile (twice the tiles, double-buffered
      // accumulators, no or a smaller cluster reduce) beat one 96- or 128-row tile while the
      // weights, which are then read twice, stay in L2.  Measured at 96 rows: 12.0 against
      // 15.2 us at 7168 x 5120, 9.2 against 13.5 us at 2048 x 5120, 13.3 against 13.7 us at
      // 5120 x 6144; at 128 rows: 12.1 against 14.3, 10.5 against 14.1, 13.5 against 16.4 us.
      // 5120 x 17408 (67 MB of weights) and 34816 x 5120 (134 MB) keep the single tile.
      const int64_t weight_bytes = (int64_t)p.n * p.k / 4 * 3;
      const bool two_tiles = p.mode == kGemmStore && p.cluster_k <= 1 && p.splits <= 1 &&
                             weight_bytes <= (32ll << 20);
      tn = two_tiles ? 64 : (rows <= 96 ? 96 : 128);
    }
    else if (rows % 256 == 0 && p.k >= 12288) tn = 256;
    else tn = 192;
  }
  const bool swiglu = p.mode == kGemmSwigluMxfp8;
  if (swiglu) {
    MX_REQUIRE(p.n % 128 == 0, "SwiGLU mode needs the intermediate size to be a multiple of 128");
    MX_REQUIRE(p.splits <= 1, "SwiGLU mode does not split K");
    // Grouped: the SwiGLU epilogue of a 128-token tile has a single accumulator pair and
    // is not hidden by the next tile, 64-token tiles are double buffered: the narrow tile
    // wins up to a mean of about 100 rows per group (83 us against 95 us at 32 rows,
    // 155 us either way at 128, 537 us against 439 us at 512).
    if (grouped && p.tile_tokens == 0) {
      tn = (p.m_total + p.groups - 1) / p.groups <= 96 ? 64 : 128;
    }
    if (tn > 128) tn = 128;
    if (tn == 96) tn = 128;
    switch (tn) {
      case 16: fill_plan<16, kModeSwiglu>(plan); break;
      case 32: fill_plan<32, kModeSwiglu>(plan); break;
      case 64: fill_plan<64, kModeSwiglu>(plan); break;
      case 128: fill_plan<128, kModeSwiglu>(plan); break;
      default:
        set_error("unsupported tile_tokens %d for SwiGLU mode (use 16, 32, 64 or 128)", tn);
        return kInvalidArgument;
    }
  } else {
    switch (tn) {
      case 16: fill_plan<16, kModeStore>(plan); break;
      case 32: fill_plan<32, kModeStore>(plan); break;
      case 64: fill_plan<64, kModeStore>(plan); break;
      case 96: fill_plan<96, kModeStore>(plan); break;
      case 128: fill_plan<128, kModeStore>(plan); break;
      case 192: fill_plan<192, kModeStore>(plan); break;
      case 256: fill_plan<256, kModeStore>(plan); break;
      default:
        set_error("unsupported tile_tokens %d (use 16, 32, 64, 96, 128, 192 or 256)", tn);
        return kInvalidArgument;
    }
  }
  // The tensor-memory address of the activation scales must sit on an even
  // column, so tiles that start inside a 128-row scale atom need 64-row steps.
  MX_REQUIRE(!(grouped && (tn == 16 || tn == 32 || tn == 96)),
             "grouped launches need tile_tokens in {64, 128, 192, 256}");
  MX_REQUIRE(!((tn == 16 || tn == 32 || tn == 96) && p.m_total > tn),
             "tile_tokens %d needs m <= %d", tn, tn);
  plan->tile_tokens = tn;
  const int n_tiles = (p.n + kTileF - 1) / kTileF;
  const int k_blocks = p.k / kTileK;
  // Upper bound of row tiles: every group may add one ragged tile.
  const int64_t row_tiles =
      grouped ? (p.m_total / tn + (p.groups < p.m_total ? p.groups : p.m_total))
              : (p.m_total + tn - 1) / tn;
  const int64_t tiles = row_tiles * n_tiles;
  const int sms = sm_count();
  int splits = p.splits;
  int cluster_k = 1;
  const int mode = p.split_mode != 0 ? p.split_mode : default_split_mode();
  if (p.cluster_k > 1) {
    MX_REQUIRE(tn <= 96 && p.cluster_k <= 8 && p.cluster_k <= k_blocks && splits <= 1,
               "cluster_k needs tile_tokens <= 96, cluster_k <= min(8, k/128) and no scratch split");
    cluster_k = p.cluster_k;
    splits = 1;
  } else if (splits == 0) {
    splits = 1;
    if (tn <= 96 && tiles * 2 <= sms) {
      if (mode == 1) {
        // Leave a few SMs of slack: clusters need all their CTAs inside one GPC.
        int64_t ck = (sms - 16) / tiles;
        if (ck > 8) ck = 8;
        if (ck > k_blocks) ck = k_blocks;
        if (ck >= 2) cluster_k = (int)ck;
      } else if (mode == 2 && !grouped && !swiglu) {
        splits = (int)(sms / tiles);
        const int max_splits = k_blocks / 2 > 0 ? k_blocks / 2 : 1;
        if (splits > max_splits) splits = max_splits;
        if (splits > 16) splits = 16;
      }
    }
  }
  MX_REQUIRE(splits >= 1 && splits <= k_blocks, "splits must be in [1, k/128]");
  MX_REQUIRE(!(splits > 1 && (grouped || swiglu)),
             "scratch split-K is available for dense store-mode launches only");
  plan->splits = splits;
  plan->cluster_k = cluster_k;
  if (cluster_k > 1) {
    const int64_t clusters = tiles < sms / cluster_k ? tiles : sms / cluster_k;
    plan->grid = (int)(clusters < 1 ? 1 : clusters) * cluster_k;
  } else {
    const int64_t work = tiles * splits;
    plan->grid = (int)(work < sms ? work : sms);
    if (plan->grid < 1) plan->grid = 1;
  }
  plan->partial_bytes = splits > 1 ? (size_t)tiles * splits * tn * kTileF * sizeof(float) : 0;
  plan->counter_bytes = splits > 1 ? (size_t)tiles * sizeof(uint32_t) : 0;
  return kOk;
}

int launch_w6a8(const GemmProblem& p, const GemmPlan& plan, cudaStream_t stream) {
  MX_REQUIRE(p.w_values && p.w_scales && p.a_values && p.a_scales && p.out,
             "operand pointers must not be null");
  MX_REQUIRE((reinterpret_cast<uintptr_t>(p.w_values) & 31) == 0,
             "packed weight values must be 32-byte aligned");
  MX_REQUIRE((reinterpret_cast<uintptr_t>(p.a_values) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(p.w_scales) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(p.a_scales) & 15) == 0,
             "activation values and scale buffers must be 16-byte aligned");
  const bool swiglu = p.mode == kGemmSwigluMxfp8;
  MX_REQUIRE(swiglu || p.out_dtype == kBF16 || p.out_dtype == kF16,
             "out_dtype must be float16 or bfloat16");
  MX_REQUIRE((reinterpret_cast<uintptr_t>(p.out) & 15) == 0, "the output must be 16-byte aligned");
  MX_REQUIRE(p.out_scale_offsets == nullptr || p.out_scale_offsets == p.scale_offsets,
             "output scales of a grouped launch use the activation's scale_offsets");
  MX_REQUIRE(!swiglu || p.out_packed_scales != nullptr || p.out_logical_scales != nullptr,
             "SwiGLU mode needs a scale output");
  if (plan.splits > 1) {
    MX_REQUIRE(p.partials != nullptr && p.counters != nullptr &&
                   p.partial_bytes >= plan.partial_bytes && p.counter_bytes >= plan.counter_bytes,
               "split-K scratch is missing or too small (%zu + %zu bytes needed)",
               plan.partial_bytes, plan.counter_bytes);
  }
  if (plan.kernel == kKernelStream) return launch_w6a8_stream(p, plan, stream);
  if (plan.cta_pair != 0) return launch_w6a8_pair(p, plan, stream);
  int device = 0;
  MX_CUDA(cudaGetDevice(&device));
  CUtensorMap tm_w, tm_a;
  if (int rc = cached_map(&tm_w, CU_TENSOR_MAP_DATA_TYPE_16U6_ALIGN16B, p.w_values,
                          (uint64_t)p.k, (uint64_t)p.groups * p.n * (swiglu ? 2 : 1),
                          (uint64_t)p.k * 3 / 4, kTileF))
    return rc;
  if (int rc = cached_map(&tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.a_values, (uint64_t)p.k,
                          (uint64_t)p.m_total, (uint64_t)p.k, (uint32_t)plan.tile_tokens))
    return rc;
  KernelArgs args;
  args.w_scales = p.w_scales;
  args.a_scales = p.a_scales;
  args.expert_offsets = p.expert_offsets;
  args.scale_offsets = p.scale_offsets;
  args.out = p.out;
  args.partials = p.partials;
  args.counters = p.counters;
  args.status = p.status_word != nullptr ? p.status_word : device_status_word(device);
  if (args.status == nullptr) return kCudaError;
  args.m_total = p.m_total;
  args.groups = p.groups;
  args.n = p.n;
  args.w_rows_per_group = p.n * (swiglu ? 2 : 1);
  args.out_packed_scales = p.out_packed_scales;
  args.out_logical_scales = p.out_logical_scales;
  args.out_scale_offsets = p.out_scale_offsets;
  args.k_blocks = p.k / kTileK;
  args.n_tiles = (p.n + kTileF - 1) / kTileF;
  args.splits = plan.cluster_k > 1 ? plan.cluster_k : plan.splits;
  args.cluster_k = plan.cluster_k;
  args.out_dtype = p.out_dtype;
  args.alpha = p.alpha;
  args.silu_lut = nullptr;
  if (swiglu) {
    if (int rc = silu_table(stream, &args.silu_lut)) return rc;
  }
  {
    const int64_t scale_rows = p.a_scale_rows > 0 ? p.a_scale_rows : round_up64(p.m_total, kAtomRows);
    args.a_scale_row_blocks = (int)(scale_rows / kAtomRows);
  }
  if (swiglu) {
    switch (plan.tile_tokens) {
      case 16: return launch_tn<16, kModeSwiglu>(tm_w, tm_a, args, plan, stream);
      case 32: return launch_tn<32, kModeSwiglu>(tm_w, tm_a, args, plan, stream);
      case 64: return launch_tn<64, kModeSwiglu>(tm_w, tm_a, args, plan, stream);
      case 128: return launch_tn<128, kModeSwiglu>(tm_w, tm_a, args, plan, stream);
    }
  } else {
    switch (plan.tile_tokens) {
      case 16: return launch_tn<16, kModeStore>(tm_w, tm_a, args, plan, stream);
      case 32: return launch_tn<32, kModeStore>(tm_w, tm_a, args, plan, stream);
      case 64: return launch_tn<64, kModeStore>(tm_w, tm_a, args, plan, stream);
      case 96: return launch_tn<96, kModeStore>(tm_w, tm_a, args, plan, stream);
      case 128: return launch_tn<128, kModeStore>(tm_w, tm_a, args, plan, stream);
      case 192: return launch_tn<192, kModeStore>(tm_w, tm_a, args, plan, stream);
      case 256: return launch_tn<256, kModeStore>(tm_w, tm_a, args, plan, stream);
    }
  }
  set_error("unsupported tile_tokens %d", plan.tile_tokens);
  return kInvalidArgument;
}

void set_default_split_mode(int mode) { g_split_mode = (mode >= 1 && mode <= 3) ? mode : 1; }
int default_split_mode() { return g_split_mode; }

// One status word per device, allocated on first use and never freed.
namespace {
std::mutex g_status_mutex;
int* g_status_words[64] = {};
}  // namespace

int* device_status_word(int device) {
  std::mutex& mutex = g_status_mutex;
  int** words = g_status_words;
  if (device < 0 || device >= 64) {
    set_error("device index %d out of range", device);
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mutex);
  if (words[device] == nullptr) {
    int* ptr = nullptr;
    if (cudaMalloc(&ptr, sizeof(int)) != cudaSuccess || cudaMemset(ptr, 0, sizeof(int)) != cudaSuccess) {
      set_error("could not allocate the device status word");
      return nullptr;
    }
    words[device] = ptr;
  }
  return words[device];
}

// ---- GEMM without allocations ------------------------------------------------------
// Some callers may not allocate device memory at all: code that runs while a CUDA
// graph is being captured by an outer framework, a serving process whose memory
// pool was sized and frozen at start-up, or a plugin that is forbidden to touch
// the allocator of its host.  For them the split-K scratch (FP32 partial tiles,
// tile counters) and the status word of one GEMM live in this fixed array, which
// every GPU that loads the library holds until the process exits.
constexpr size_t kStaticPartialBytes = size_t(4) << 20;  // FP32 partial tiles
constexpr size_t kStaticCounterBytes = 4096;             // one counter per output tile
constexpr size_t kStaticStatusBytes = 256;
static __device__ __align__(256) unsigned char
    g_static_scratch[kStaticPartialBytes + kStaticCounterBytes + kStaticStatusBytes];

namespace {
std::mutex g_static_mutex;
unsigned char* g_static_base[64] = {};  // device address of g_static_scratch, per device

// In host code `g_static_scratch` only names the symbol; its device address has to
// be asked for, once per device, with that device current.
int static_scratch_base(int device, unsigned char** base) {
  if (device < 0 || device >= 64) {
    set_error("device index %d out of range", device);
    return kInvalidArgument;
  }
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_base[device] == nullptr) {
    unsigned char* ptr = nullptr;
    MX_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_scratch));
    g_static_base[device] = ptr;
  }
  *base = g_static_base[device];
  return kOk;
}
}  // namespace

int launch_w6a8_static_scratch(GemmProblem& p, cudaStream_t stream) {
  int device = 0;
  MX_CUDA(cudaGetDevice(&device));
  unsigned char* base = nullptr;
  if (int rc = static_scratch_base(device, &base)) return rc;
  p.split_mode = 2;  // this entry point exists for the scratch-based split
  GemmPlan plan;
  if (int rc = plan_w6a8(p, &plan)) return rc;
  if (plan.splits > 1) {
    if (plan.partial_bytes > kStaticPartialBytes || plan.counter_bytes > kStaticCounterBytes) {
      set_error(
          "this problem needs %zu + %zu bytes of split-K scratch; the built-in array holds "
          "%zu + %zu. Use mxfp6_gemm_w6a8 or mxfp6_gemm_w6a8_ex with caller-owned scratch",
          plan.partial_bytes, plan.counter_bytes, kStaticPartialBytes, kStaticCounterBytes);
      return kInvalidArgument;
    }
    p.partials = reinterpret_cast<float*>(base);
    p.partial_bytes = kStaticPartialBytes;
    p.counters = reinterpret_cast<uint32_t*>(base + kStaticPartialBytes);
    p.counter_bytes = kStaticCounterBytes;
    // The array keeps whatever the previous call left; the tile counters must start at zero.
    MX_CUDA(cudaMemsetAsync(p.counters, 0, plan.counter_bytes, stream));
  }
  p.status_word = reinterpret_cast<int*>(base + kStaticPartialBytes + kStaticCounterBytes);
  return launch_w6a8(p, plan, stream);
}

int read_device_status(int device, int* value, bool reset) {
  if (device < 0 || device >= 64) {
    set_error("device index %d out of range", device);
    return kInvalidArgument;
  }
  // Reading never allocates: a device whose ordinary status word does not exist yet has
  // launched no kernel that could have set it.
  int* word = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_status_mutex);
    word = g_status_words[device];
  }
  MX_CUDA(cudaDeviceSynchronize());
  *value = 0;
  if (word != nullptr) {
    MX_CUDA(cudaMemcpy(value, word, sizeof(int), cudaMemcpyDeviceToHost));
    if (reset && *value != 0) MX_CUDA(cudaMemset(word, 0, sizeof(int)));
  }
  // Fold in the status word of the allocation-free entry point, if it was used here.
  unsigned char* base = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (device >= 0 && device < 64) base = g_static_base[device];
  }
  if (base != nullptr) {
    int extra = 0;
    int* extra_word = reinterpret_cast<int*>(base + kStaticPartialBytes + kStaticCounterBytes);
    MX_CUDA(cudaMemcpy(&extra, extra_word, sizeof(int), cudaMemcpyDeviceToHost));
    if (reset && extra != 0) MX_CUDA(cudaMemset(extra_word, 0, sizeof(int)));
    if (*value == 0) *value = extra;
  }
  return kOk;
}

}  // namespace mx
