// CTA-pair variant of the dense W6A8 GEMM for large M (prefill).
//
// Two CTAs of a cluster compute one 256-feature x TN-token tile with
// tcgen05.mma.cta_group::2: each CTA loads its own 128 weight rows and only HALF of
// the activation tile (TN / 2 rows); the MMA reads operand B from both CTAs' shared
// memory.  Per 128-K block a CTA therefore pulls 12 KB of weights + TN/2 x 128 bytes
// of activations from L2 instead of TN x 128, which is what bounded the single-CTA
// kernel at large M (its 5-stage ring delivered a block per ~580 cycles against ~390
// cycles of MMA work).  Every CTA issues its own loads; no load is shared between CTAs.
//
// Roles per CTA (320 threads): warp 0 TMA producer; warp 1 MMA issuer in the leader CTA
// (rank 0), idle in the peer; warps 2..9 epilogue, two per tensor-memory lane quarter.
// Barriers live at the same shared-memory offsets in both CTAs; tcgen05.commit with
// a CTA mask releases stages and publishes accumulators in both at once.
// Every wait is bounded, as in the single-CTA kernel.
#include "gemm.cuh"
#include "ptx.cuh"

#include <cuda.h>

namespace mx {
namespace {

constexpr int kTileF = 128;
constexpr int kTileK = 128;
constexpr int kMmaK = 32;
constexpr int kEpiWarps = 8;                  // two per tensor-memory lane quarter
constexpr int kThreads = 64 + 32 * kEpiWarps;  // producer warp, MMA warp, epilogue warps
constexpr uint32_t kWTileBytes = kTileF * kTileK;
constexpr uint32_t kWTileTxBytes = kWTileBytes / 4 * 3;
constexpr uint32_t kAtomBytes = 512;
constexpr long long kWaitCycles = 4000000000ll;

struct PairArgs {
  const uint8_t* w_scales;
  const uint8_t* a_scales;
  void* out;
  int* status;
  int64_t m;
  int n;
  int k_blocks;
  int n_pair_tiles;  // ceil(n / 256); with n % 256 == 128 the peer half of the last pair is empty
  int out_dtype;
  float alpha;
  int a_scale_row_blocks;
  // Grouped launches: rows [expert_offsets[g], expert_offsets[g + 1]) use weight rows
  // [g * n, (g + 1) * n) and packed scale rows from scale_offsets[g]; null = dense.
  const int64_t* expert_offsets;
  const int64_t* scale_offsets;
  int groups;
};

constexpr int kPairMaxGroups = 512;

struct PairWork {
  int group, n_pair, rows;
  int64_t row0;        // first activation row of the tile
  int64_t scale_row0;  // packed-scale row of row0
};

// tile_prefix[g] = row tiles of groups < g; row_begin / scale_begin follow at a stride of
// kPairMaxGroups + 1 ints.  Tiles of one group are adjacent, row tile fastest.
template <int TN>
__device__ __forceinline__ bool pair_decode(int t, const PairArgs& a, const int* tile_prefix,
                                            PairWork* out) {
  const int total = tile_prefix[a.groups] * a.n_pair_tiles;
  if (t >= total) return false;
  int lo = 0, hi = a.groups;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (tile_prefix[mid] * a.n_pair_tiles <= t) lo = mid; else hi = mid;
  }
  while (lo + 1 < a.groups && tile_prefix[lo + 1] * a.n_pair_tiles <= t) ++lo;  // empty groups
  const int local = t - tile_prefix[lo] * a.n_pair_tiles;
  const int mt = tile_prefix[lo + 1] - tile_prefix[lo];
  const int n_pair = mt == 1 ? local : local / mt;  // one row tile per group is the common case
  const int m_tile = local - n_pair * mt;
  const int* row_begin = tile_prefix + (kPairMaxGroups + 1);
  const int* scale_begin = row_begin + (kPairMaxGroups + 1);
  out->group = lo;
  out->n_pair = n_pair;
  out->row0 = (int64_t)row_begin[lo] + (int64_t)m_tile * TN;
  const int64_t left = (int64_t)row_begin[lo + 1] - out->row0;
  out->rows = left < TN ? (int)left : TN;
  out->scale_row0 = (int64_t)scale_begin[lo] + (int64_t)m_tile * TN;
  return true;
}

template <int TN>
struct PairCfg {
  static constexpr int kHalf = TN / 2;                       // activation rows per CTA
  static constexpr int kSfbAtoms = TN <= 128 ? 1 : 2;
  static constexpr int kSfSets = 4;
  static constexpr int kSfSetCols = 4 + 4 * kSfbAtoms;
  static constexpr int kAcc = (2 * TN + kSfSets * kSfSetCols <= 512) ? 2 : 1;
  static constexpr int kSfaCol = kAcc * TN;
  static constexpr int kSfbCol = kSfaCol + 4;
  static constexpr int kColsUsed = kSfaCol + kSfSets * kSfSetCols;
  static_assert(kColsUsed <= 512, "tile does not fit tensor memory");
  static constexpr int kTmemCols = kColsUsed <= 256 ? 256 : 512;
  static constexpr uint32_t kATileBytes = kHalf * kTileK;
  static constexpr uint32_t kStageBytes = kWTileBytes + kATileBytes;
  static constexpr uint32_t kSfStageBytes = kAtomBytes * (1 + kSfbAtoms);
  static constexpr uint32_t kEpiWarpBytes = 2048;
  // align slack, barriers, three group tables, epilogue staging
  static constexpr uint32_t kTableBytes = 3 * (512 + 1) * 4 + 4;
  static constexpr uint32_t kFixedBytes =
      1024 + 1024 + kEpiWarps * kEpiWarpBytes + ((kTableBytes + 127) / 128) * 128;
  static constexpr int kStagesRaw = (int)((232448u - kFixedBytes) / (kStageBytes + kSfStageBytes));
  static constexpr int kStages = kStagesRaw > 10 ? 10 : kStagesRaw;
  static constexpr size_t kSmemBytes = kFixedBytes + (size_t)kStages * (kStageBytes + kSfStageBytes);
};

__device__ __forceinline__ bool pair_wait(uint32_t bar, uint32_t parity, volatile int* abort,
                                          int* status, int code) {
  if (ptx::mbar_try_wait_cluster(bar, parity)) return true;
  const long long start = clock64();
#pragma unroll 1
  for (uint32_t spin = 0;; ++spin) {
    if (ptx::mbar_try_wait_cluster(bar, parity)) return true;
    if ((spin & 63u) == 63u) {
      if (*abort != 0) return false;
      if (clock64() - start > kWaitCycles) {
        *abort = 1;
        atomicCAS(status, 0, code);
        return false;
      }
    }
  }
}

template <int TN>
__global__ void __launch_bounds__(kThreads, 1)
w6a8_gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_w,
                      const __grid_constant__ CUtensorMap tm_a,
                      const __grid_constant__ CUtensorMap tm_ws,
                      const __grid_constant__ CUtensorMap tm_as, const PairArgs args) {
  using C = PairCfg<TN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* w_tiles = smem;
  uint8_t* a_tiles = w_tiles + (size_t)C::kStages * kWTileBytes;
  uint8_t* sf_tiles = a_tiles + (size_t)C::kStages * C::kATileBytes;
  uint8_t* fixed = sf_tiles + (size_t)C::kStages * C::kSfStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(fixed);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(fixed + 8 * (2 * C::kStages + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* epi_stage = fixed + 1024;
  int* tile_prefix = reinterpret_cast<int*>(fixed + 1024 + kEpiWarps * C::kEpiWarpBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();  // 0 = leader
  const uint32_t full0 = ptx::smem_u32(bars);
  const uint32_t empty0 = full0 + 8 * C::kStages;
  const uint32_t tfull0 = empty0 + 8 * C::kStages;
  const uint32_t tempty0 = tfull0 + 16;                   // leader only: both epilogues done

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < C::kStages; ++s) {
      ptx::mbar_init(full0 + 8 * s, 1);
      ptx::mbar_init(empty0 + 8 * s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(tfull0 + 8 * i, 1);
      ptx::mbar_init(tempty0 + 8 * i, 2 * kEpiWarps);
    }
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tm_w);
    ptx::prefetch_tensormap(&tm_a);
    ptx::prefetch_tensormap(&tm_ws);
    ptx::prefetch_tensormap(&tm_as);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(ptx::smem_u32(tmem_slot), C::kTmemCols);
    ptx::tmem_relinquish_pair();
  }
  ptx::grid_dependency_wait();
  ptx::grid_launch_dependents();
  {
    int* row_begin_tab = tile_prefix + (kPairMaxGroups + 1);
    int* scale_begin_tab = row_begin_tab + (kPairMaxGroups + 1);
    if (args.expert_offsets == nullptr) {
      if (threadIdx.x == 0) {
        tile_prefix[0] = 0;
        tile_prefix[1] = (int)((args.m + TN - 1) / TN);
        row_begin_tab[0] = 0;
        row_begin_tab[1] = (int)args.m;
        scale_begin_tab[0] = 0;
      }
    } else {
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
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  ptx::cluster_sync_all();  // both CTAs' barriers are initialised

  const int pair = blockIdx.x >> 1;
  const int pairs = gridDim.x >> 1;
  const int kb_total = args.k_blocks;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    // Every load of either CTA completes its bytes on the LEADER's full barrier, so the
    // MMA issuer waits on one barrier per stage; a CTA reuses a stage of its own shared
    // memory once the leader's commit has reached its local empty barrier.
    int stage = 0;
    uint32_t phase = 0;
    constexpr uint32_t kTxPerCta = kWTileTxBytes + C::kATileBytes + kAtomBytes * (1 + C::kSfbAtoms);
    const uint32_t leader_full0 = ptx::mapa(full0, 0u);
    bool ok = true;
    PairWork wk;
    for (int t = pair; ok && pair_decode<TN>(t, args, tile_prefix, &wk); t += pairs) {
      const int w_row = wk.group * args.n + wk.n_pair * 2 * kTileF + (int)rank * kTileF;
      const int a_row = (int)(wk.row0 + rank * C::kHalf);
      const int sfb_rb0 = (int)(wk.scale_row0 / kAtomRows);
      const int sfa_atom0 = (w_row / kAtomRows) * kb_total;
      for (int kb = 0; kb < kb_total; ++kb) {
        ok = __all_sync(0xffffffffu,
                        pair_wait(empty0 + 8 * stage, phase ^ 1u, abort_flag, args.status, 201));
        if (!ok) break;
        if (ptx::elect_one()) {
          const uint32_t bar = leader_full0 + 8 * stage;
          if (rank == 0) ptx::mbar_arrive_expect_tx(full0 + 8 * stage, 2 * kTxPerCta);
          ptx::tma_load_2d_pair(ptx::smem_u32(w_tiles + (size_t)stage * kWTileBytes), &tm_w,
                                kb * kTileK, w_row, bar);
          ptx::tma_load_2d_pair(ptx::smem_u32(a_tiles + (size_t)stage * C::kATileBytes), &tm_a,
                                kb * kTileK, a_row, bar);
          const uint32_t sf = ptx::smem_u32(sf_tiles + (size_t)stage * C::kSfStageBytes);
          ptx::tma_load_2d_pair(sf, &tm_ws, 0, sfa_atom0 + kb, bar);
#pragma unroll
          for (int j = 0; j < C::kSfbAtoms; ++j) {
            int rb = sfb_rb0 + j;
            if (rb >= args.a_scale_row_blocks) rb = args.a_scale_row_blocks - 1;
            ptx::tma_load_2d_pair(sf + kAtomBytes * (1 + j), &tm_as, 0, rb * kb_total + kb, bar);
          }
        }
        __syncwarp();
        if (++stage == C::kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1 && rank == 0) {
    // ---------------- leader: MMA issuer for the pair ----------------
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    uint32_t sf_set = 0;
    // E3M2 x E4M3, K-major, UE8M0 scales, M = 256 over the pair, N = TN.
    constexpr uint32_t kIdesc = (4u << 7) | (0u << 10) | ((uint32_t)(TN >> 3) << 17) | (1u << 23) |
                                ((uint32_t)(256 >> 4) << 24);
    bool ok = true;
    // The poll of the next stage's barrier is issued before the commit of this one, so
    // its latency overlaps the commit.
    bool ready = false;
    PairWork wk;
    for (int t = pair; ok && pair_decode<TN>(t, args, tile_prefix, &wk); t += pairs) {
      const uint32_t sfb_sub = (uint32_t)((wk.scale_row0 % kAtomRows) / 32);
      if (!__all_sync(0xffffffffu, pair_wait(tempty0 + 8 * acc, acc_phase ^ 1u, abort_flag,
                                             args.status, 203)))
        break;
      ptx::tc_fence_after();
      const uint32_t d_t = tmem_base + acc * TN;
      for (int kb = 0; kb < kb_total; ++kb) {
        if (!ready) {
          ok = __all_sync(0xffffffffu,
                          pair_wait(full0 + 8 * stage, phase, abort_flag, args.status, 204));
          if (!ok) break;
        }
        ptx::tc_fence_after();
        const bool leader_lane = ptx::elect_one();
        if (leader_lane) {
          const uint32_t sf = ptx::smem_u32(sf_tiles + (size_t)stage * C::kSfStageBytes);
          const uint32_t sfa_t = tmem_base + C::kSfaCol + sf_set * C::kSfSetCols;
          const uint32_t sfb_base = tmem_base + C::kSfbCol + sf_set * C::kSfSetCols;
          ptx::tc_cp_32x128b_warpx4_pair(sfa_t, ptx::smem_desc_scale_atom(sf));
#pragma unroll
          for (int j = 0; j < C::kSfbAtoms; ++j) {
            ptx::tc_cp_32x128b_warpx4_pair(sfb_base + 4 * j,
                                           ptx::smem_desc_scale_atom(sf + kAtomBytes * (1 + j)));
          }
          const uint64_t a_desc =
              ptx::smem_desc_sw128(ptx::smem_u32(w_tiles + (size_t)stage * kWTileBytes));
          const uint64_t b_desc =
              ptx::smem_desc_sw128(ptx::smem_u32(a_tiles + (size_t)stage * C::kATileBytes));
#pragma unroll
          for (int ks = 0; ks < kTileK / kMmaK; ++ks) {
            const uint32_t idesc = kIdesc | ((uint32_t)ks << 4) | ((uint32_t)ks << 29);
            ptx::tc_mma_mxf8f6f4_pair(d_t, a_desc + 2 * ks, b_desc + 2 * ks, idesc, sfa_t,
                                      sfb_base + sfb_sub, (kb > 0 || ks > 0) ? 1u : 0u);
          }
        }
        sf_set = (sf_set + 1u) % C::kSfSets;
        const int used = stage;
        if (++stage == C::kStages) {
          stage = 0;
          phase ^= 1u;
        }
        ready = ptx::mbar_test_wait_cluster(full0 + 8 * stage, phase);
        if (leader_lane) ptx::tc_commit_pair(empty0 + 8 * used, 3);  // stage free in both CTAs
        ready = __all_sync(0xffffffffu, ready);
      }
      if (!ok) break;
      if (ptx::elect_one()) ptx::tc_commit_pair(tfull0 + 8 * acc, 3);  // accumulators ready in both
      __syncwarp();
      if (++acc == C::kAcc) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
  } else if (warp >= 2) {
    // ---------------- epilogue (warps 2..9 of both CTAs) ----------------
    // A warp reads the tensor-memory lanes of quarter warp % 4; the two warps of a quarter
    // take alternate 32-column chunks.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    int acc = 0;
    uint32_t acc_phase = 0;
    uint16_t* stage16 = reinterpret_cast<uint16_t*>(epi_stage + (warp - 2) * C::kEpiWarpBytes);
    const bool bf16_out = args.out_dtype == kBF16;
    PairWork wk;
    for (int t = pair; pair_decode<TN>(t, args, tile_prefix, &wk); t += pairs) {
      const int n_pair = wk.n_pair;
      const int64_t row0 = wk.row0;
      const int rows = wk.rows;
      if (!pair_wait(tfull0 + 8 * acc, acc_phase, abort_flag, args.status, 206)) break;
      ptx::tc_fence_after();
      const uint32_t t_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * TN;
      const int f0 = n_pair * 2 * kTileF + (int)rank * kTileF + quarter * 32;
#pragma unroll 1
      for (int c0 = 32 * half; c0 < rows; c0 += 32 * (kEpiWarps / 4)) {
        uint32_t r[32];
        ptx::tmem_ld_x32(t_addr + c0, r);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float v = args.alpha * __uint_as_float(r[j]);
          stage16[j * 32 + lane] = bf16_out ? __bfloat16_as_ushort(__float2bfloat16_rn(v))
                                            : __half_as_ushort(__float2half_rn(v));
        }
        __syncwarp();
        const int seg = lane & 3;
        const int fseg = f0 + seg * 8;
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) {
          const int rr = (lane >> 2) + 8 * pass;
          const int tr = c0 + rr;
          if (tr < rows && fseg < args.n) {
            const uint4 v = *reinterpret_cast<const uint4*>(stage16 + rr * 32 + seg * 8);
            *reinterpret_cast<uint4*>(static_cast<uint16_t*>(args.out) + (row0 + tr) * args.n +
                                      fseg) = v;
          }
        }
        __syncwarp();
      }
      ptx::tc_fence_before();
      __syncwarp();
      // The leader's MMA warp may reuse the buffer once the epilogue warps of both CTAs are done.
      if (lane == 0) ptx::mbar_arrive_remote_relaxed(ptx::mapa(tempty0 + 8 * acc, 0u));
      if (++acc == C::kAcc) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
  }

  // ---------------- teardown ----------------
  ptx::tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  // Neither CTA may leave while its peer can still signal barriers in its shared memory
  // or run MMAs that read it.
  ptx::cluster_sync_all();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem_base, C::kTmemCols);
  }
}

template <int TN>
int launch_pair_tn(const CUtensorMap& tm_w, const CUtensorMap& tm_a, const CUtensorMap& tm_ws,
                   const CUtensorMap& tm_as, const PairArgs& args, int pairs, cudaStream_t stream) {
  using C = PairCfg<TN>;
  static bool configured[64] = {};
  int device = 0;
  MX_CUDA(cudaGetDevice(&device));
  if (device < 64 && !configured[device]) {
    MX_CUDA(cudaFuncSetAttribute(w6a8_gemm_pair_kernel<TN>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::kSmemBytes));
    configured[device] = true;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((unsigned)(2 * pairs));
  config.blockDim = dim3(kThreads);
  config.dynamicSmemBytes = C::kSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = 2;
  attribute[0].val.clusterDim.y = 1;
  attribute[0].val.clusterDim.z = 1;
  attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 2;
  static int max_clusters[64] = {};
  if (device < 64 && max_clusters[device] == 0) {
    int fit = 0;
    MX_CUDA(cudaOccupancyMaxActiveClusters(&fit, w6a8_gemm_pair_kernel<TN>, &config));
    max_clusters[device] = fit > 0 ? fit : 1;
  }
  if (device < 64 && pairs > max_clusters[device]) {
    config.gridDim = dim3((unsigned)(2 * max_clusters[device]));
  }
  MX_CUDA(cudaLaunchKernelEx(&config, w6a8_gemm_pair_kernel<TN>, tm_w, tm_a, tm_ws, tm_as, args));
  return kOk;
}

}  // namespace

int make_tensor_map_2d(CUtensorMap* out, int type, const void* base, uint64_t inner, uint64_t rows,
                       uint64_t stride, uint32_t box_rows);

// tile_tokens 0 lets the planner choose among 128, 192 and 256.  Grouped launches
// qualify when the mean group is large enough for those tiles.
bool pair_kernel_applies(const GemmProblem& p, int tile_tokens) {
  // n % 256 == 128: the peer CTA of the last pair loads out-of-range (zero-filled or
  // foreign) weight rows and stores nothing.
  if (p.mode != kGemmStore || p.n % 128 != 0 || p.n < 256) return false;
  if (!(tile_tokens == 0 || tile_tokens == 128 || tile_tokens == 192 || tile_tokens == 256))
    return false;
  if (p.expert_offsets != nullptr) {
    if (p.groups < 1 || p.groups > kPairMaxGroups || p.scale_offsets == nullptr) return false;
    return tile_tokens != 0 || p.m_total > (int64_t)48 * p.groups;
  }
  return p.groups == 1 && p.m_total > 128;
}

namespace {
template <int TN>
void fill_pair_plan(GemmPlan* plan) {
  plan->tile_tokens = TN;
  plan->stages = PairCfg<TN>::kStages;
  plan->smem_bytes = PairCfg<TN>::kSmemBytes;
}
}  // namespace

int plan_w6a8_pair(const GemmProblem& p, int sms, GemmPlan* plan) {
  const int pairs = sms / 2 > 0 ? sms / 2 : 1;
  const int64_t n_pairs = (p.n + 255) / 256;
  const int64_t k_blocks = p.k / kTileK;
  const bool grouped = p.expert_offsets != nullptr;
  int tn = p.tile_tokens;
  if (tn == 0 && grouped) {
    // Group sizes are device data; a tile somewhat wider than the mean group lets most
    // groups finish in one row tile.
    tn = p.m_total <= (int64_t)96 * p.groups ? 128 : 192;
  }
  if (tn == 0) {
    // Cycles one CTA pair spends: per 128-K block the slower of the MMA (2 cycles per
    // token column) and the issue loop; the 256-token tile has a single accumulator, so
    // its epilogue is not hidden behind the next tile.  Waves of tiles over the pairs
    // decide the rest.
    const int candidates[3] = {128, 192, 256};
    const int64_t block_cycles[3] = {400, 410, 530};
    const int64_t exposed_epilogue[3] = {0, 0, 3000};
    int64_t best = 0;
    for (int i = 0; i < 3; ++i) {
      const int64_t tiles = ((p.m_total + candidates[i] - 1) / candidates[i]) * n_pairs;
      const int64_t waves = (tiles + pairs - 1) / pairs;
      const int64_t cost = waves * (k_blocks * block_cycles[i] + exposed_epilogue[i]);
      if (tn == 0 || cost < best) {
        best = cost;
        tn = candidates[i];
      }
    }
  }
  switch (tn) {
    case 128: fill_pair_plan<128>(plan); break;
    case 192: fill_pair_plan<192>(plan); break;
    case 256: fill_pair_plan<256>(plan); break;
    default: set_error("the CTA-pair kernel takes tile_tokens 128, 192 or 256"); return kInvalidArgument;
  }
  // Grouped: every group may add one ragged row tile.
  const int64_t row_tiles = grouped ? p.m_total / tn + (p.groups < p.m_total ? p.groups : p.m_total)
                                    : (p.m_total + tn - 1) / tn;
  const int64_t tiles = row_tiles * n_pairs;
  plan->splits = 1;
  plan->cluster_k = 1;
  plan->cta_pair = 1;
  plan->kernel = kKernelPair;
  plan->grid = 2 * (int)(tiles < pairs ? tiles : pairs);
  plan->partial_bytes = 0;
  plan->counter_bytes = 0;
  return kOk;
}

int launch_w6a8_pair(const GemmProblem& p, const GemmPlan& plan, cudaStream_t stream) {
  const int tile_tokens = plan.tile_tokens;
  MX_REQUIRE(plan.cta_pair != 0 && pair_kernel_applies(p, tile_tokens),
             "the CTA-pair kernel does not cover this problem");
  int device = 0;
  MX_CUDA(cudaGetDevice(&device));
  CUtensorMap tm_w, tm_a, tm_ws, tm_as;
  if (int rc = make_tensor_map_2d(&tm_w, (int)CU_TENSOR_MAP_DATA_TYPE_16U6_ALIGN16B, p.w_values,
                                  (uint64_t)p.k, (uint64_t)p.groups * p.n, (uint64_t)p.k * 3 / 4,
                                  kTileF))
    return rc;
  if (int rc = make_tensor_map_2d(&tm_a, (int)CU_TENSOR_MAP_DATA_TYPE_UINT8, p.a_values,
                                  (uint64_t)p.k, (uint64_t)p.m_total, (uint64_t)p.k,
                                  (uint32_t)(tile_tokens / 2)))
    return rc;
  const int64_t scale_rows = p.a_scale_rows > 0 ? p.a_scale_rows : round_up64(p.m_total, kAtomRows);
  const uint64_t k_blocks = (uint64_t)(p.k / kTileK);
  if (int rc = make_tensor_map_2d(&tm_ws, (int)CU_TENSOR_MAP_DATA_TYPE_UINT32, p.w_scales, 128,
                                  (uint64_t)p.groups * (p.n / kAtomRows) * k_blocks, kAtomBytes,
                                  1))
    return rc;
  if (int rc = make_tensor_map_2d(&tm_as, (int)CU_TENSOR_MAP_DATA_TYPE_UINT32, p.a_scales, 128,
                                  (uint64_t)(scale_rows / kAtomRows) * k_blocks, kAtomBytes, 1))
    return rc;
  PairArgs args;
  args.w_scales = p.w_scales;
  args.a_scales = p.a_scales;
  args.out = p.out;
  args.status = p.status_word != nullptr ? p.status_word : device_status_word(device);
  if (args.status == nullptr) return kCudaError;
  args.m = p.m_total;
  args.n = p.n;
  args.k_blocks = p.k / kTileK;
  args.n_pair_tiles = (p.n + 255) / 256;
  args.out_dtype = p.out_dtype;
  args.alpha = p.alpha;
  args.a_scale_row_blocks = (int)(scale_rows / kAtomRows);
  args.expert_offsets = p.expert_offsets;
  args.scale_offsets = p.scale_offsets;
  args.groups = p.expert_offsets != nullptr ? p.groups : 1;
  const int pairs = plan.grid / 2;
  switch (tile_tokens) {
    case 128: return launch_pair_tn<128>(tm_w, tm_a, tm_ws, tm_as, args, pairs, stream);
    case 192: return launch_pair_tn<192>(tm_w, tm_a, tm_ws, tm_as, args, pairs, stream);
    case 256: return launch_pair_tn<256>(tm_w, tm_a, tm_ws, tm_as, args, pairs, stream);
  }
  return kInvalidArgument;
}

}  // namespace mx
