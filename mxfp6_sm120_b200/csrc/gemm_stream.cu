// Weight-streaming W6A8 GEMM for decode batches: dense, m <= 64, FP16/BF16 output.
//
// The reference serves this regime with its swapped-AB CUTLASS SM120 kernels and the
// per-M dispatch tables (csrc/include/mxfp6_gemm/kernel_swapped.hpp:98-317,
// csrc/torch_extension.cu:1203-1461); every launch there is a programmatic dependent
// launch of the activation quantizer (csrc/quantization.cu:184-190).
//
// A decode GEMM reads its whole weight matrix once and does almost no arithmetic, so
// the time of a launch is the HBM stream plus whatever cannot overlap it: prologue,
// first-byte latency, split-K reduction, exit.  This kernel is built so that those
// overlap the NEIGHBOURING launches instead:
//   * a CTA needs under half of an SM's shared memory and a quarter of its tensor
//     memory, so the CTAs of the next launch become resident beside the running ones;
//   * griddepcontrol.launch_dependents is the first instruction, and the producer warp
//     fills its whole shared-memory ring with WEIGHT tiles and weight scales before
//     griddepcontrol.wait: weights never depend on the previous kernel, activations
//     and the output do.  After the wait only the small activation tiles (L2 hits) are
//     added to the armed barriers and the MMAs start on a full ring;
//   * two warps issue the MMAs, taking alternate ring stages into an accumulator each.
//     One issuing warp needs about 260 ns per 128-K block of a 16-row tile (barrier
//     wait, fence, two scale copies, four tcgen05.mma whose issue blocks on the pipe,
//     commit), 46 GB/s of weights per CTA; two overlap their fixed costs.  The
//     epilogue adds the two accumulators in a fixed order;
//   * K is split over a thread-block cluster; every CTA PUSHES its FP32 partial rows
//     into the shared memory of the CTA that owns them: the rows go from tensor memory
//     to the CTA's own (by then idle) ring, and one cp.async.bulk per epilogue warp and
//     owner moves them, completing its bytes on the owner's mbarrier.  The owner sums
//     in rank order and stores.  One hop, no per-thread remote stores, deterministic.
// Operand roles, TMA types, scale atoms and the instruction descriptor are those of
// the persistent kernel in gemm.cu: weights are MMA operand A (128 features x 128 K,
// 16U6_ALIGN16B), activations operand B (TN rows), UE8M0 scales in tensor memory.
#include "gemm.cuh"
#include "ptx.cuh"
#include "wait.cuh"

#include <cuda.h>

namespace mx {

int make_tensor_map_2d(CUtensorMap* out, int type, const void* base, uint64_t inner, uint64_t rows,
                       uint64_t stride, uint32_t box_rows);

namespace {

constexpr int kTileF = 128;    // output features per tile (MMA M)
constexpr int kTileK = 128;    // K values per pipeline stage
constexpr int kMmaK = 32;      // K values per tcgen05.mma
constexpr int kThreads = 224;  // warp 0 TMA, warps 1-2 MMA, warps 3..6 epilogue
constexpr uint32_t kWTileBytes = kTileF * kTileK;
// A 16U6_ALIGN16B load counts the packed bytes it read on the mbarrier.
constexpr uint32_t kWTileTxBytes = kWTileBytes / 4 * 3;
constexpr uint32_t kAtomBytes = 512;

struct StreamArgs {
  const uint8_t* w_scales;
  const uint8_t* a_scales;
  void* out;
  int* status;
  int m;
  int n;
  int k_blocks;
  int n_tiles;
  int cluster_k;
  int out_dtype;
  float alpha;
};

// Timeline of CTA 0 (development builds only, -DMXFP6_STREAM_STAMPS): slot s of launch l
// is g_stream_stamps[16 * (l % 64) + s], nanoseconds of the global timer.
#ifdef MXFP6_STREAM_STAMPS
__device__ long long g_stream_stamps[16 * 64];
__device__ unsigned int g_stream_launches;
#define MX_STAMP(slot)                                                                  \
  do {                                                                                  \
    if (blockIdx.x == 0) {                                                              \
      long long t__;                                                                    \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__));                           \
      g_stream_stamps[16 * (*stamp_launch) + (slot)] = t__;                             \
    }                                                                                   \
  } while (0)
#else
#define MX_STAMP(slot) \
  do {                 \
  } while (0)
#endif

template <int TN>
struct SCfg {
  static constexpr uint32_t kATileBytes = TN * kTileK;
  static constexpr uint32_t kSfBytes = 2 * kAtomBytes;  // weight atom + activation atom
  // Partial rows pushed by the cluster: ceil(TN / ck) rows from each of ck ranks,
  // at most TN + 7 rows of 128 floats.  The direct epilogue (no split) uses the same
  // bytes as four 2 KB transpose patches.
  static constexpr uint32_t kRedBytes = (TN + 8) * kTileF * 4;
  // Tensor memory: one accumulator per issuing warp, then four rotating sets of
  // (weight scales, activation scales) per issuing warp, so that the scale copy of a
  // block never overwrites scales an earlier, still running MMA reads.
  static constexpr int kSfCol = 2 * TN;
  static constexpr int kSfSets = 4;
  static constexpr int kColsUsed = kSfCol + 2 * kSfSets * 8;
  static constexpr int kTmemCols = TN <= 32 ? 128 : 256;  // of the SM's 512; two CTAs share it
  static_assert(kColsUsed <= kTmemCols, "accumulator and scale columns exceed the allocation");
  // An SM has 228 KB of shared memory and reserves 1 KB per resident CTA; two CTAs share it.
  static constexpr size_t kBudget = 233472 / 2 - 1024;
  static constexpr uint32_t kStageBytes = kWTileBytes + kATileBytes + kSfBytes;
  static constexpr int kStages = (int)((kBudget - 2048 - kRedBytes) / kStageBytes);
  static_assert(kStages >= 3, "the ring needs a few stages");
  static constexpr size_t kSmemBytes = 1024 + (size_t)kStages * kStageBytes + kRedBytes + 1024;
  static_assert(kSmemBytes <= kBudget, "two CTAs must fit one SM");
  static_assert(kRedBytes >= 8192, "the transpose patches need 8 KB");
};

template <int TN>
__global__ void __launch_bounds__(kThreads, 2)
w6a8_stream_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_a,
                   const StreamArgs args) {
  using C = SCfg<TN>;
  // The next kernel on the stream only needs a free CTA slot to start its own prologue
  // and weight prefetch; it waits for this grid's completion before it reads or writes
  // anything this grid touches.
  ptx::grid_launch_dependents();

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* w_tiles = smem;
  uint8_t* a_tiles = w_tiles + (size_t)C::kStages * kWTileBytes;
  uint8_t* sf_tiles = a_tiles + (size_t)C::kStages * C::kATileBytes;
  float* red = reinterpret_cast<float*>(sf_tiles + (size_t)C::kStages * C::kSfBytes);
  uint8_t* fixed = reinterpret_cast<uint8_t*>(red) + C::kRedBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(fixed);  // full[S], empty[S], tfull, tempty, red
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(fixed + 8 * (2 * C::kStages + 3));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
#ifdef MXFP6_STREAM_STAMPS
  volatile int* stamp_launch = reinterpret_cast<volatile int*>(tmem_slot + 2);
#endif

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t full0 = ptx::smem_u32(bars);
  const uint32_t empty0 = full0 + 8 * C::kStages;
  const uint32_t tfull0 = empty0 + 8 * C::kStages;
  const uint32_t tempty0 = tfull0 + 8;
  const uint32_t red_full = tempty0 + 8;  // every rank's partial rows for this CTA have landed

  const int ck = args.cluster_k;
  const int rank = ck > 1 ? (int)ptx::cluster_ctarank() : 0;
  // A cluster computes exactly one feature tile; without a split the CTAs walk the tiles.
  const int first_tile = ck > 1 ? (int)blockIdx.x / ck : (int)blockIdx.x;
  const int tile_step = ck > 1 ? args.n_tiles : (int)gridDim.x;
  const int kb0 = ck > 1 ? (rank * args.k_blocks) / ck : 0;
  const int kb1 = ck > 1 ? ((rank + 1) * args.k_blocks) / ck : args.k_blocks;
  const int nkb = kb1 - kb0;
  const uint32_t tx_stage = kWTileTxBytes + C::kATileBytes + 2 * kAtomBytes;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
#ifdef MXFP6_STREAM_STAMPS
    if (blockIdx.x == 0) *stamp_launch = (int)(atomicAdd(&g_stream_launches, 1u) % 64u);
    MX_STAMP(0);
#endif
    for (int s = 0; s < C::kStages; ++s) {
      ptx::mbar_init(full0 + 8 * s, 1);
      ptx::mbar_init(empty0 + 8 * s, 1);
    }
    ptx::mbar_init(tfull0, 2);   // one commit per issuing warp
    ptx::mbar_init(tempty0, 4);  // one arrival per epilogue warp
    ptx::mbar_init(red_full, 1);
    if (ck > 1) {
      // This CTA owns rows [rank * m / ck, (rank + 1) * m / ck) of the tile and receives
      // them from every rank: 512 bytes per row and rank.  Armed before the cluster
      // synchronisation below, so before any peer can send.
      const int mine = ((rank + 1) * args.m) / ck - (rank * args.m) / ck;
      if (mine > 0) ptx::mbar_arrive_expect_tx(red_full, (uint32_t)(ck * mine * 512));
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
  if (threadIdx.x == 0) MX_STAMP(1);

  bool cluster_arrived = false;  // this thread has made its arrival on the exit barrier

  // ---- weight prefetch, before anything of the previous kernel is needed ----------
  int pre_tile = first_tile, pre_kb = kb0, prefetched = 0;
  if (warp == 0) {
    while (prefetched < C::kStages && pre_tile < args.n_tiles) {
      if (ptx::elect_one()) {
        const uint32_t bar = full0 + 8 * prefetched;
        ptx::mbar_arrive_expect_tx(bar, tx_stage);
        ptx::tma_load_2d(ptx::smem_u32(w_tiles + (size_t)prefetched * kWTileBytes), &tm_w,
                         pre_kb * kTileK, pre_tile * kTileF, bar);
        ptx::bulk_load(ptx::smem_u32(sf_tiles + (size_t)prefetched * C::kSfBytes),
                       args.w_scales + ((int64_t)pre_tile * args.k_blocks + pre_kb) * kAtomBytes,
                       kAtomBytes, bar);
      }
      __syncwarp();
      ++prefetched;
      if (++pre_kb == kb1) {
        pre_kb = kb0;
        pre_tile += tile_step;
      }
    }
  }
  // Peers must see this CTA's barriers initialised before they arrive on them.
  if (ck > 1) ptx::cluster_sync_all();
  if (threadIdx.x == 0) MX_STAMP(2);

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    ptx::grid_dependency_wait();
    if (lane == 0) MX_STAMP(3);
    // Activation tiles and activation scales of the prefetched stages.
    {
      int tile = first_tile, kb = kb0;
      for (int s = 0; s < prefetched; ++s) {
        if (ptx::elect_one()) {
          const uint32_t bar = full0 + 8 * s;
          ptx::tma_load_2d(ptx::smem_u32(a_tiles + (size_t)s * C::kATileBytes), &tm_a, kb * kTileK,
                           0, bar);
          ptx::bulk_load(ptx::smem_u32(sf_tiles + (size_t)s * C::kSfBytes + kAtomBytes),
                         args.a_scales + (int64_t)kb * kAtomBytes, kAtomBytes, bar);
        }
        __syncwarp();
        if (++kb == kb1) {
          kb = kb0;
          tile += tile_step;
        }
      }
    }
    int stage = prefetched == C::kStages ? 0 : prefetched;
    uint32_t phase = prefetched == C::kStages ? 1u : 0u;
    bool ok = true;
    for (int tile = pre_tile, kb = pre_kb; ok && tile < args.n_tiles;) {
      ok = __all_sync(0xffffffffu, bounded_wait(empty0 + 8 * stage, phase ^ 1u, abort_flag,
                                                args.status, 111));
      if (!ok) break;
      if (ptx::elect_one()) {
        const uint32_t bar = full0 + 8 * stage;
        ptx::mbar_arrive_expect_tx(bar, tx_stage);
        ptx::tma_load_2d(ptx::smem_u32(w_tiles + (size_t)stage * kWTileBytes), &tm_w, kb * kTileK,
                         tile * kTileF, bar);
        ptx::tma_load_2d(ptx::smem_u32(a_tiles + (size_t)stage * C::kATileBytes), &tm_a,
                         kb * kTileK, 0, bar);
        uint8_t* sf = sf_tiles + (size_t)stage * C::kSfBytes;
        ptx::bulk_load(ptx::smem_u32(sf),
                       args.w_scales + ((int64_t)tile * args.k_blocks + kb) * kAtomBytes, kAtomBytes,
                       bar);
        ptx::bulk_load(ptx::smem_u32(sf + kAtomBytes), args.a_scales + (int64_t)kb * kAtomBytes,
                       kAtomBytes, bar);
      }
      __syncwarp();
      if (++stage == C::kStages) {
        stage = 0;
        phase ^= 1u;
      }
      if (++kb == kb1) {
        kb = kb0;
        tile += tile_step;
      }
    }
  } else if (warp <= 2) {
    // ---------------- MMA issuers ----------------
    // The K blocks of this CTA's tiles form one sequence; block i sits in ring stage
    // i % kStages.  Issuer `which` takes the blocks in stages of parity `which` into its
    // own accumulator (columns which * TN) through its own scale columns.  The split is
    // by STAGE, not by block: a stage's barrier must have a single waiter that sees every
    // one of its phases.  A parity wait can only tell the current phase from the one
    // before; with an odd number of stages and a split by block the two warps would
    // take turns on a barrier, and the one that runs three blocks ahead of the other
    // would take the completion of phase k - 1 for that of phase k + 1.
    const int which = warp - 1;
    // E3M2 weights (A, format 4) x E4M3 activations (B, format 0), both K-major,
    // UE8M0 scales, M = 128, N = TN.
    constexpr uint32_t kIdesc = (4u << 7) | (0u << 10) | ((uint32_t)(TN >> 3) << 17) | (1u << 23) |
                                ((uint32_t)(kTileF >> 4) << 24);
    const uint32_t d_t = tmem_base + which * TN;
    const uint32_t sf_t0 = tmem_base + C::kSfCol + which * (C::kSfSets * 8);
    uint32_t sf_set = 0;
    uint32_t acc_phase = 0;
    int i = 0;      // index of the next block of the sequence
    int stage = 0;  // i % kStages
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = first_tile; ok && tile < args.n_tiles; tile += tile_step) {
      if (!__all_sync(0xffffffffu,
                      bounded_wait(tempty0, acc_phase ^ 1u, abort_flag, args.status, 112)))
        break;
      ptx::tc_fence_after();
      bool first = true;
      for (int kb = kb0; kb < kb1; ++kb, ++i) {
        if ((stage & 1) == which) {
          ok = __all_sync(0xffffffffu,
                          bounded_wait(full0 + 8 * stage, phase, abort_flag, args.status, 113));
          if (!ok) break;
          ptx::tc_fence_after();
          if (lane == 0 && i == 0) MX_STAMP(4);
          if (ptx::elect_one()) {
            const uint32_t sf = ptx::smem_u32(sf_tiles + (size_t)stage * C::kSfBytes);
            const uint32_t sfa_t = sf_t0 + sf_set * 8;
            const uint32_t sfb_t = sfa_t + 4;
            ptx::tc_cp_32x128b_warpx4(sfa_t, ptx::smem_desc_scale_atom(sf));
            ptx::tc_cp_32x128b_warpx4(sfb_t, ptx::smem_desc_scale_atom(sf + kAtomBytes));
            const uint64_t a_desc =
                ptx::smem_desc_sw128(ptx::smem_u32(w_tiles + (size_t)stage * kWTileBytes));
            const uint64_t b_desc =
                ptx::smem_desc_sw128(ptx::smem_u32(a_tiles + (size_t)stage * C::kATileBytes));
#pragma unroll
            for (int ks = 0; ks < kTileK / kMmaK; ++ks) {
              const uint32_t idesc = kIdesc | ((uint32_t)ks << 4) | ((uint32_t)ks << 29);
              // 32 K values = 32 bytes = 2 descriptor address units.
              ptx::tc_mma_mxf8f6f4(d_t, a_desc + 2 * ks, b_desc + 2 * ks, idesc, sfa_t, sfb_t,
                                   (!first || ks > 0) ? 1u : 0u);
            }
            ptx::tc_commit(empty0 + 8 * stage);
          }
          __syncwarp();
          first = false;
          sf_set = (sf_set + 1u) % C::kSfSets;
        }
        if (++stage == C::kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (!ok) break;
      // Arrives when every MMA this warp issued for the tile has completed (at once when
      // the tile had a single block and it was the other warp's).
      if (ptx::elect_one()) ptx::tc_commit(tfull0);
      __syncwarp();
      if (lane == 0 && tile == first_tile && which == 0) MX_STAMP(5);
      acc_phase ^= 1u;
    }
  } else {
    // ---------------- epilogue (warps 3..6) ----------------
    const int quarter = warp & 3;  // tensor-memory lane quarter this warp may read
    const int rows = args.m;
    const bool bf16_out = args.out_dtype == kBF16;
    // Everything of the cluster exchange that does not depend on data, ahead of the wait.
    const int slots = (TN + ck - 1) / ck;  // rows an owner reserves per sending rank
    const int my0 = (rank * rows) / ck, my1 = ((rank + 1) * rows) / ck;
    float* send = reinterpret_cast<float*>(w_tiles);  // [quarter][row][32 floats]
    float* send_mine = send + (quarter * TN) * 32 + lane;
    uint32_t push_dst = 0, push_src = 0, push_bytes = 0, push_bar = 0;
    if (ck > 1 && lane < ck) {
      const int r0 = (lane * rows) / ck, r1 = ((lane + 1) * rows) / ck;
      push_bytes = (uint32_t)(r1 - r0) * 128u;
      push_src = ptx::smem_u32(send + (quarter * TN + r0) * 32);
      push_dst = ptx::mapa(ptx::smem_u32(red + ((rank * 4 + quarter) * slots) * 32), (uint32_t)lane);
      push_bar = ptx::mapa(red_full, (uint32_t)lane);
    }
    const float* recv = red + (quarter * slots) * 32 + lane;  // + src * 4 * slots * 32 + row * 32
    const int recv_stride = 4 * slots * 32;
    uint32_t acc_phase = 0;
    int seq0 = 0;  // index of the tile's first block in the CTA's block sequence
    // The output may still be read by the previous kernel until it has completed.
    ptx::grid_dependency_wait();
    for (int tile = first_tile; tile < args.n_tiles; tile += tile_step, seq0 += nkb) {
      if (!bounded_wait(tfull0, acc_phase, abort_flag, args.status, 114)) break;
      ptx::tc_fence_after();
      if (threadIdx.x == 96 && tile == first_tile) MX_STAMP(6);
      const uint32_t t_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
      // A tile of one or two blocks may have fed one accumulator only; the other is stale.
      bool use0 = nkb > 2, use1 = nkb > 2;
      for (int j = 0; j < nkb && j < 2; ++j) {
        const int owner = ((seq0 + j) % C::kStages) & 1;
        use0 = use0 || owner == 0;
        use1 = use1 || owner == 1;
      }
      const int f0 = tile * kTileF + quarter * 32;  // first feature of this warp
      if (ck > 1) {
        // ---- partial rows -> this CTA's shared memory -> their owners.  The ring is idle:
        //      the commits that completed tfull followed this CTA's last MMAs.  Each warp
        //      keeps its 32 features of every row together, so the rows one owner gets
        //      from one warp are one contiguous block. ----
#pragma unroll 1
        for (int c0 = 0; c0 < rows; c0 += 16) {
          uint32_t a[16], b[16];
          ptx::tmem_ld_x16(t_addr + c0, a);
          ptx::tmem_ld_x16(t_addr + TN + c0, b);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float v =
                (use0 ? __uint_as_float(a[j]) : 0.0f) + (use1 ? __uint_as_float(b[j]) : 0.0f);
            if (c0 + j < rows) send_mine[(c0 + j) * 32] = v;
          }
        }
        ptx::fence_proxy_async();  // the bulk copies below read what the lanes just wrote
        __syncwarp();
        if (push_bytes != 0) ptx::bulk_copy_to_peer(push_dst, push_src, push_bytes, push_bar);
        if (threadIdx.x == 96) MX_STAMP(7);
        bool landed = true;
        if (my1 > my0) landed = bounded_wait_cluster(red_full, 0u, abort_flag, args.status, 116);
        if (threadIdx.x == 96) MX_STAMP(8);
        // Exit barrier: once every owner has its rows, no copy is in flight that still
        // reads a sender's shared memory.  Nothing is published by this arrival.
        ptx::cluster_arrive_relaxed();
        cluster_arrived = true;
        const int f = f0 + lane;
        if (landed && f < args.n) {
          // Two rows at a time, all their loads issued before the sums (rank order).
#pragma unroll 1
          for (int s0 = 0; s0 < my1 - my0; s0 += 2) {
            const bool two = s0 + 1 < my1 - my0;
            const float* p = recv + s0 * 32;
            float part[2][8];
#pragma unroll
            for (int src = 0; src < 8; ++src) {
              part[0][src] = src < ck ? p[src * recv_stride] : 0.0f;
              part[1][src] = (src < ck && two) ? p[src * recv_stride + 32] : 0.0f;
            }
            float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
            for (int src = 0; src < 8; ++src) {
              sum0 += part[0][src];  // ranks beyond ck contribute +0.0f
              sum1 += part[1][src];
            }
            const int64_t at = (int64_t)(my0 + s0) * args.n + f;
            if (bf16_out) {
              __nv_bfloat16* o = static_cast<__nv_bfloat16*>(args.out) + at;
              o[0] = __float2bfloat16_rn(args.alpha * sum0);
              if (two) o[args.n] = __float2bfloat16_rn(args.alpha * sum1);
            } else {
              __half* o = static_cast<__half*>(args.out) + at;
              o[0] = __float2half_rn(args.alpha * sum0);
              if (two) o[args.n] = __float2half_rn(args.alpha * sum1);
            }
          }
        }
        if (threadIdx.x == 96) MX_STAMP(9);
        break;  // one tile per cluster
      }
      // ---- no split: transpose 16 token columns at a time through a private patch of
      //      shared memory and write 16-byte row segments ----
      uint16_t* patch = reinterpret_cast<uint16_t*>(red) + quarter * 1024;  // [16][32] halves
#pragma unroll 1
      for (int c0 = 0; c0 < rows; c0 += 16) {
        uint32_t a[16], b[16];
        ptx::tmem_ld_x16(t_addr + c0, a);
        ptx::tmem_ld_x16(t_addr + TN + c0, b);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float v = args.alpha * ((use0 ? __uint_as_float(a[j]) : 0.0f) +
                                        (use1 ? __uint_as_float(b[j]) : 0.0f));
          patch[j * 32 + lane] = bf16_out ? __bfloat16_as_ushort(__float2bfloat16_rn(v))
                                          : __half_as_ushort(__float2half_rn(v));
        }
        __syncwarp();
        // 4 lanes cover one 64-byte row segment; a warp writes 8 rows per pass.
        const int seg = lane & 3;
        const int fseg = f0 + seg * 8;
#pragma unroll
        for (int pass = 0; pass < 2; ++pass) {
          const int rr = (lane >> 2) + 8 * pass;
          const int t = c0 + rr;
          if (t < rows && fseg < args.n) {
            const uint4 v = *reinterpret_cast<const uint4*>(patch + rr * 32 + seg * 8);
            *reinterpret_cast<uint4*>(static_cast<uint16_t*>(args.out) + (int64_t)t * args.n + fseg) = v;
          }
        }
        __syncwarp();
      }
      // The accumulators are free for the next tile.
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(tempty0);
      acc_phase ^= 1u;
    }
  }

  // ---------------- teardown ----------------
  ptx::tc_fence_before();
  __syncthreads();
  if (ck > 1) {
    if (!cluster_arrived) ptx::cluster_arrive_relaxed();
    ptx::cluster_wait();
  }
  if (threadIdx.x == 0) MX_STAMP(10);
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

bool use_pdl() {
  static const bool enabled = []() {
    const char* env = std::getenv("MXFP6_B200_PDL");
    return env == nullptr || env[0] != '0';
  }();
  return enabled;
}

template <int TN>
int launch_tn(const CUtensorMap& tm_w, const CUtensorMap& tm_a, const StreamArgs& args,
              const GemmPlan& plan, cudaStream_t stream) {
  using C = SCfg<TN>;
  static bool configured[64] = {};
  int device = 0;
  MX_CUDA(cudaGetDevice(&device));
  if (device < 64 && !configured[device]) {
    MX_CUDA(cudaFuncSetAttribute(w6a8_stream_kernel<TN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)C::kSmemBytes));
    MX_CUDA(cudaFuncSetAttribute(w6a8_stream_kernel<TN>,
                                 cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared));
    configured[device] = true;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((unsigned)plan.grid);
  config.blockDim = dim3(kThreads);
  config.dynamicSmemBytes = C::kSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  int count = 0;
  if (plan.cluster_k > 1) {
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
  MX_CUDA(cudaLaunchKernelEx(&config, w6a8_stream_kernel<TN>, tm_w, tm_a, args));
  return kOk;
}

int g_stream_mode = 1;

}  // namespace

#ifdef MXFP6_STREAM_STAMPS
extern "C" int mxfp6_debug_stream_stamps(long long* host_out, unsigned int* launches) {
  if (cudaMemcpyFromSymbol(host_out, g_stream_stamps, sizeof(long long) * 16 * 64) != cudaSuccess)
    return 1;
  return cudaMemcpyFromSymbol(launches, g_stream_launches, sizeof(unsigned int)) != cudaSuccess;
}
#endif

void set_stream_kernel_mode(int enabled) { g_stream_mode = enabled != 0 ? 1 : 0; }
int stream_kernel_mode() { return g_stream_mode; }

// Dense FP16/BF16 launches of at most 64 rows whose K split (if any) stays inside a cluster.
bool stream_kernel_applies(const GemmProblem& p) {
  if (p.expert_offsets != nullptr || p.groups != 1 || p.mode != kGemmStore) return false;
  if (p.m_total > 64 || p.splits > 1) return false;
  if (p.tile_tokens != 0 && p.tile_tokens != 16 && p.tile_tokens != 32 && p.tile_tokens != 64)
    return false;
  if (p.tile_tokens != 0 && p.tile_tokens < p.m_total) return false;
  const int mode = p.split_mode != 0 ? p.split_mode : default_split_mode();
  return mode != 2;  // mode 2 asks for the scratch-arena split of the persistent kernel
}

int plan_w6a8_stream(const GemmProblem& p, int sms, GemmPlan* plan) {
  const int tn =
      p.tile_tokens != 0 ? p.tile_tokens : (p.m_total <= 16 ? 16 : p.m_total <= 32 ? 32 : 64);
  const int n_tiles = (p.n + kTileF - 1) / kTileF;
  const int k_blocks = p.k / kTileK;
  const int mode = p.split_mode != 0 ? p.split_mode : default_split_mode();
  // Two CTAs fit one SM.  A launch fills most of those slots when it can: the bytes a
  // CTA keeps in flight are bounded by its ring, and the stream needs all of them.
  const int slots = sms + sms / 2 + 18;  // 240 on 148 SMs: measured, 280 CTAs ran 40 % slower
  int ck = 1;
  if (p.cluster_k > 0) {
    MX_REQUIRE(p.cluster_k <= 8 && p.cluster_k <= k_blocks,
               "cluster_k must be at most min(8, k/128); got %d", p.cluster_k);
    ck = p.cluster_k;
  } else if (mode == 1 && n_tiles * 2 <= slots) {
    ck = slots / n_tiles;
    if (ck > 8) ck = 8;
    if (ck > k_blocks) ck = k_blocks;
    if (ck < 1) ck = 1;
  }
  plan->tile_tokens = tn;
  plan->splits = 1;
  plan->cluster_k = ck;
  plan->cta_pair = 0;
  plan->kernel = kKernelStream;
  plan->stages = tn == 16 ? SCfg<16>::kStages : tn == 32 ? SCfg<32>::kStages : SCfg<64>::kStages;
  plan->smem_bytes =
      tn == 16 ? SCfg<16>::kSmemBytes : tn == 32 ? SCfg<32>::kSmemBytes : SCfg<64>::kSmemBytes;
  if (ck > 1) {
    plan->grid = n_tiles * ck;
  } else {
    // Equal shares: every CTA walks the same number of tiles (up to two CTAs per SM).
    const int resident = 2 * sms - 8;
    const int waves = (n_tiles + resident - 1) / resident;
    plan->grid = (n_tiles + waves - 1) / waves;
  }
  plan->partial_bytes = 0;
  plan->counter_bytes = 0;
  return kOk;
}

int launch_w6a8_stream(const GemmProblem& p, const GemmPlan& plan, cudaStream_t stream) {
  int device = 0;
  MX_CUDA(cudaGetDevice(&device));
  CUtensorMap tm_w, tm_a;
  if (int rc = make_tensor_map_2d(&tm_w, (int)CU_TENSOR_MAP_DATA_TYPE_16U6_ALIGN16B, p.w_values,
                                  (uint64_t)p.k, (uint64_t)p.n, (uint64_t)p.k * 3 / 4, kTileF))
    return rc;
  if (int rc = make_tensor_map_2d(&tm_a, (int)CU_TENSOR_MAP_DATA_TYPE_UINT8, p.a_values,
                                  (uint64_t)p.k, (uint64_t)p.m_total, (uint64_t)p.k,
                                  (uint32_t)plan.tile_tokens))
    return rc;
  StreamArgs args;
  args.w_scales = p.w_scales;
  args.a_scales = p.a_scales;
  args.out = p.out;
  args.status = p.status_word != nullptr ? p.status_word : device_status_word(device);
  if (args.status == nullptr) return kCudaError;
  args.m = (int)p.m_total;
  args.n = p.n;
  args.k_blocks = p.k / kTileK;
  args.n_tiles = (p.n + kTileF - 1) / kTileF;
  args.cluster_k = plan.cluster_k;
  args.out_dtype = p.out_dtype;
  args.alpha = p.alpha;
  if (plan.tile_tokens == 16) return launch_tn<16>(tm_w, tm_a, args, plan, stream);
  if (plan.tile_tokens == 32) return launch_tn<32>(tm_w, tm_a, args, plan, stream);
  if (plan.tile_tokens == 64) return launch_tn<64>(tm_w, tm_a, args, plan, stream);
  set_error("the weight-streaming kernel has tiles of 16, 32 and 64 rows; got %d",
            plan.tile_tokens);
  return kInvalidArgument;
}

}  // namespace mx
