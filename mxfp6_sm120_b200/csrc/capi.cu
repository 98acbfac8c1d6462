// extern "C" boundary of libmxfp6_b200.so and the split-K workspace arena.
//
// The arena follows the reference's contract (csrc/torch_extension.cu:103-138,
// 247-335,1955-2116): Disabled -> Planning (record needs, transient scratch) ->
// Frozen (one persistent lane per stream, counters zeroed once, kernels reset
// their own counters, capture on a lane-less stream is an error).
#include "../../include/mxfp6_b200.h"

#include "gemm.cuh"

#include <algorithm>
#include <map>
#include <mutex>
#include <set>
#include <shared_mutex>
#include <tuple>
#include <unordered_map>
#include <vector>

namespace mx {

// ---- error text -------------------------------------------------------------
namespace {
thread_local char g_error[512] = "";
}
void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}
const char* last_error() { return g_error; }

// ---- kernels implemented in the other translation units ------------------------
int quantize_mxfp8(const void*, int, int64_t, int64_t, uint8_t*, uint8_t*, uint8_t*, cudaStream_t);
void tp_set_wait_limit(long long);
long long tp_wait_limit();
int tp_block_alloc(size_t, void**, unsigned char*);
int tp_block_open(const unsigned char*, void**);
int tp_block_close(void*);
int tp_block_free(void*);
int tp_allreduce_sum(void* const*, int, int, int, size_t, void*, int64_t, int64_t, cudaStream_t);
int tp_reduce_scatter(void* const*, int, int, int, size_t, void*, int64_t, int64_t, cudaStream_t);
int tp_allreduce_pointers(const uint64_t*, const uint64_t*, int, int, void*, int64_t, int64_t,
                          cudaStream_t);
int tp_allreduce_two_phase(void* const*, int, int, int, size_t, void*, int64_t, int64_t,
                           cudaStream_t);
int tp_allgather(void* const*, int, int, int, size_t, int, const int64_t*, const int64_t*,
                 void* const*, cudaStream_t);
int tp_allreduce_rmsnorm_quantize(void* const*, int, int, int, size_t, void*, const void*, float,
                                  int64_t, int64_t, uint8_t*, uint8_t*, cudaStream_t);
int rmsnorm_quantize_mxfp8(const void*, const void*, void*, int, const void*, float, int64_t,
                           int64_t, uint8_t*, uint8_t*, uint8_t*, cudaStream_t);
int quantize_mxfp6(const void*, int, int64_t, int64_t, uint8_t*, uint8_t*, uint8_t*, cudaStream_t);
int pack_fp6(const uint8_t*, int64_t, uint8_t*, cudaStream_t);
int unpack_fp6(const uint8_t*, int64_t, int64_t, uint8_t*, cudaStream_t);
int expand_fp6_to_fp8(const uint8_t*, int64_t, int64_t, uint8_t*, cudaStream_t);
int pad_fp6(const uint8_t*, int64_t, uint8_t*, cudaStream_t);
int pack_scales(const uint8_t*, int64_t, int64_t, uint8_t*, cudaStream_t);
int unpack_scales(const uint8_t*, int64_t, int64_t, uint8_t*, cudaStream_t);
int grouped_scale_offsets(const int64_t*, int, int64_t*, cudaStream_t);
int pack_grouped_scales(const uint8_t*, const int64_t*, const int64_t*, int, int64_t, int64_t,
                        uint8_t*, cudaStream_t);

int moe_topk_quant(const void*, const void*, int64_t, int, int, int, int, uint8_t*, uint8_t*,
                   uint8_t*, float*, int32_t*, cudaStream_t);
int moe_route(const uint8_t*, const uint8_t*, const void*, int, int64_t, int, int, const int32_t*,
              int, int, int, int64_t*, int64_t*, int32_t*, uint8_t*, uint8_t*, int32_t*, int32_t*,
              cudaStream_t);
int moe_topk_quant_route(const void*, const void*, int64_t, int, int, int, int, uint8_t*, uint8_t*,
                         uint8_t*, float*, int32_t*, const int32_t*, int, int, int64_t*, int64_t*,
                         int32_t*, uint8_t*, uint8_t*, int32_t*, int32_t*, cudaStream_t);
int silu_mul_quant(const void*, int, int64_t, int, uint8_t*, uint8_t*, uint8_t*, const int64_t*,
                   const int64_t*, int, cudaStream_t);
int moe_reduce(void*, const void*, int, const float*, const int32_t*, const void*, const void*, int,
               int, int64_t, int, int, int64_t, cudaStream_t);

int moe_route_gemm(void*, uint8_t*, int, int, const uint8_t*, const uint8_t*, int64_t,
                   const uint8_t*, const uint8_t*, int, const uint8_t*, const uint8_t*,
                   const void*, int, int64_t, int, int, int64_t, int64_t, cudaStream_t);
int moe_route_w2_reduce(void*, int, const uint8_t*, const uint8_t*, const uint8_t*, const uint8_t*,
                        int, const uint8_t*, const uint8_t*, const void*, int, const float*,
                        const void*, int, int, const void*, int, int64_t, int, int64_t, int64_t,
                        int, const void*, int, int, cudaStream_t);
int moe_decode_layer_supported(int64_t, int, int, int64_t, int64_t);
int moe_decode_layer_preferred(int64_t, int, int, int64_t, int64_t);
int moe_decode_layer(void*, int, const void*, const void*, const void*, int, int, const uint8_t*,
                     const uint8_t*, const uint8_t*, const uint8_t*, int, const uint8_t*,
                     const uint8_t*, const uint8_t*, const uint8_t*, uint8_t*, uint8_t*, int32_t*,
                     float*, int64_t, int, int, int, int64_t, int64_t, int, cudaStream_t);
int moe_reduce_array(void*, const void*, int, const float*, const void*, int, int, int64_t, int,
                     int64_t, cudaStream_t);
int moe_router_logits(const void*, const void*, const void*, void*, void*, int64_t, int64_t, int,
                      int, cudaStream_t);

// ---- explicit configurations and the per-shape override registry -----------------
// Ids: 0-15 weight-streaming kernel (tile 16: 0-7, tile 32: 8-15; cluster_k = id % 8 + 1);
// 16-31 persistent kernel, cluster split (tiles 16, 32, 64, 96 x cluster_k 1, 2, 4, 8);
// 32-34 persistent kernel, tiles 128, 192, 256, no split; 35-37 CTA-pair kernel, tiles
// 128, 192, 256; 38-49 persistent kernel, scratch split (tiles 16, 32, 64, 96 x splits 2, 4, 8);
// 50-57 weight-streaming kernel, tile 64 (cluster_k = id - 49).
const char* const kW6A8ConfigAbi = "b200-w6a8-58-v1";

int describe_w6a8_candidate(int id, int out[4]) {
  MX_REQUIRE(id >= 0 && id < kW6A8Candidates, "config_id must be in [0, %d]; got %d",
             kW6A8Candidates - 1, id);
  static const int narrow[4] = {16, 32, 64, 96};
  static const int wide[3] = {128, 192, 256};
  static const int pow2[4] = {1, 2, 4, 8};
  int kernel = kKernelPersistent, tile = 0, cluster_k = 1, splits = 1;
  if (id < 16) {
    kernel = kKernelStream;
    tile = id < 8 ? 16 : 32;
    cluster_k = id % 8 + 1;
  } else if (id < 32) {
    tile = narrow[(id - 16) / 4];
    cluster_k = pow2[(id - 16) % 4];
  } else if (id < 35) {
    tile = wide[id - 32];
  } else if (id < 38) {
    kernel = kKernelPair;
    tile = wide[id - 35];
  } else if (id < 50) {
    tile = narrow[(id - 38) / 3];
    splits = pow2[(id - 38) % 3 + 1];
  } else {
    kernel = kKernelStream;
    tile = 64;
    cluster_k = id - 49;
  }
  out[0] = kernel;
  out[1] = tile;
  out[2] = cluster_k;
  out[3] = splits;
  return kOk;
}

int apply_w6a8_candidate(int id, GemmProblem* p) {
  int c[4];
  if (int rc = describe_w6a8_candidate(id, c)) return rc;
  p->force_kernel = c[0];
  p->tile_tokens = c[1];
  p->cluster_k = c[2] > 1 || c[0] == kKernelStream ? c[2] : 0;
  p->splits = c[3] > 1 ? c[3] : 1;
  // A persistent-kernel candidate without any split must not pick one up from the default mode.
  p->split_mode = c[3] > 1 ? 2 : (c[2] > 1 || c[0] == kKernelStream ? 1 : 3);
  return kOk;
}

namespace {
using ShapeKey = std::tuple<int, int64_t, int64_t, int64_t, int>;  // device, m, n, k, out dtype
std::shared_mutex g_override_mutex;
std::map<ShapeKey, int> g_overrides;

// Installs the override of this exact problem, if one is registered
// (the reference looks its map up first too, csrc/torch_extension.cu:1192-1199).
int apply_override(GemmProblem* p) {
  {
    std::shared_lock<std::shared_mutex> lock(g_override_mutex);
    if (g_overrides.empty()) return kOk;  // the common case; also keeps planning free of CUDA calls
  }
  int device = 0;
  MX_CUDA(cudaGetDevice(&device));
  int id = -1;
  {
    std::shared_lock<std::shared_mutex> lock(g_override_mutex);
    auto it = g_overrides.find(ShapeKey{device, p->m_total, p->n, p->k, p->out_dtype});
    if (it == g_overrides.end()) return kOk;
    id = it->second;
  }
  return apply_w6a8_candidate(id, p);
}
}  // namespace

// ---- workspace arena ------------------------------------------------------------
namespace {

enum class ArenaMode { Disabled, Planning, Frozen };

struct Lane {
  cudaStream_t stream = nullptr;
  uint8_t* storage = nullptr;
};

struct Arena {
  ArenaMode mode = ArenaMode::Disabled;
  size_t max_reduction_bytes = 0;
  size_t max_barrier_bytes = 0;
  std::set<std::pair<size_t, size_t>> layouts;
  std::vector<Lane> lanes;
  int64_t persistent_launches = 0;
  int64_t fallback_launches = 0;
};

std::mutex g_arena_mutex;
std::unordered_map<int, Arena> g_arenas;

bool stream_is_capturing(cudaStream_t stream) {
  cudaStreamCaptureStatus status = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &status) != cudaSuccess) return false;
  return status != cudaStreamCaptureStatusNone;
}

void fill_stats(const Arena& a, int64_t out[10]) {
  const int64_t bytes = (int64_t)(a.max_reduction_bytes + a.max_barrier_bytes);
  out[0] = (int64_t)a.layouts.size();
  out[1] = (int64_t)a.max_reduction_bytes;
  out[2] = (int64_t)a.max_barrier_bytes;
  out[3] = bytes;
  out[4] = (int64_t)a.lanes.size();
  out[5] = bytes * (int64_t)a.lanes.size();
  out[6] = a.mode == ArenaMode::Planning;
  out[7] = a.mode == ArenaMode::Frozen;
  out[8] = a.persistent_launches;
  out[9] = a.fallback_launches;
}

int new_lane(Arena& arena, cudaStream_t stream, Lane* lane) {
  const size_t bytes = arena.max_reduction_bytes + arena.max_barrier_bytes;
  uint8_t* storage = nullptr;
  MX_CUDA(cudaMalloc(&storage, bytes));
  MX_CUDA(cudaMemsetAsync(storage + arena.max_reduction_bytes, 0, arena.max_barrier_bytes,
                          stream));
  lane->stream = stream;
  lane->storage = storage;
  return kOk;
}

struct Scratch {
  float* partials = nullptr;
  uint32_t* counters = nullptr;
  uint8_t* transient = nullptr;  // freed (stream-ordered) after the launch
};

// Picks scratch for a split-K launch: a persistent lane when the arena is frozen
// and large enough, otherwise a stream-ordered transient allocation.
int select_scratch(int device, cudaStream_t stream, size_t reduction_bytes, size_t barrier_bytes,
                   Scratch* out) {
  {
    std::lock_guard<std::mutex> lock(g_arena_mutex);
    auto it = g_arenas.find(device);
    if (it != g_arenas.end()) {
      Arena& arena = it->second;
      if (arena.mode == ArenaMode::Planning) {
        arena.layouts.emplace(reduction_bytes, barrier_bytes);
        arena.max_reduction_bytes = std::max(arena.max_reduction_bytes, reduction_bytes);
        arena.max_barrier_bytes = std::max(arena.max_barrier_bytes, barrier_bytes);
      } else if (arena.mode == ArenaMode::Frozen) {
        if (reduction_bytes <= arena.max_reduction_bytes &&
            barrier_bytes <= arena.max_barrier_bytes) {
          auto lane = std::find_if(arena.lanes.begin(), arena.lanes.end(),
                                   [stream](const Lane& l) { return l.stream == stream; });
          if (lane == arena.lanes.end()) {
            if (stream_is_capturing(stream)) {
              set_error(
                  "split-K persistent workspace has no lane for the current CUDA Graph capture "
                  "stream; run an eager warm-up on this stream after "
                  "finalize_workspace_planning() and before capture");
              return kWorkspaceError;
            }
            Lane fresh;
            if (int rc = new_lane(arena, stream, &fresh)) return rc;
            arena.lanes.push_back(fresh);
            lane = std::prev(arena.lanes.end());
          }
          out->partials = reinterpret_cast<float*>(lane->storage);
          out->counters = reinterpret_cast<uint32_t*>(lane->storage + arena.max_reduction_bytes);
          ++arena.persistent_launches;
          return kOk;
        }
        ++arena.fallback_launches;
        if (stream_is_capturing(stream)) {
          set_error(
              "split-K persistent workspace is unavailable during CUDA Graph capture: the "
              "selected layout exceeds the frozen arena capacity; re-run workspace planning "
              "with every captured shape");
          return kWorkspaceError;
        }
      }
    }
  }
  uint8_t* storage = nullptr;
  const size_t reduction_padded = (reduction_bytes + 255) & ~size_t(255);
  MX_CUDA(cudaMallocAsync(&storage, reduction_padded + barrier_bytes, stream));
  MX_CUDA(cudaMemsetAsync(storage + reduction_padded, 0, barrier_bytes, stream));
  out->transient = storage;
  out->partials = reinterpret_cast<float*>(storage);
  out->counters = reinterpret_cast<uint32_t*>(storage + reduction_padded);
  return kOk;
}

int dense_problem(GemmProblem* p, const uint8_t* a_values, const uint8_t* a_scales,
                  const uint8_t* w_values, const uint8_t* w_scales, int64_t m, int64_t n,
                  int64_t k, float alpha, void* out, int out_dtype) {
  MX_REQUIRE(m > 0, "m must be positive; got %lld", (long long)m);
  MX_REQUIRE(n > 0 && n % 8 == 0 && n <= INT32_MAX, "n must be a positive multiple of 8; got %lld",
             (long long)n);
  MX_REQUIRE(k > 0 && k % 128 == 0 && k <= INT32_MAX,
             "k must be a positive multiple of 128; got %lld", (long long)k);
  p->a_values = a_values;
  p->a_scales = a_scales;
  p->w_values = w_values;
  p->w_scales = w_scales;
  p->m_total = m;
  p->n = (int)n;
  p->k = (int)k;
  p->alpha = alpha;
  p->out = out;
  p->out_dtype = out_dtype;
  p->groups = 1;
  return kOk;
}

}  // namespace

int run_gemm_with_arena(GemmProblem& p, cudaStream_t stream) {
  if (p.force_kernel < 0 && p.tile_tokens == 0) {
    if (int rc = apply_override(&p)) return rc;
  }
  GemmPlan plan;
  if (int rc = plan_w6a8(p, &plan)) return rc;
  Scratch scratch;
  if (plan.splits > 1) {
    int device = 0;
    MX_CUDA(cudaGetDevice(&device));
    if (int rc = select_scratch(device, stream, plan.partial_bytes, plan.counter_bytes, &scratch))
      return rc;
    p.partials = scratch.partials;
    p.partial_bytes = plan.partial_bytes;
    p.counters = scratch.counters;
    p.counter_bytes = plan.counter_bytes;
  }
  const int rc = launch_w6a8(p, plan, stream);
  if (scratch.transient != nullptr) cudaFreeAsync(scratch.transient, stream);
  return rc;
}

}  // namespace mx

using namespace mx;

extern "C" {

int mxfp6_b200_abi_version(void) { return MXFP6_B200_ABI_VERSION; }
const char* mxfp6_b200_last_error(void) { return last_error(); }

int mxfp6_b200_device_status(int* value, int reset) {
  MX_REQUIRE(value != nullptr, "value must not be null");
  int device = 0;
  MX_CUDA(cudaGetDevice(&device));
  return read_device_status(device, value, reset != 0);
}

int mxfp6_set_split_k_mode(int mode) {
  MX_REQUIRE(mode >= 1 && mode <= 3, "mode must be 1 (cluster), 2 (scratch arena) or 3 (off)");
  set_default_split_mode(mode);
  return kOk;
}
int mxfp6_get_split_k_mode(void) { return default_split_mode(); }

int mxfp6_set_cta_pair_mode(int enabled) {
  set_cta_pair_mode(enabled);
  return kOk;
}

int mxfp6_get_cta_pair_mode(void) { return cta_pair_mode(); }

int mxfp6_pack_fp6(const uint8_t* codes, int64_t n, uint8_t* packed, void* stream) {
  return pack_fp6(codes, n, packed, static_cast<cudaStream_t>(stream));
}
int mxfp6_unpack_fp6(const uint8_t* packed, int64_t rows, int64_t k, uint8_t* codes,
                     void* stream) {
  return unpack_fp6(packed, rows, k, codes, static_cast<cudaStream_t>(stream));
}
int mxfp6_pad_fp6(const uint8_t* packed, int64_t bytes, uint8_t* padded, void* stream) {
  return pad_fp6(packed, bytes, padded, static_cast<cudaStream_t>(stream));
}
int mxfp6_expand_fp6_to_fp8(const uint8_t* packed, int64_t rows, int64_t k, uint8_t* e4m3,
                            void* stream) {
  return expand_fp6_to_fp8(packed, rows, k, e4m3, static_cast<cudaStream_t>(stream));
}
int mxfp6_pack_scales(const uint8_t* logical, int64_t rows, int64_t k, uint8_t* packed,
                      void* stream) {
  return pack_scales(logical, rows, k, packed, static_cast<cudaStream_t>(stream));
}
int mxfp6_unpack_scales(const uint8_t* packed, int64_t rows, int64_t k, uint8_t* logical,
                        void* stream) {
  return unpack_scales(packed, rows, k, logical, static_cast<cudaStream_t>(stream));
}
int64_t mxfp6_packed_scale_bytes(int64_t rows, int64_t k) { return packed_scale_bytes(rows, k); }
int mxfp6_grouped_scale_offsets(const int64_t* expert_offsets, int experts,
                                int64_t* scale_offsets, void* stream) {
  return grouped_scale_offsets(expert_offsets, experts, scale_offsets,
                               static_cast<cudaStream_t>(stream));
}
int mxfp6_pack_grouped_scales(const uint8_t* logical, const int64_t* expert_offsets,
                              const int64_t* scale_offsets, int experts, int64_t padded_rows,
                              int64_t k, uint8_t* packed, void* stream) {
  return pack_grouped_scales(logical, expert_offsets, scale_offsets, experts, padded_rows, k,
                             packed, static_cast<cudaStream_t>(stream));
}

int mxfp6_quantize_mxfp8(const void* input, int dtype, int64_t rows, int64_t k, uint8_t* values,
                         uint8_t* packed_scales, uint8_t* logical_scales, void* stream) {
  return quantize_mxfp8(input, dtype, rows, k, values, packed_scales, logical_scales,
                        static_cast<cudaStream_t>(stream));
}
int mxfp6_rmsnorm_quantize_mxfp8(const void* input, const void* residual, void* updated,
                                 int dtype, const void* weight, float eps, int64_t rows, int64_t k,
                                 uint8_t* values, uint8_t* packed_scales, uint8_t* logical_scales,
                                 void* stream) {
  return rmsnorm_quantize_mxfp8(input, residual, updated, dtype, weight, eps, rows, k, values,
                                packed_scales, logical_scales, static_cast<cudaStream_t>(stream));
}
int mxfp6_tp_block_alloc(size_t partial_bytes, void** block, unsigned char handle[64]) {
  return tp_block_alloc(partial_bytes, block, handle);
}
int mxfp6_tp_block_open(const unsigned char handle[64], void** block) {
  return tp_block_open(handle, block);
}
int mxfp6_tp_block_close(void* block) { return tp_block_close(block); }
int mxfp6_tp_set_wait_limit(int64_t clock_ticks) {
  MX_REQUIRE(clock_ticks > 0, "the wait limit must be positive");
  tp_set_wait_limit((long long)clock_ticks);
  return kOk;
}
int64_t mxfp6_tp_get_wait_limit(void) { return (int64_t)tp_wait_limit(); }
int mxfp6_tp_block_free(void* block) { return tp_block_free(block); }
int mxfp6_tp_allreduce_bf16(void* const* blocks, int world, int rank, int buffer,
                            size_t partial_bytes, void* out, int64_t rows, int64_t k,
                            void* stream) {
  return tp_allreduce_sum(blocks, world, rank, buffer, partial_bytes, out, rows, k,
                          static_cast<cudaStream_t>(stream));
}
int mxfp6_tp_allreduce_two_phase_bf16(void* const* blocks, int world, int rank, int buffer,
                                      size_t partial_bytes, void* out, int64_t rows, int64_t k,
                                      void* stream) {
  return tp_allreduce_two_phase(blocks, world, rank, buffer, partial_bytes, out, rows, k,
                                static_cast<cudaStream_t>(stream));
}
int mxfp6_tp_reduce_scatter_bf16(void* const* blocks, int world, int rank, int buffer,
                                 size_t partial_bytes, void* out, int64_t rows_per_rank, int64_t k,
                                 void* stream) {
  return tp_reduce_scatter(blocks, world, rank, buffer, partial_bytes, out, rows_per_rank, k,
                           static_cast<cudaStream_t>(stream));
}
int mxfp6_tp_allgather(void* const* blocks, int world, int rank, int buffer, size_t partial_bytes,
                       int segments, const int64_t* offsets, const int64_t* bytes,
                       void* const* dsts, void* stream) {
  return tp_allgather(blocks, world, rank, buffer, partial_bytes, segments, offsets, bytes, dsts,
                      static_cast<cudaStream_t>(stream));
}
int mxfp6_tp_allreduce_rmsnorm_quantize_mxfp8(void* const* blocks, int world, int rank, int buffer,
                                              size_t partial_bytes, void* x, const void* weight,
                                              float eps, int64_t rows, int64_t k, uint8_t* values,
                                              uint8_t* packed_scales, void* stream) {
  return tp_allreduce_rmsnorm_quantize(blocks, world, rank, buffer, partial_bytes, x, weight, eps,
                                       rows, k, values, packed_scales,
                                       static_cast<cudaStream_t>(stream));
}
int mxfp6_quantize_mxfp6(const void* input, int dtype, int64_t rows, int64_t k, uint8_t* values,
                         uint8_t* packed_scales, uint8_t* logical_scales, void* stream) {
  return quantize_mxfp6(input, dtype, rows, k, values, packed_scales, logical_scales,
                        static_cast<cudaStream_t>(stream));
}

int mxfp6_gemm_w6a8(const uint8_t* a_values, const uint8_t* a_scales, const uint8_t* w_values,
                    const uint8_t* w_scales, int64_t m, int64_t n, int64_t k, float alpha,
                    void* out, int out_dtype, void* stream) {
  GemmProblem p;
  if (int rc = dense_problem(&p, a_values, a_scales, w_values, w_scales, m, n, k, alpha, out,
                             out_dtype))
    return rc;
  return run_gemm_with_arena(p, static_cast<cudaStream_t>(stream));
}

int mxfp6_gemm_w6a8_ex(const uint8_t* a_values, const uint8_t* a_scales, const uint8_t* w_values,
                       const uint8_t* w_scales, int64_t m, int64_t n, int64_t k, float alpha,
                       void* out, int out_dtype, int tile_tokens, int splits, void* scratch,
                       size_t scratch_bytes, void* stream) {
  GemmProblem p;
  if (int rc = dense_problem(&p, a_values, a_scales, w_values, w_scales, m, n, k, alpha, out,
                             out_dtype))
    return rc;
  p.tile_tokens = tile_tokens;
  p.splits = splits;
  GemmPlan plan;
  if (int rc = plan_w6a8(p, &plan)) return rc;
  if (plan.splits > 1) {
    const size_t reduction_padded = (plan.partial_bytes + 255) & ~size_t(255);
    MX_REQUIRE(scratch != nullptr && scratch_bytes >= reduction_padded + plan.counter_bytes,
               "scratch must hold %zu bytes for this plan", reduction_padded + plan.counter_bytes);
    p.partials = static_cast<float*>(scratch);
    p.partial_bytes = plan.partial_bytes;
    p.counters = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(scratch) + reduction_padded);
    p.counter_bytes = plan.counter_bytes;
  }
  return launch_w6a8(p, plan, static_cast<cudaStream_t>(stream));
}

int mxfp6_gemm_w6a8_static_scratch(const uint8_t* a_values, const uint8_t* a_scales,
                                   const uint8_t* w_values, const uint8_t* w_scales, int64_t m,
                                   int64_t n, int64_t k, float alpha, void* out, int out_dtype,
                                   void* stream) {
  GemmProblem p;
  if (int rc = dense_problem(&p, a_values, a_scales, w_values, w_scales, m, n, k, alpha, out,
                             out_dtype))
    return rc;
  return launch_w6a8_static_scratch(p, static_cast<cudaStream_t>(stream));
}

int mxfp6_set_stream_kernel_mode(int enabled) {
  set_stream_kernel_mode(enabled);
  return kOk;
}
int mxfp6_get_stream_kernel_mode(void) { return stream_kernel_mode(); }

const char* mxfp6_w6a8_config_abi(void) { return kW6A8ConfigAbi; }
int mxfp6_w6a8_config_count(void) { return kW6A8Candidates; }
int mxfp6_w6a8_config_describe(int config_id, int out[4]) {
  MX_REQUIRE(out != nullptr, "out must not be null");
  return describe_w6a8_candidate(config_id, out);
}

int mxfp6_set_w6a8_config(int64_t m, int64_t n, int64_t k, int out_dtype, int config_id) {
  MX_REQUIRE(m > 0, "m must be positive; got %lld", (long long)m);
  MX_REQUIRE(n > 0 && n % 8 == 0, "n must be a positive multiple of 8; got %lld", (long long)n);
  MX_REQUIRE(k > 0 && k % 128 == 0, "k must be a positive multiple of 128; got %lld",
             (long long)k);
  MX_REQUIRE(out_dtype == kF16 || out_dtype == kBF16, "out_dtype must be float16 or bfloat16");
  int device = 0;
  MX_CUDA(cudaGetDevice(&device));
  const ShapeKey key{device, m, n, k, out_dtype};
  if (config_id < 0) {
    std::unique_lock<std::shared_mutex> lock(g_override_mutex);
    g_overrides.erase(key);
    return kOk;
  }
  MX_REQUIRE(config_id < kW6A8Candidates, "config_id must be in [0, %d], or negative to erase; got %d",
             kW6A8Candidates - 1, config_id);
  // Reject a configuration that cannot run this problem now, not at the first launch.
  GemmProblem p;
  if (int rc = dense_problem(&p, nullptr, nullptr, nullptr, nullptr, m, n, k, 1.0f, nullptr,
                             out_dtype))
    return rc;
  if (int rc = apply_w6a8_candidate(config_id, &p)) return rc;
  GemmPlan plan;
  if (int rc = plan_w6a8(p, &plan)) return rc;
  std::unique_lock<std::shared_mutex> lock(g_override_mutex);
  g_overrides[key] = config_id;
  return kOk;
}

int mxfp6_gemm_w6a8_config(const uint8_t* a_values, const uint8_t* a_scales,
                           const uint8_t* w_values, const uint8_t* w_scales, int64_t m, int64_t n,
                           int64_t k, float alpha, void* out, int out_dtype, int config_id,
                           void* stream) {
  GemmProblem p;
  if (int rc = dense_problem(&p, a_values, a_scales, w_values, w_scales, m, n, k, alpha, out,
                             out_dtype))
    return rc;
  if (int rc = apply_w6a8_candidate(config_id, &p)) return rc;
  return run_gemm_with_arena(p, static_cast<cudaStream_t>(stream));
}

int mxfp6_gemm_w6a8_plan(int64_t m, int64_t n, int64_t k, int tile_tokens, int splits,
                         int64_t out_plan[10]) {
  MX_REQUIRE(out_plan != nullptr, "out_plan must not be null");
  GemmProblem p;
  if (int rc = dense_problem(&p, nullptr, nullptr, nullptr, nullptr, m, n, k, 1.0f, nullptr,
                             kBF16))
    return rc;
  p.tile_tokens = tile_tokens;
  p.splits = splits;
  if (tile_tokens == 0 && splits == 0) {
    if (int rc = apply_override(&p)) return rc;
  }
  GemmPlan plan;
  if (int rc = plan_w6a8(p, &plan)) return rc;
  out_plan[0] = plan.tile_tokens;
  out_plan[1] = plan.splits;
  out_plan[2] = plan.stages;
  out_plan[3] = plan.grid;
  out_plan[4] = (int64_t)((plan.partial_bytes + 255) & ~size_t(255));
  out_plan[5] = (int64_t)plan.counter_bytes;
  out_plan[6] = plan.cluster_k;
  out_plan[7] = plan.cta_pair;
  out_plan[8] = plan.kernel;
  out_plan[9] = (int64_t)plan.smem_bytes;
  return kOk;
}

int mxfp6_gemm_from_float(const void* a, int a_dtype, const uint8_t* w_values,
                          const uint8_t* w_scales, int64_t m, int64_t n, int64_t k, float alpha,
                          void* out, int out_dtype, uint8_t* a_values_stage,
                          uint8_t* a_scales_stage, void* stream) {
  MX_REQUIRE(a_values_stage != nullptr && a_scales_stage != nullptr,
             "staging buffers must not be null");
  GemmProblem p;
  if (int rc = dense_problem(&p, a_values_stage, a_scales_stage, w_values, w_scales, m, n, k,
                             alpha, out, out_dtype))
    return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (int rc = quantize_mxfp8(a, a_dtype, m, k, a_values_stage, a_scales_stage, nullptr, s))
    return rc;
  return run_gemm_with_arena(p, s);
}

int mxfp6_grouped_gemm_w6a8(void* out, int out_dtype, const uint8_t* activation,
                            const uint8_t* activation_scales, int64_t activation_scale_rows,
                            const uint8_t* weight, const uint8_t* weight_scales,
                            const int64_t* expert_offsets, const int64_t* scale_offsets,
                            int experts, int64_t m_total, int64_t n, int64_t k, int tile_tokens,
                            void* stream) {
  MX_REQUIRE(expert_offsets != nullptr && scale_offsets != nullptr,
             "expert_offsets and scale_offsets must not be null");
  GemmProblem p;
  if (int rc = dense_problem(&p, activation, activation_scales, weight, weight_scales, m_total, n,
                             k, 1.0f, out, out_dtype))
    return rc;
  p.groups = experts;
  p.expert_offsets = expert_offsets;
  p.scale_offsets = scale_offsets;
  p.a_scale_rows = activation_scale_rows;
  p.tile_tokens = tile_tokens;
  p.splits = 1;
  GemmPlan plan;
  if (int rc = plan_w6a8(p, &plan)) return rc;
  return launch_w6a8(p, plan, static_cast<cudaStream_t>(stream));
}

int mxfp6_w1_swiglu_mxfp8(uint8_t* output, uint8_t* out_packed_scales,
                          uint8_t* out_logical_scales, const uint8_t* activation,
                          const uint8_t* activation_scales, int64_t activation_scale_rows,
                          const uint8_t* weight, const uint8_t* weight_scales,
                          const int64_t* expert_offsets, const int64_t* scale_offsets,
                          int experts, int64_t m_total, int64_t inter, int64_t k, int tile_tokens,
                          void* stream) {
  MX_REQUIRE((expert_offsets == nullptr) == (scale_offsets == nullptr),
             "expert_offsets and scale_offsets go together");
  MX_REQUIRE(expert_offsets != nullptr || experts == 1, "a dense launch has exactly one weight");
  GemmProblem p;
  if (int rc = dense_problem(&p, activation, activation_scales, weight, weight_scales, m_total,
                             inter, k, 1.0f, output, kBF16))
    return rc;
  p.mode = kGemmSwigluMxfp8;
  p.groups = experts;
  p.expert_offsets = expert_offsets;
  p.scale_offsets = scale_offsets;
  p.out_scale_offsets = scale_offsets;
  p.out_packed_scales = out_packed_scales;
  p.out_logical_scales = out_logical_scales;
  p.a_scale_rows = activation_scale_rows;
  p.tile_tokens = tile_tokens;
  p.splits = 1;
  GemmPlan plan;
  if (int rc = plan_w6a8(p, &plan)) return rc;
  return launch_w6a8(p, plan, static_cast<cudaStream_t>(stream));
}

int mxfp6_moe_topk_quant(const void* hidden, const void* logits, int64_t tokens, int hidden_size,
                         int experts, int topk, int renormalize, uint8_t* quantized,
                         uint8_t* logical_scales, uint8_t* dense_scales, float* topk_weights,
                         int32_t* topk_ids, void* stream) {
  return moe_topk_quant(hidden, logits, tokens, hidden_size, experts, topk, renormalize, quantized,
                        logical_scales, dense_scales, topk_weights, topk_ids,
                        static_cast<cudaStream_t>(stream));
}

int mxfp6_moe_route(const uint8_t* activation, const uint8_t* logical_scales, const void* topk_ids,
                    int ids_are_int64, int64_t tokens, int topk, int hidden_size,
                    const int32_t* expert_map, int expert_map_size, int local_experts,
                    int64_t* expert_offsets, int64_t* scale_offsets, int32_t* cursors,
                    uint8_t* permuted, uint8_t* grouped_scales, int32_t* inverse_permutation,
                    int32_t* source_tokens, void* stream) {
  return moe_route(activation, logical_scales, topk_ids, ids_are_int64, tokens, topk, hidden_size,
                   expert_map, expert_map_size, local_experts, 0, expert_offsets, scale_offsets,
                   cursors, permuted, grouped_scales, inverse_permutation, source_tokens,
                   static_cast<cudaStream_t>(stream));
}

int mxfp6_moe_route_shared(const uint8_t* activation, const uint8_t* logical_scales,
                           const void* topk_ids, int ids_are_int64, int64_t tokens, int topk,
                           int hidden_size, const int32_t* expert_map, int expert_map_size,
                           int local_experts, int include_shared, int64_t* expert_offsets,
                           int64_t* scale_offsets, int32_t* cursors, uint8_t* permuted,
                           uint8_t* grouped_scales, int32_t* inverse_permutation,
                           int32_t* source_tokens, void* stream) {
  return moe_route(activation, logical_scales, topk_ids, ids_are_int64, tokens, topk, hidden_size,
                   expert_map, expert_map_size, local_experts, include_shared ? 1 : 0,
                   expert_offsets, scale_offsets, cursors, permuted, grouped_scales,
                   inverse_permutation, source_tokens, static_cast<cudaStream_t>(stream));
}

int mxfp6_moe_topk_quant_route(const void* hidden, const void* logits, int64_t tokens,
                               int hidden_size, int experts, int topk, int renormalize,
                               uint8_t* quantized, uint8_t* logical_scales, uint8_t* dense_scales,
                               float* topk_weights, int32_t* topk_ids, const int32_t* expert_map,
                               int expert_map_size, int local_experts, int64_t* expert_offsets,
                               int64_t* scale_offsets, int32_t* cursors, uint8_t* permuted,
                               uint8_t* grouped_scales, int32_t* inverse_permutation,
                               int32_t* source_tokens, void* stream) {
  return moe_topk_quant_route(hidden, logits, tokens, hidden_size, experts, topk, renormalize,
                              quantized, logical_scales, dense_scales, topk_weights, topk_ids,
                              expert_map, expert_map_size, local_experts, expert_offsets,
                              scale_offsets, cursors, permuted, grouped_scales,
                              inverse_permutation, source_tokens,
                              static_cast<cudaStream_t>(stream));
}

int mxfp6_silu_and_mul_mxfp8(const void* input, int dtype, int64_t rows, int64_t inter,
                             uint8_t* output, uint8_t* logical_scales, uint8_t* packed_scales,
                             const int64_t* expert_offsets, const int64_t* scale_offsets,
                             int experts, void* stream) {
  MX_REQUIRE(inter > 0 && inter <= INT32_MAX, "intermediate size out of range");
  return silu_mul_quant(input, dtype, rows, (int)inter, output, logical_scales, packed_scales,
                        expert_offsets, scale_offsets, experts, static_cast<cudaStream_t>(stream));
}

int mxfp6_moe_reduce(void* out, const void* routed, int dtype, const float* topk_weights,
                     const int32_t* inverse_permutation, const void* shared,
                     const void* shared_gate, int gate_dtype, int gate_stride, int64_t tokens,
                     int hidden_size, int topk, int64_t routed_rows, void* stream) {
  return moe_reduce(out, routed, dtype, topk_weights, inverse_permutation, shared, shared_gate,
                    gate_dtype, gate_stride, tokens, hidden_size, topk, routed_rows,
                    static_cast<cudaStream_t>(stream));
}

int mxfp6_moe_reduce_tp_pointers(void* out, const void* routed, const float* topk_weights,
                                 const int32_t* inverse_permutation, const void* shared,
                                 const void* shared_gate, int gate_dtype, int gate_stride,
                                 int64_t tokens, int hidden_size, int topk, int64_t routed_rows,
                                 const uint64_t* signal_ptrs, const uint64_t* buffer_ptrs,
                                 int world, int rank, void* stream) {
  MX_REQUIRE(signal_ptrs != nullptr && buffer_ptrs != nullptr && world >= 1 && world <= 8 &&
                 rank >= 0 && rank < world,
             "world must be in [1, 8], rank inside it, pointer lists non-null");
  void* partial = reinterpret_cast<void*>(static_cast<uintptr_t>(buffer_ptrs[rank]));
  if (int rc = moe_reduce(partial, routed, kBF16, topk_weights, inverse_permutation, shared,
                          shared_gate, gate_dtype, gate_stride, tokens, hidden_size, topk,
                          routed_rows, static_cast<cudaStream_t>(stream)))
    return rc;
  return tp_allreduce_pointers(signal_ptrs, buffer_ptrs, world, rank, out, tokens, hidden_size,
                               static_cast<cudaStream_t>(stream));
}

int mxfp6_array_gemm_w6a8(void* output, int out_dtype, const uint8_t* activation,
                          const uint8_t* logical_scales, int64_t activation_rows,
                          const uint8_t* weight, const uint8_t* weight_scales, int experts,
                          const void* topk_ids, int ids_are_int64, int64_t tokens, int topk,
                          int include_shared, int64_t n, int64_t k, void* stream) {
  return moe_route_gemm(output, nullptr, out_dtype, 0, activation, logical_scales, activation_rows,
                        weight, weight_scales, experts, nullptr, nullptr, topk_ids, ids_are_int64,
                        tokens, topk, include_shared, n, k, static_cast<cudaStream_t>(stream));
}

int mxfp6_array_gemm_w6a8_silu_mxfp8(uint8_t* output, uint8_t* output_scales,
                                     const uint8_t* activation, const uint8_t* logical_scales,
                                     int64_t activation_rows, const uint8_t* weight,
                                     const uint8_t* weight_scales, int experts,
                                     const uint8_t* shared_weight,
                                     const uint8_t* shared_weight_scales, const void* topk_ids,
                                     int ids_are_int64, int64_t tokens, int topk,
                                     int include_shared, int64_t inter, int64_t k, void* stream) {
  return moe_route_gemm(output, output_scales, kBF16, 1, activation, logical_scales,
                        activation_rows, weight, weight_scales, experts, shared_weight,
                        shared_weight_scales, topk_ids, ids_are_int64, tokens, topk,
                        include_shared, inter, k, static_cast<cudaStream_t>(stream));
}

int mxfp6_array_gemm_w6a8_reduce(void* output, int out_dtype, const uint8_t* activation,
                                 const uint8_t* logical_scales, const uint8_t* weight,
                                 const uint8_t* weight_scales, int experts,
                                 const uint8_t* shared_weight, const uint8_t* shared_weight_scales,
                                 const void* topk_ids, int ids_are_int64, const float* topk_weights,
                                 const void* shared_gate, int gate_dtype, int gate_stride,
                                 const void* shared_output, int compute_shared, int64_t tokens,
                                 int topk, int64_t n, int64_t k, int routing_ready, void* stream) {
  return moe_route_w2_reduce(output, out_dtype, activation, logical_scales, weight, weight_scales,
                             experts, shared_weight, shared_weight_scales, topk_ids, ids_are_int64,
                             topk_weights, shared_gate, gate_dtype, gate_stride, shared_output,
                             compute_shared, tokens, topk, n, k, routing_ready, nullptr, 0, 0,
                             static_cast<cudaStream_t>(stream));
}

int mxfp6_moe_decode_layer_supported(int64_t tokens, int topk, int logit_experts,
                                     int64_t hidden_size, int64_t inter) {
  return moe_decode_layer_supported(tokens, topk, logit_experts, hidden_size, inter);
}

int mxfp6_moe_decode_layer_preferred(int64_t tokens, int topk, int logit_experts,
                                     int64_t hidden_size, int64_t inter) {
  return moe_decode_layer_preferred(tokens, topk, logit_experts, hidden_size, inter);
}

int mxfp6_moe_decode_layer(void* output, int out_dtype, const void* hidden, const void* router_logits,
                           const void* shared_gate, int gate_dtype, int gate_stride,
                           const uint8_t* w1, const uint8_t* w1_scales, const uint8_t* w2,
                           const uint8_t* w2_scales, int experts, const uint8_t* shared_w1,
                           const uint8_t* shared_w1_scales, const uint8_t* shared_w2,
                           const uint8_t* shared_w2_scales, uint8_t* activation,
                           uint8_t* activation_scales, int32_t* topk_ids, float* topk_weights,
                           int64_t tokens, int topk, int logit_experts, int renormalize,
                           int64_t hidden_size, int64_t inter, int w2_own_routing, void* stream) {
  return moe_decode_layer(output, out_dtype, hidden, router_logits, shared_gate, gate_dtype,
                          gate_stride, w1, w1_scales, w2, w2_scales, experts, shared_w1,
                          shared_w1_scales, shared_w2, shared_w2_scales, activation,
                          activation_scales, topk_ids, topk_weights, tokens, topk, logit_experts,
                          renormalize, hidden_size, inter, w2_own_routing,
                          static_cast<cudaStream_t>(stream));
}

int mxfp6_moe_reduce_array(void* output, const void* combined, int dtype, const float* topk_weights,
                           const void* shared_gate, int gate_dtype, int gate_stride, int64_t tokens,
                           int topk, int64_t hidden_size, void* stream) {
  return moe_reduce_array(output, combined, dtype, topk_weights, shared_gate, gate_dtype,
                          gate_stride, tokens, topk, hidden_size, static_cast<cudaStream_t>(stream));
}

int mxfp6_moe_router_logits(const void* hidden, const void* gate_weight,
                            const void* shared_gate_weight, void* routed_logits, void* shared_gate,
                            int64_t batch, int64_t k, int routed_experts, int gate_rows,
                            void* stream) {
  return moe_router_logits(hidden, gate_weight, shared_gate_weight, routed_logits, shared_gate,
                           batch, k, routed_experts, gate_rows, static_cast<cudaStream_t>(stream));
}

int mxfp6_workspace_begin_planning(void) {
  int device = 0;
  MX_CUDA(cudaGetDevice(&device));
  std::lock_guard<std::mutex> lock(g_arena_mutex);
  Arena& arena = g_arenas[device];
  if (arena.mode == ArenaMode::Frozen) {
    set_error(
        "persistent split-K workspace for CUDA device %d is already frozen; resizing it could "
        "invalidate captured graphs",
        device);
    return kWorkspaceError;
  }
  if (arena.mode == ArenaMode::Planning) {
    set_error("workspace planning is already active for CUDA device %d", device);
    return kWorkspaceError;
  }
  arena = Arena{};
  arena.mode = ArenaMode::Planning;
  return kOk;
}

int mxfp6_workspace_finalize_planning(void* stream, int64_t out_stats[10]) {
  MX_REQUIRE(out_stats != nullptr, "out_stats must not be null");
  int device = 0;
  MX_CUDA(cudaGetDevice(&device));
  std::lock_guard<std::mutex> lock(g_arena_mutex);
  auto it = g_arenas.find(device);
  if (it == g_arenas.end() || it->second.mode != ArenaMode::Planning) {
    set_error("workspace planning is not active for CUDA device %d", device);
    return kWorkspaceError;
  }
  Arena& arena = it->second;
  if (arena.max_reduction_bytes + arena.max_barrier_bytes > 0) {
    arena.max_reduction_bytes = (arena.max_reduction_bytes + 255) & ~size_t(255);
    Lane lane;
    if (int rc = new_lane(arena, static_cast<cudaStream_t>(stream), &lane)) return rc;
    arena.lanes.push_back(lane);
  }
  arena.mode = ArenaMode::Frozen;
  fill_stats(arena, out_stats);
  return kOk;
}

int mxfp6_workspace_stats(int64_t out_stats[10]) {
  MX_REQUIRE(out_stats != nullptr, "out_stats must not be null");
  int device = 0;
  MX_CUDA(cudaGetDevice(&device));
  std::lock_guard<std::mutex> lock(g_arena_mutex);
  auto it = g_arenas.find(device);
  if (it == g_arenas.end()) {
    fill_stats(Arena{}, out_stats);
  } else {
    fill_stats(it->second, out_stats);
  }
  return kOk;
}

int mxfp6_workspace_barriers_zero(int* all_zero) {
  MX_REQUIRE(all_zero != nullptr, "all_zero must not be null");
  int device = 0;
  MX_CUDA(cudaGetDevice(&device));
  std::vector<uint8_t*> tails;
  size_t bytes = 0;
  {
    std::lock_guard<std::mutex> lock(g_arena_mutex);
    auto it = g_arenas.find(device);
    if (it == g_arenas.end() || it->second.mode != ArenaMode::Frozen) {
      set_error("persistent workspace is not frozen for CUDA device %d", device);
      return kWorkspaceError;
    }
    bytes = it->second.max_barrier_bytes;
    for (const Lane& lane : it->second.lanes) {
      tails.push_back(lane.storage + it->second.max_reduction_bytes);
    }
  }
  *all_zero = 1;
  if (bytes == 0) return kOk;
  MX_CUDA(cudaDeviceSynchronize());
  std::vector<uint8_t> host(bytes);
  for (uint8_t* tail : tails) {
    MX_CUDA(cudaMemcpy(host.data(), tail, bytes, cudaMemcpyDeviceToHost));
    if (!std::all_of(host.begin(), host.end(), [](uint8_t v) { return v == 0; })) {
      *all_zero = 0;
      return kOk;
    }
  }
  return kOk;
}

int mxfp6_workspace_reset(void) {
  int device = 0;
  MX_CUDA(cudaGetDevice(&device));
  MX_CUDA(cudaDeviceSynchronize());
  std::lock_guard<std::mutex> lock(g_arena_mutex);
  auto it = g_arenas.find(device);
  if (it != g_arenas.end()) {
    for (Lane& lane : it->second.lanes) cudaFree(lane.storage);
    g_arenas.erase(it);
  }
  return kOk;
}

}  // extern "C"
