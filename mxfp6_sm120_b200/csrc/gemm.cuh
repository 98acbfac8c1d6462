// Host-visible description of one W6A8 GEMM launch (dense or row-grouped).
#pragma once

#include "common.cuh"

namespace mx {

// Epilogue selector of the tcgen05 kernel.
enum GemmMode : int {
  kGemmStore = 0,        // out[row, f] = cast(alpha * acc), FP16/BF16
  // Weights hold 2 * n rows per group (gate rows, then up rows).  out[row, f] =
  // MXFP8 of bf16(silu(bf16(gate)) ) * bf16(up) with one UE8M0 scale per 32 features
  // (the reference's fused W1 epilogue, csrc/moe.cu:2226-2235).
  kGemmSwigluMxfp8 = 1,
};

// Kernel family a plan runs on.
enum GemmKernel : int {
  kKernelPersistent = 0,  // gemm.cu: one CTA per tile, any mode, cluster or scratch split-K
  kKernelPair = 1,        // gemm_pair.cu: CTA pairs (cta_group::2), m > 128
  kKernelStream = 2,      // gemm_stream.cu: decode batches, two CTAs per SM, weight prefetch
};

struct GemmProblem {
  // Weights: `groups` matrices of [n, k] E3M2 codes, packed rows of k*3/4 bytes,
  // stored back to back; packed scales likewise (n % 128 == 0 when groups > 1).
  const uint8_t* w_values = nullptr;
  const uint8_t* w_scales = nullptr;
  // Activations: [m_total, k] E4M3 bytes with packed scales.  For grouped
  // launches rows [expert_offsets[g], expert_offsets[g+1]) belong to matrix g and
  // their scales start at packed row scale_offsets[g] (a multiple of 128).
  const uint8_t* a_values = nullptr;
  const uint8_t* a_scales = nullptr;
  int64_t a_scale_rows = 0;  // padded row count of the activation scale buffer
  const int64_t* expert_offsets = nullptr;  // device, groups + 1 entries, or null (dense)
  const int64_t* scale_offsets = nullptr;   // device, groups + 1 entries, or null (dense)
  int groups = 1;
  int64_t m_total = 0;
  int n = 0;
  int k = 0;
  float alpha = 1.0f;
  void* out = nullptr;  // [m_total, n]
  int out_dtype = kBF16;
  // Split-K scratch: fp32 partial tiles and one counter per output tile.
  float* partials = nullptr;
  size_t partial_bytes = 0;
  uint32_t* counters = nullptr;
  size_t counter_bytes = 0;
  int mode = kGemmStore;
  // SwiGLU mode outputs: scales of the E4M3 result, logical [m_total, n/32] and/or
  // packed; out_scale_offsets (device, groups + 1) maps group rows to packed rows.
  uint8_t* out_packed_scales = nullptr;
  uint8_t* out_logical_scales = nullptr;
  const int64_t* out_scale_offsets = nullptr;
  // Status word the kernel reports an expired wait to; null = the per-device word.
  int* status_word = nullptr;
  // How K is split when a launch has too few tiles for the GPU: 0 = library default,
  // 1 = thread-block clusters reducing through distributed shared memory,
  // 2 = FP32 partial tiles in the scratch arena, 3 = never split.
  int split_mode = 0;
  int cluster_k = 0;  // explicit cluster size along K (0 = choose)
  // Optional overrides (0 = choose from the static table).
  int tile_tokens = 0;
  int splits = 0;
  int force_kernel = -1;  // a GemmKernel value, or -1 = choose
};

struct GemmPlan {
  int kernel = kKernelPersistent;
  int tile_tokens = 0;  // activation rows per tile (MMA N)
  int splits = 1;      // scratch-arena split-K factor
  int cluster_k = 1;   // cluster split-K factor (CTAs per cluster)
  int cta_pair = 0;    // 1: the two-CTA (cta_group::2) kernel computes 256-feature tiles
  int stages = 0;
  int grid = 0;
  size_t smem_bytes = 0;
  size_t partial_bytes = 0;   // scratch the plan needs when splits > 1
  size_t counter_bytes = 0;
};

// Chooses tile/split-K for a problem; pure host arithmetic.
int plan_w6a8(const GemmProblem& p, GemmPlan* plan);
// Launches the kernel on `stream`; the plan must come from plan_w6a8.
int launch_w6a8(const GemmProblem& p, const GemmPlan& plan, cudaStream_t stream);

// Explicit configurations ("candidates") of the dense GEMM, the counterpart of the
// reference's 30 ahead-of-time kernels (csrc/torch_extension.cu:979-1137): an id names a
// kernel family, a token tile and a K split.  apply_w6a8_candidate writes the overrides
// of candidate `id` into `p`.
constexpr int kW6A8Candidates = 58;
extern const char* const kW6A8ConfigAbi;
int describe_w6a8_candidate(int id, int out[4]);  // kernel, tile_tokens, cluster_k, splits
int apply_w6a8_candidate(int id, GemmProblem* p);

// Process-wide default of GemmProblem::split_mode (1 = cluster, 2 = scratch arena, 3 = off).
void set_default_split_mode(int mode);
int default_split_mode();

// Weight-streaming kernel for dense launches of at most 32 rows (default on).
void set_stream_kernel_mode(int enabled);
int stream_kernel_mode();
// Two-CTA kernel for dense store-mode launches with m > 128 and n % 256 == 0 (default on).
void set_cta_pair_mode(int enabled);
int cta_pair_mode();

// GEMM whose split-K scratch and status word live in a fixed array inside the
// library image, for callers that must not allocate device memory.
int launch_w6a8_static_scratch(GemmProblem& p, cudaStream_t stream);

// Device status word (0 = ok) shared by all kernels with bounded waits.
int* device_status_word(int device);
int read_device_status(int device, int* value, bool reset);

}  // namespace mx
