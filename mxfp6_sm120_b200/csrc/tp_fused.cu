// Tensor-parallel decode path: all-reduce of a row-parallel projection fused with the
// residual add, RMSNorm and MXFP8 quantization that consume it, over peer memory.
//
// Every rank of one node owns a "symmetric" block (one cudaMalloc, exported with CUDA IPC
// and mapped by its peers): a flag word per rank, a small state record and two partial
// buffers.  A row-parallel GEMM writes its [M, hidden] BF16 partial into one of its OWN
// partial buffers (plain local stores).  The consumer kernel on every rank then
//   1. tells every peer "my partial of this step is complete" (one 32-bit store into the
//      peer's flag array, after a system-scope fence; the GEMM ended earlier on the stream),
//   2. waits (bounded) until every rank's flag has reached this step,
//   3. loads the same row from all ranks' buffers over NVLink (plain peer loads, no
//      multicast), sums them in rank order in FP32 -> BF16 (every rank forms the same
//      sum, so the replicas of the residual stream stay bit-identical),
//   4. adds the residual stream, normalises, quantizes (as rmsnorm_quantize_mxfp8).
// So the collective costs one flag round trip plus the peer loads; nothing is written to a
// peer but the flag.  The reference's counterpart is the two-rank reducer with peer signal
// pointers and unbounded spins (csrc/moe.cu:7698-7925).
//
// Buffers alternate (the projection before the first norm of a layer uses buffer 0, the one
// before the second norm buffer 1): a rank that has passed step s + 1 has seen every peer
// finish step s, so a buffer is rewritten only after all its readers are done.
// The step number lives in device memory and is advanced by the last CTA of the kernel,
// which keeps CUDA-graph replays correct.  So does the number of the buffer the last step
// used: a step that names the same buffer again (a captured graph with an odd number of
// collectives, replayed) records code 302 and moves no data instead of racing with a peer
// that may still be reading.  Every wait is bounded (about 2 s unless
// mxfp6_tp_set_wait_limit shortens it): on expiry the kernel records code 301 in the
// status word and returns without touching peer data.
#include "common.cuh"

#include <cuda_fp8.h>
#include <cstring>

namespace mx {

int* device_status_word(int device);  // gemm.cu: one status word per device

constexpr int kTpMaxRanks = 8;
constexpr int kTpThreads = 256;
constexpr int kTpChunks = 8;  // 8-value chunks per thread: hidden <= 16384
constexpr size_t kTpHeaderBytes = 1024;

struct TpState {
  uint32_t done_step;    // steps this rank has completed
  uint32_t finished;     // CTAs of the running kernel that are done
  uint32_t last_buffer;  // 1 + the partial buffer the last completed step used (0: none yet)
};

struct TpPeers {
  const void* partial[kTpMaxRanks];  // every rank's partial buffer of this step (peer mapped)
  uint32_t* flags[kTpMaxRanks];      // every rank's flag array (index = sender)
  int world;
  int rank;
  int buffer;             // which of the two partial buffers this step reads
  int second_phase;       // 1: this step re-reads the buffer of the step before it (see below)
  long long wait_cycles;  // limit of the flag wait in clock64 ticks
};

namespace {

__device__ __forceinline__ uint32_t ld_volatile_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_volatile_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_volatile_u128(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

__device__ __forceinline__ void unpack_bf16x8(const uint4& raw, float (&v)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ uint4 pack_bf16x8(const float (&v)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t lo = __bfloat16_as_ushort(__float2bfloat16_rn(v[2 * i]));
    const uint32_t hi = __bfloat16_as_ushort(__float2bfloat16_rn(v[2 * i + 1]));
    w[i] = lo | (hi << 16);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// Signals "my partial of this step is complete" to every peer (block 0), waits (bounded)
// for every rank's signal, and returns the step number; *ok_shared is 0 after a timeout.
__device__ __forceinline__ uint32_t tp_handshake(const TpPeers& peers, TpState* state, int* status,
                                                 uint32_t* step_shared, int* ok_shared) {
  if (threadIdx.x == 0) {
    *step_shared = ld_volatile_u32(&state->done_step) + 1u;
    *ok_shared = 1;
    // Two steps in a row on one buffer: a peer may still be reading what the producer of
    // this step has just overwritten.  The handshake still runs (the ranks stay in step),
    // the data phase does not.
    // (The second phase of a two-phase all-reduce gathers the slices the first phase has
    // just reduced in place: nothing produced that buffer again in between.)
    if (peers.world > 1 && peers.second_phase == 0 &&
        ld_volatile_u32(&state->last_buffer) == (uint32_t)peers.buffer + 1u) {
      *ok_shared = 0;
      atomicCAS(status, 0, 302);
    }
  }
  __syncthreads();
  const uint32_t step = *step_shared;
  if (blockIdx.x == 0 && threadIdx.x < peers.world) {
    // The kernel that wrote this rank's partial finished earlier on this stream; the fence
    // orders its (already performed) writes before the flag for observers on other GPUs.
    __threadfence_system();
    st_volatile_u32(peers.flags[threadIdx.x] + peers.rank, step);
  }
  if (threadIdx.x < peers.world) {
    const uint32_t* flag = peers.flags[peers.rank] + threadIdx.x;
    const long long start = clock64();
    bool seen = false;
#pragma unroll 1
    for (uint32_t spin = 0;; ++spin) {
      if (static_cast<int32_t>(ld_volatile_u32(flag) - step) >= 0) {
        seen = true;
        break;
      }
      if ((spin & 255u) == 255u && clock64() - start > peers.wait_cycles) break;
    }
    if (!seen) {
      *ok_shared = 0;
      atomicCAS(status, 0, 301);
    }
    __threadfence_system();
  }
  __syncthreads();
  return step;
}

// The last CTA advances the step (also after a timeout, so that the ranks stay aligned).
__device__ __forceinline__ void tp_finish(TpState* state, uint32_t step, int buffer) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t done = atomicAdd(&state->finished, 1u);
    if (done == gridDim.x - 1) {
      state->finished = 0u;
      st_volatile_u32(&state->last_buffer, (uint32_t)buffer + 1u);
      st_volatile_u32(&state->done_step, step);
      __threadfence();
    }
  }
}

// out[row] <- bf16(sum over ranks, in rank order, of partial_r[row]): the plain all-reduce,
// for consumers that are not a norm (the MoE reducer's tensor-parallel sum).
__global__ void __launch_bounds__(kTpThreads)
allreduce_sum_kernel(const TpPeers peers, TpState* state, __nv_bfloat16* out, int64_t chunks,
                     int* status) {
  __shared__ uint32_t step_shared;
  __shared__ int ok_shared;
  const uint32_t step = tp_handshake(peers, state, status, &step_shared, &ok_shared);
  if (ok_shared != 0) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t c = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; c < chunks;
         c += stride) {
      uint4 part[kTpMaxRanks];
#pragma unroll
      for (int r = 0; r < kTpMaxRanks; ++r) {
        if (r < peers.world) {
          part[r] = ld_volatile_u128(reinterpret_cast<const uint4*>(peers.partial[r]) + c);
        }
      }
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < kTpMaxRanks; ++r) {
        if (r < peers.world) {
          float v[8];
          unpack_bf16x8(part[r], v);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] += v[i];
        }
      }
      reinterpret_cast<uint4*>(out)[c] = pack_bf16x8(acc);
    }
  }
  tp_finish(state, step, peers.buffer);
}

// out <- bf16(sum over ranks of rows [first_chunk, first_chunk + chunks) of every rank's buffer):
// the reduce-scatter form (every rank sums ITS slice of all the partials), used by the
// expert-parallel combine.
__global__ void __launch_bounds__(kTpThreads)
reduce_scatter_kernel(const TpPeers peers, TpState* state, __nv_bfloat16* out, int64_t first_chunk,
                      int64_t chunks, int* status) {
  __shared__ uint32_t step_shared;
  __shared__ int ok_shared;
  const uint32_t step = tp_handshake(peers, state, status, &step_shared, &ok_shared);
  if (ok_shared != 0) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t c = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; c < chunks;
         c += stride) {
      uint4 part[kTpMaxRanks];
#pragma unroll
      for (int r = 0; r < kTpMaxRanks; ++r) {
        if (r < peers.world) {
          part[r] = ld_volatile_u128(reinterpret_cast<const uint4*>(peers.partial[r]) +
                                     first_chunk + c);
        }
      }
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < kTpMaxRanks; ++r) {
        if (r < peers.world) {
          float v[8];
          unpack_bf16x8(part[r], v);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] += v[i];
        }
      }
      reinterpret_cast<uint4*>(out)[c] = pack_bf16x8(acc);
    }
  }
  tp_finish(state, step, peers.buffer);
}

// All-gather of up to four byte segments: segment s of rank r (at seg_offset[s] inside r's
// buffer) lands at dst[s] + r * seg_bytes[s].  One handshake for the whole payload (the
// expert-parallel dispatch: MXFP8 rows, scale rows, top-k ids and weights).
struct TpSegments {
  int count;
  int rank_strided;   // 1: rank r's segment starts at offset + r * bytes (slices of one tensor)
  int64_t offset[4];  // bytes from the start of the partial buffer, multiples of 16
  int64_t bytes[4];   // multiples of 16
  uint8_t* dst[4];
};

__global__ void __launch_bounds__(kTpThreads)
allgather_kernel(const TpPeers peers, TpState* state, const TpSegments seg, int* status) {
  __shared__ uint32_t step_shared;
  __shared__ int ok_shared;
  const uint32_t step = tp_handshake(peers, state, status, &step_shared, &ok_shared);
  if (ok_shared != 0) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    // (rank, chunk) pairs are dealt to the threads, so that the loads from different peers
    // are in flight together instead of one NVLink round trip after the other.
    for (int s = 0; s < seg.count; ++s) {
      const int64_t chunks = seg.bytes[s] / 16;
      const int64_t total = chunks * peers.world;
      // Four loads in flight per thread: a bandwidth-bound gather needs megabytes on the wire.
      for (int64_t base = tid; base < total; base += 4 * stride) {
        uint4 v[4];
        int64_t at[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int64_t idx = base + u * stride;
          at[u] = -1;
          if (idx < total) {
            const int r = static_cast<int>(idx / chunks);
            const int64_t c = idx - r * chunks;
            const uint4* src = reinterpret_cast<const uint4*>(
                static_cast<const uint8_t*>(peers.partial[r]) + seg.offset[s] +
                (seg.rank_strided != 0 ? r * seg.bytes[s] : 0));
            v[u] = ld_volatile_u128(src + c);
            at[u] = r * chunks + c;
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (at[u] >= 0) reinterpret_cast<uint4*>(seg.dst[s])[at[u]] = v[u];
        }
      }
    }
  }
  tp_finish(state, step, peers.buffer);
}

// x[row] <- bf16(x[row] + bf16(sum over ranks of partial_r[row])); then RMSNorm * weight and
// MXFP8 with packed scales.  One CTA per row.
template <int kChunks>
__global__ void __launch_bounds__(kTpThreads)
allreduce_rmsnorm_quantize_kernel(const TpPeers peers, TpState* state, __nv_bfloat16* x,
                                  const __nv_bfloat16* __restrict__ weight, float eps,
                                  uint8_t* __restrict__ out, uint8_t* __restrict__ packed,
                                  int64_t rows, int k, int* status) {
  __shared__ float warp_sums[kTpThreads / 32];
  __shared__ uint32_t step_shared;
  __shared__ int ok_shared;
  const int row_chunks = k / 8;
  const int groups = k / kScaleVec;
  const int64_t row = blockIdx.x;

  // ---- the cross-rank handshake -------------------------------------------------------
  const uint32_t step = tp_handshake(peers, state, status, &step_shared, &ok_shared);
  const bool ok = ok_shared != 0;

  if (ok) {
    // ---- all-reduce of this row + residual --------------------------------------------
    uint4 raw[kChunks];
    uint4* xrow = reinterpret_cast<uint4*>(x) + row * row_chunks;
    float sum_sq = 0.0f;
#pragma unroll
    for (int u = 0; u < kChunks; ++u) {
      const int c = u * kTpThreads + threadIdx.x;
      raw[u] = make_uint4(0u, 0u, 0u, 0u);
      if (c < row_chunks) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        // All ranks' loads are issued before the first is used: one NVLink round trip
        // per chunk instead of one per rank.
        uint4 part[kTpMaxRanks];
#pragma unroll
        for (int r = 0; r < kTpMaxRanks; ++r) {
          if (r < peers.world) {
            part[r] = ld_volatile_u128(reinterpret_cast<const uint4*>(peers.partial[r]) +
                                       row * row_chunks + c);
          }
        }
#pragma unroll
        for (int r = 0; r < kTpMaxRanks; ++r) {
          if (r < peers.world) {
            float v[8];
            unpack_bf16x8(part[r], v);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] += v[i];
          }
        }
        float xv[8];
        unpack_bf16x8(xrow[c], xv);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float reduced = __bfloat162float(__float2bfloat16_rn(acc[i]));
          xv[i] = __bfloat162float(__float2bfloat16_rn(xv[i] + reduced));
          sum_sq = fmaf(xv[i], xv[i], sum_sq);
        }
        raw[u] = pack_bf16x8(xv);
        xrow[c] = raw[u];
      }
    }
    // ---- RMSNorm + MXFP8 (as rmsnorm_quantize_mxfp8_kernel) ---------------------------
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) sum_sq += __shfl_xor_sync(0xffffffffu, sum_sq, d);
    if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = sum_sq;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < kTpThreads / 32; ++w) total += warp_sums[w];
    const float inv_rms = rsqrtf(total / static_cast<float>(k) + eps);
    const uint4* wsrc = reinterpret_cast<const uint4*>(weight);
#pragma unroll
    for (int u = 0; u < kChunks; ++u) {
      const int c = u * kTpThreads + threadIdx.x;
      const bool valid = c < row_chunks;
      float v[8], g[8];
      unpack_bf16x8(raw[u], v);
      uint4 wraw = make_uint4(0u, 0u, 0u, 0u);
      if (valid) wraw = __ldg(wsrc + c);
      unpack_bf16x8(wraw, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = round_bf16((v[i] * inv_rms) * g[i]);
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
        uint32_t w2[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const uint32_t lo = __nv_cvt_float2_to_fp8x2(
              make_float2(v[4 * i] * inv, v[4 * i + 1] * inv), __NV_SATFINITE, __NV_E4M3);
          const uint32_t hi = __nv_cvt_float2_to_fp8x2(
              make_float2(v[4 * i + 2] * inv, v[4 * i + 3] * inv), __NV_SATFINITE, __NV_E4M3);
          w2[i] = lo | (hi << 16);
        }
        reinterpret_cast<uint2*>(out)[row * row_chunks + c] = make_uint2(w2[0], w2[1]);
        // groups % 4 == 0 is required by the host: 16 lanes = four groups = one word.
        if ((threadIdx.x & 15) == 0) {
          *reinterpret_cast<uint32_t*>(packed + packed_scale_offset(row, c >> 2, groups)) = word;
        }
      }
    }
  }

  tp_finish(state, step, peers.buffer);
}

}  // namespace

namespace {
long long g_tp_wait_cycles = 4000000000ll;  // about two seconds
}
// Limit of the cross-rank flag wait, in clock64 ticks (about 1.9e9 per second).
void tp_set_wait_limit(long long cycles) {
  g_tp_wait_cycles = cycles < 1000 ? 1000 : (cycles > 40000000000ll ? 40000000000ll : cycles);
}
long long tp_wait_limit() { return g_tp_wait_cycles; }

// ---- symmetric block: allocation and CUDA IPC ------------------------------------------
// Layout: [flags: kTpMaxRanks x u32 | TpState | pad to 1024 B | partial 0 | partial 1].
int tp_block_alloc(size_t partial_bytes, void** block, unsigned char handle[64]) {
  MX_REQUIRE(block != nullptr && handle != nullptr, "pointers must not be null");
  MX_REQUIRE(partial_bytes > 0 && partial_bytes % 256 == 0,
             "the partial buffer size must be a positive multiple of 256 bytes");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handles are 64 bytes");
  void* p = nullptr;
  const size_t bytes = kTpHeaderBytes + 2 * partial_bytes;
  MX_CUDA(cudaMalloc(&p, bytes));
  MX_CUDA(cudaMemset(p, 0, bytes));
  MX_CUDA(cudaDeviceSynchronize());
  cudaIpcMemHandle_t h;
  MX_CUDA(cudaIpcGetMemHandle(&h, p));
  memcpy(handle, &h, 64);
  *block = p;
  return kOk;
}

int tp_block_open(const unsigned char handle[64], void** block) {
  MX_REQUIRE(block != nullptr && handle != nullptr, "pointers must not be null");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  MX_CUDA(cudaIpcOpenMemHandle(block, h, cudaIpcMemLazyEnablePeerAccess));
  return kOk;
}

int tp_block_close(void* block) {
  MX_CUDA(cudaIpcCloseMemHandle(block));
  return kOk;
}

int tp_block_free(void* block) {
  MX_CUDA(cudaFree(block));
  return kOk;
}

int tp_allreduce_rmsnorm_quantize(void* const* blocks, int world, int rank, int buffer,
                                  size_t partial_bytes, void* x, const void* weight, float eps,
                                  int64_t rows, int64_t k, uint8_t* values, uint8_t* packed,
                                  cudaStream_t stream) {
  MX_REQUIRE(blocks != nullptr && world >= 1 && world <= kTpMaxRanks && rank >= 0 && rank < world,
             "world must be in [1, %d] and rank inside it", kTpMaxRanks);
  MX_REQUIRE(buffer == 0 || buffer == 1, "buffer must be 0 or 1");
  MX_REQUIRE(x != nullptr && weight != nullptr && values != nullptr && packed != nullptr,
             "pointers must not be null");
  MX_REQUIRE(rows > 0 && rows <= INT32_MAX, "rows must be positive");
  MX_REQUIRE(k > 0 && k % 128 == 0 && k <= kTpChunks * 8 * kTpThreads,
             "k must be a multiple of 128 and at most %d; got %lld", kTpChunks * 8 * kTpThreads,
             (long long)k);
  MX_REQUIRE((size_t)rows * (size_t)k * 2 <= partial_bytes,
             "the partial buffers hold %zu bytes, %lld x %lld BF16 need more", partial_bytes,
             (long long)rows, (long long)k);
  MX_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(weight) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(values) & 7) == 0 &&
                 (reinterpret_cast<uintptr_t>(packed) & 3) == 0,
             "x / weight must be 16-byte, values 8-byte, scales 4-byte aligned");
  int device = 0;
  MX_CUDA(cudaGetDevice(&device));
  int* status = device_status_word(device);
  if (status == nullptr) return kCudaError;
  TpPeers peers;
  peers.world = world;
  peers.rank = rank;
  peers.buffer = buffer;
  peers.second_phase = 0;
  peers.wait_cycles = g_tp_wait_cycles;
  for (int r = 0; r < kTpMaxRanks; ++r) {
    peers.partial[r] = nullptr;
    peers.flags[r] = nullptr;
  }
  for (int r = 0; r < world; ++r) {
    MX_REQUIRE(blocks[r] != nullptr, "block of rank %d is null", r);
    auto* base = static_cast<uint8_t*>(blocks[r]);
    peers.flags[r] = reinterpret_cast<uint32_t*>(base);
    peers.partial[r] = base + kTpHeaderBytes + (size_t)buffer * partial_bytes;
  }
  auto* state = reinterpret_cast<TpState*>(static_cast<uint8_t*>(blocks[rank]) +
                                           kTpMaxRanks * sizeof(uint32_t));
  // The row lives in registers: instantiate for the 8-value chunks a thread holds.
  const int need = static_cast<int>((k / 8 + kTpThreads - 1) / kTpThreads);
#define MX_LAUNCH_TP(CH)                                                                         \
  allreduce_rmsnorm_quantize_kernel<CH><<<(unsigned)rows, kTpThreads, 0, stream>>>(              \
      peers, state, static_cast<__nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(weight),   \
      eps, values, packed, rows, static_cast<int>(k), status)
  if (need <= 1) MX_LAUNCH_TP(1);
  else if (need <= 2) MX_LAUNCH_TP(2);
  else if (need <= 3) MX_LAUNCH_TP(3);
  else if (need <= 4) MX_LAUNCH_TP(4);
  else MX_LAUNCH_TP(kTpChunks);
#undef MX_LAUNCH_TP
  MX_CUDA(cudaGetLastError());
  return kOk;
}

int tp_allreduce_sum(void* const* blocks, int world, int rank, int buffer, size_t partial_bytes,
                     void* out, int64_t rows, int64_t k, cudaStream_t stream) {
  MX_REQUIRE(blocks != nullptr && world >= 1 && world <= kTpMaxRanks && rank >= 0 && rank < world,
             "world must be in [1, %d] and rank inside it", kTpMaxRanks);
  MX_REQUIRE(buffer == 0 || buffer == 1, "buffer must be 0 or 1");
  MX_REQUIRE(out != nullptr && (reinterpret_cast<uintptr_t>(out) & 15) == 0,
             "out must be a 16-byte aligned device pointer");
  MX_REQUIRE(rows > 0 && k > 0 && k % 8 == 0, "rows must be positive and k a multiple of 8");
  MX_REQUIRE((size_t)rows * (size_t)k * 2 <= partial_bytes,
             "the partial buffers hold %zu bytes, %lld x %lld BF16 need more", partial_bytes,
             (long long)rows, (long long)k);
  int device = 0;
  MX_CUDA(cudaGetDevice(&device));
  int* status = device_status_word(device);
  if (status == nullptr) return kCudaError;
  TpPeers peers;
  peers.world = world;
  peers.rank = rank;
  peers.buffer = buffer;
  peers.second_phase = 0;
  peers.wait_cycles = g_tp_wait_cycles;
  for (int r = 0; r < kTpMaxRanks; ++r) {
    peers.partial[r] = nullptr;
    peers.flags[r] = nullptr;
  }
  for (int r = 0; r < world; ++r) {
    MX_REQUIRE(blocks[r] != nullptr, "block of rank %d is null", r);
    auto* base = static_cast<uint8_t*>(blocks[r]);
    peers.flags[r] = reinterpret_cast<uint32_t*>(base);
    peers.partial[r] = base + kTpHeaderBytes + (size_t)buffer * partial_bytes;
  }
  auto* state = reinterpret_cast<TpState*>(static_cast<uint8_t*>(blocks[rank]) +
                                           kTpMaxRanks * sizeof(uint32_t));
  const int64_t chunks = rows * k / 8;
  int64_t grid = (chunks + kTpThreads - 1) / kTpThreads;
  if (grid > 148 * 4) grid = 148 * 4;
  allreduce_sum_kernel<<<(unsigned)grid, kTpThreads, 0, stream>>>(
      peers, state, static_cast<__nv_bfloat16*>(out), chunks, status);
  MX_CUDA(cudaGetLastError());
  return kOk;
}

namespace {
// Common argument checks and the peer table of the plain collectives.
int tp_prepare(void* const* blocks, int world, int rank, int buffer, size_t partial_bytes,
               TpPeers* peers, TpState** state, int** status) {
  MX_REQUIRE(blocks != nullptr && world >= 1 && world <= kTpMaxRanks && rank >= 0 && rank < world,
             "world must be in [1, %d] and rank inside it", kTpMaxRanks);
  MX_REQUIRE(buffer == 0 || buffer == 1, "buffer must be 0 or 1");
  for (int r = 0; r < world; ++r) MX_REQUIRE(blocks[r] != nullptr, "block of rank %d is null", r);
  int device = 0;
  MX_CUDA(cudaGetDevice(&device));
  *status = device_status_word(device);
  if (*status == nullptr) return kCudaError;
  peers->world = world;
  peers->rank = rank;
  peers->buffer = buffer;
  peers->second_phase = 0;
  peers->wait_cycles = g_tp_wait_cycles;
  for (int r = 0; r < kTpMaxRanks; ++r) {
    peers->partial[r] = nullptr;
    peers->flags[r] = nullptr;
  }
  for (int r = 0; r < world; ++r) {
    auto* base = static_cast<uint8_t*>(blocks[r]);
    peers->flags[r] = reinterpret_cast<uint32_t*>(base);
    peers->partial[r] = base + kTpHeaderBytes + (size_t)buffer * partial_bytes;
  }
  *state = reinterpret_cast<TpState*>(static_cast<uint8_t*>(blocks[rank]) +
                                      kTpMaxRanks * sizeof(uint32_t));
  return kOk;
}
}  // namespace

int tp_reduce_scatter(void* const* blocks, int world, int rank, int buffer, size_t partial_bytes,
                      void* out, int64_t rows_per_rank, int64_t k, cudaStream_t stream) {
  MX_REQUIRE(out != nullptr && (reinterpret_cast<uintptr_t>(out) & 15) == 0,
             "out must be a 16-byte aligned device pointer");
  MX_REQUIRE(rows_per_rank > 0 && k > 0 && k % 8 == 0,
             "rows_per_rank must be positive and k a multiple of 8");
  MX_REQUIRE((size_t)world * (size_t)rows_per_rank * (size_t)k * 2 <= partial_bytes,
             "the partial buffers hold %zu bytes, %d x %lld x %lld BF16 need more", partial_bytes,
             world, (long long)rows_per_rank, (long long)k);
  TpPeers peers;
  TpState* state = nullptr;
  int* status = nullptr;
  if (int rc = tp_prepare(blocks, world, rank, buffer, partial_bytes, &peers, &state, &status))
    return rc;
  const int64_t chunks = rows_per_rank * k / 8;
  int64_t grid = (chunks + kTpThreads - 1) / kTpThreads;
  if (grid > 148 * 4) grid = 148 * 4;
  reduce_scatter_kernel<<<(unsigned)grid, kTpThreads, 0, stream>>>(
      peers, state, static_cast<__nv_bfloat16*>(out), (int64_t)rank * chunks, chunks, status);
  MX_CUDA(cudaGetLastError());
  return kOk;
}

int tp_allgather(void* const* blocks, int world, int rank, int buffer, size_t partial_bytes,
                 int segments, const int64_t* offsets, const int64_t* bytes, void* const* dsts,
                 cudaStream_t stream) {
  MX_REQUIRE(segments >= 1 && segments <= 4 && offsets != nullptr && bytes != nullptr &&
                 dsts != nullptr,
             "one to four segments with their offsets, sizes and destinations");
  TpSegments seg;
  seg.count = segments;
  seg.rank_strided = 0;
  int64_t largest = 0;
  for (int s = 0; s < 4; ++s) {
    seg.offset[s] = 0;
    seg.bytes[s] = 0;
    seg.dst[s] = nullptr;
  }
  for (int s = 0; s < segments; ++s) {
    MX_REQUIRE(offsets[s] >= 0 && bytes[s] > 0 && offsets[s] % 16 == 0 && bytes[s] % 16 == 0 &&
                   (size_t)(offsets[s] + bytes[s]) <= partial_bytes,
               "segment %d must be 16-byte granular and inside the partial buffer", s);
    MX_REQUIRE(dsts[s] != nullptr && (reinterpret_cast<uintptr_t>(dsts[s]) & 15) == 0,
               "destination %d must be a 16-byte aligned device pointer", s);
    seg.offset[s] = offsets[s];
    seg.bytes[s] = bytes[s];
    seg.dst[s] = static_cast<uint8_t*>(dsts[s]);
    if (bytes[s] > largest) largest = bytes[s];
  }
  TpPeers peers;
  TpState* state = nullptr;
  int* status = nullptr;
  if (int rc = tp_prepare(blocks, world, rank, buffer, partial_bytes, &peers, &state, &status))
    return rc;
  int64_t grid = (largest / 16 * world + 4 * kTpThreads - 1) / (4 * kTpThreads);
  if (grid > 148 * 4) grid = 148 * 4;
  if (grid < 1) grid = 1;
  allgather_kernel<<<(unsigned)grid, kTpThreads, 0, stream>>>(peers, state, seg, status);
  MX_CUDA(cudaGetLastError());
  return kOk;
}

// All-reduce of a bandwidth-bound [rows, k] BF16 partial in two launches over buffer
// `buffer`: every rank first sums ITS slice of rows over all ranks and writes the sums over
// its own copy of that slice (nobody else reads that part of its buffer in this phase), then
// all ranks gather the reduced slices.  Each rank moves 2 * (world - 1) / world of the tensor
// over NVLink, as a ring does, but in one hop and on all links at once.
int tp_allreduce_two_phase(void* const* blocks, int world, int rank, int buffer,
                           size_t partial_bytes, void* out, int64_t rows, int64_t k,
                           cudaStream_t stream) {
  MX_REQUIRE(out != nullptr && (reinterpret_cast<uintptr_t>(out) & 15) == 0,
             "out must be a 16-byte aligned device pointer");
  MX_REQUIRE(rows > 0 && k > 0 && k % 8 == 0 && world >= 1 && rows % world == 0,
             "rows must be a positive multiple of the world size and k a multiple of 8");
  MX_REQUIRE((size_t)rows * (size_t)k * 2 <= partial_bytes,
             "the partial buffers hold %zu bytes, %lld x %lld BF16 need more", partial_bytes,
             (long long)rows, (long long)k);
  TpPeers peers;
  TpState* state = nullptr;
  int* status = nullptr;
  if (int rc = tp_prepare(blocks, world, rank, buffer, partial_bytes, &peers, &state, &status))
    return rc;
  const int64_t slice_chunks = rows / world * k / 8;
  int64_t grid = (slice_chunks + kTpThreads - 1) / kTpThreads;
  if (grid > 148 * 4) grid = 148 * 4;
  auto* mine = static_cast<__nv_bfloat16*>(const_cast<void*>(peers.partial[rank])) +
               (int64_t)rank * slice_chunks * 8;
  reduce_scatter_kernel<<<(unsigned)grid, kTpThreads, 0, stream>>>(
      peers, state, mine, (int64_t)rank * slice_chunks, slice_chunks, status);
  MX_CUDA(cudaGetLastError());
  TpSegments seg;
  seg.count = 1;
  seg.rank_strided = 1;
  for (int s = 0; s < 4; ++s) {
    seg.offset[s] = 0;
    seg.bytes[s] = 0;
    seg.dst[s] = nullptr;
  }
  seg.bytes[0] = slice_chunks * 16;
  seg.dst[0] = static_cast<uint8_t*>(out);
  peers.second_phase = 1;
  grid = (slice_chunks * world + 4 * kTpThreads - 1) / (4 * kTpThreads);
  if (grid > 148 * 4) grid = 148 * 4;
  if (grid < 1) grid = 1;
  allgather_kernel<<<(unsigned)grid, kTpThreads, 0, stream>>>(peers, state, seg, status);
  MX_CUDA(cudaGetLastError());
  return kOk;
}

namespace {
// Handshake only: a rank that has passed it has seen every peer leave the step before, so
// whatever that step read may be overwritten.  It records the OTHER buffer index as the last
// one used, so that the next sum on the single caller-owned buffer is not taken for a repeat.
__global__ void __launch_bounds__(kTpThreads)
step_barrier_kernel(const TpPeers peers, TpState* state, int* status) {
  __shared__ uint32_t step_shared;
  __shared__ int ok_shared;
  const uint32_t step = tp_handshake(peers, state, status, &step_shared, &ok_shared);
  tp_finish(state, step, peers.buffer ^ 1);
}
}  // namespace

// The all-reduce over caller-owned memory, as the reference's fused reducer takes it from
// vLLM's custom all-reduce (csrc/moe.cu:7698-7925: one signal area and one data buffer per
// rank, every rank's pointers valid on this device).  signals[r] points to at least 64
// zero-initialised bytes (eight flags and the step state), buffers[r] to the rank's
// [rows, k] BF16 partial; this rank's partial is complete on `stream` before the call.  One
// buffer per rank means a closing barrier: the second launch returns only when every peer has
// finished reading, and only then may the caller's next producer overwrite the buffer.
int tp_allreduce_pointers(const uint64_t* signals, const uint64_t* buffers, int world, int rank,
                          void* out, int64_t rows, int64_t k, cudaStream_t stream) {
  MX_REQUIRE(signals != nullptr && buffers != nullptr && world >= 1 && world <= kTpMaxRanks &&
                 rank >= 0 && rank < world,
             "world must be in [1, %d] and rank inside it", kTpMaxRanks);
  MX_REQUIRE(out != nullptr && (reinterpret_cast<uintptr_t>(out) & 15) == 0,
             "out must be a 16-byte aligned device pointer");
  MX_REQUIRE(rows > 0 && k > 0 && k % 8 == 0, "rows must be positive and k a multiple of 8");
  int device = 0;
  MX_CUDA(cudaGetDevice(&device));
  int* status = device_status_word(device);
  if (status == nullptr) return kCudaError;
  TpPeers peers;
  peers.world = world;
  peers.rank = rank;
  peers.buffer = 0;
  peers.second_phase = 0;
  peers.wait_cycles = g_tp_wait_cycles;
  for (int r = 0; r < kTpMaxRanks; ++r) {
    peers.partial[r] = nullptr;
    peers.flags[r] = nullptr;
  }
  for (int r = 0; r < world; ++r) {
    MX_REQUIRE(signals[r] != 0 && buffers[r] != 0 && (signals[r] & 3) == 0 && (buffers[r] & 15) == 0,
               "signal and buffer pointers of rank %d must be non-null and aligned (4 / 16 bytes)", r);
    peers.flags[r] = reinterpret_cast<uint32_t*>(static_cast<uintptr_t>(signals[r]));
    peers.partial[r] = reinterpret_cast<const void*>(static_cast<uintptr_t>(buffers[r]));
  }
  auto* state = reinterpret_cast<TpState*>(reinterpret_cast<uint8_t*>(peers.flags[rank]) +
                                           kTpMaxRanks * sizeof(uint32_t));
  const int64_t chunks = rows * k / 8;
  int64_t grid = (chunks + kTpThreads - 1) / kTpThreads;
  if (grid > 148 * 4) grid = 148 * 4;
  allreduce_sum_kernel<<<(unsigned)grid, kTpThreads, 0, stream>>>(
      peers, state, static_cast<__nv_bfloat16*>(out), chunks, status);
  MX_CUDA(cudaGetLastError());
  peers.second_phase = 1;
  step_barrier_kernel<<<1, kTpThreads, 0, stream>>>(peers, state, status);
  MX_CUDA(cudaGetLastError());
  return kOk;
}

size_t tp_block_header_bytes() { return kTpHeaderBytes; }

}  // namespace mx
