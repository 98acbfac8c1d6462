// BF16/FP16 -> MXFP8 (E4M3) and -> MXFP6 (E3M2) dynamic quantizers, one UE8M0
// scale per 32 consecutive K values.
//
// Arithmetic follows the reference quantizer (csrc/quantization.cu:96-144):
//   absmax over the 32 values (FP32), raw = max(absmax / T, 1e-30) with IEEE
//   division (T = 448 for E4M3, 28 for E3M2), scale = raw rounded up to a power
//   of two, code = exponent byte, q = cvt_rn_satfinite(x * (1 / scale)).
// The launch shape is new: every thread moves one (MXFP8) or two (MXFP6) 16-byte
// vectors, the group maximum is a 2- or 1-step shuffle, value stores are 8- or
// 12-byte vectors, and the padding bytes of the packed scale buffer are written
// by the same launch instead of a preceding memset.
#include "common.cuh"

#include <cuda_fp8.h>
#include <cuda_fp6.h>

#include <algorithm>

namespace mx {
namespace {

constexpr int kQuantThreads = 256;

template <class T>
struct Vec8 {
  uint4 raw;
  __device__ __forceinline__ void unpack(float (&v)[8]) const;
};

template <>
__device__ __forceinline__ void Vec8<__nv_bfloat16>::unpack(float (&v)[8]) const {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

template <>
__device__ __forceinline__ void Vec8<__half>::unpack(float (&v)[8]) const {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
    const float2 f = __half22float2(h);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

__device__ __forceinline__ float absmax8(const float (&v)[8]) {
  float m = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(v[i]));
  return m;
}

// Writes 0x7f into every byte of the packed scale buffer that belongs to a
// padded row or a padded k-group, starting at byte `begin`.
__device__ __forceinline__ void fill_scale_padding(uint8_t* packed, int64_t begin, int64_t total,
                                                   int64_t rows, int groups, int64_t tid,
                                                   int64_t nthreads) {
  const int64_t atoms_per_rb = (groups + kAtomGroups - 1) / kAtomGroups;
  for (int64_t idx = begin + tid; idx < total; idx += nthreads) {
    const int64_t atom = idx / 512;
    const int within = static_cast<int>(idx % 512);
    const int64_t row = (atom / atoms_per_rb) * kAtomRows + ((within % 16) / 4) * 32 + within / 16;
    const int64_t g = (atom % atoms_per_rb) * kAtomGroups + within % 4;
    if (row >= rows || g >= groups) packed[idx] = kUe8m0One;
  }
}

// The same for buffers whose rows hold whole quads of groups (the lean kernel's case): the
// padding is then whole 32-bit words (four groups of one row), all in the last 128-row
// block, and every index fits 32 bits.  A decode batch of one row has 127 rows of padding,
// forty times its payload, so this loop must not crawl.
__device__ __forceinline__ void fill_scale_padding_words(uint8_t* packed, uint32_t begin,
                                                         uint32_t total, uint32_t rows,
                                                         uint32_t tid, uint32_t nthreads) {
  const uint32_t valid = rows & 127u;  // rows of the last block that hold real scales
  uint32_t* words = reinterpret_cast<uint32_t*>(packed + begin);
  const uint32_t count = (total - begin) >> 2;
  for (uint32_t w = tid; w < count; w += nthreads) {
    const uint32_t in_atom = w & 127u;  // word (r % 32) * 4 + r / 32 of its atom
    const uint32_t row = ((in_atom & 3u) << 5) + (in_atom >> 2);
    if (row >= valid) words[w] = 0x7f7f7f7fu;
  }
}

// One thread per 8 consecutive K values, four threads per scale group.
template <class T>
__global__ void __launch_bounds__(kQuantThreads)
quantize_mxfp8_kernel(const T* __restrict__ in, uint8_t* __restrict__ out,
                      uint8_t* __restrict__ packed, uint8_t* __restrict__ logical, int64_t rows,
                      int k, int64_t pad_begin, int64_t pad_total, bool quad_scales) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int groups = k / kScaleVec;
  const int64_t chunks = rows * (k / 8);
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  // Four independent 16-byte loads per thread are issued before any of them is
  // used, so that enough bytes are in flight to cover HBM latency.
  constexpr int kUnroll = 4;
  const int64_t per_round = nthreads * kUnroll;
  const int64_t rounds = (chunks + per_round - 1) / per_round;
  for (int64_t it = 0; it < rounds; ++it) {
    Vec8<T> raw[kUnroll];
    int64_t cs[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      cs[u] = it * per_round + u * nthreads + tid;
      raw[u].raw = make_uint4(0u, 0u, 0u, 0u);
      if (cs[u] < chunks) raw[u].raw = __ldg(reinterpret_cast<const uint4*>(in) + cs[u]);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t c = cs[u];
      const bool valid = c < chunks;
      float v[8];
      raw[u].unpack(v);
      float amax = absmax8(v);
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      const uint32_t sbits = ue8m0_scale_bits(amax, 448.0f);
      const float inv = ue8m0_inverse(sbits);
      if (valid) {
        uint32_t w[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const uint32_t lo = __nv_cvt_float2_to_fp8x2(
              make_float2(v[4 * i] * inv, v[4 * i + 1] * inv), __NV_SATFINITE, __NV_E4M3);
          const uint32_t hi = __nv_cvt_float2_to_fp8x2(
              make_float2(v[4 * i + 2] * inv, v[4 * i + 3] * inv), __NV_SATFINITE, __NV_E4M3);
          w[i] = lo | (hi << 16);
        }
        reinterpret_cast<uint2*>(out)[c] = make_uint2(w[0], w[1]);
      }
      // Scale bytes.  Four consecutive groups of a row are four consecutive bytes in
      // both layouts when the row holds a multiple of four groups, so lanes 0 and 16
      // collect the codes of lanes +4, +8, +12 and store one 32-bit word each.
      const uint32_t code = sbits >> 23;
      if (quad_scales) {
        uint32_t word = code;
        word |= __shfl_down_sync(0xffffffffu, code, 4) << 8;
        word |= __shfl_down_sync(0xffffffffu, code, 8) << 16;
        word |= __shfl_down_sync(0xffffffffu, code, 12) << 24;
        if (valid && (threadIdx.x & 15) == 0) {
          const uint32_t group = static_cast<uint32_t>(c >> 2);  // fits: checked on the host
          if (logical != nullptr) *reinterpret_cast<uint32_t*>(logical + group) = word;
          if (packed != nullptr) {
            const uint32_t row = group / static_cast<uint32_t>(groups);
            const int g = static_cast<int>(group - row * static_cast<uint32_t>(groups));
            *reinterpret_cast<uint32_t*>(packed + packed_scale_offset(row, g, groups)) = word;
          }
        }
      } else if (valid && (c & 3) == 0) {
        const int64_t group = c >> 2;
        if (logical != nullptr) logical[group] = static_cast<uint8_t>(code);
        if (packed != nullptr) {
          const int64_t row = group / groups;
          const int g = static_cast<int>(group - row * groups);
          packed[packed_scale_offset(row, g, groups)] = static_cast<uint8_t>(code);
        }
      }
    }
  }
  if (packed != nullptr && pad_begin < pad_total) {
    fill_scale_padding(packed, pad_begin, pad_total, rows, groups, tid, nthreads);
  }
}

// Lean form of the kernel above for the common case (a row of whole quads of scale groups,
// fewer than 2^31 chunks): the general kernel spends ~140 instructions per 8 values, most
// of them on 64-bit index arithmetic and the division that turns a group index into
// (row, group); here the row and the position in the row advance incrementally and all
// offsets are 32-bit, which matters because the kernel is issue-bound, not memory-bound.
template <class T>
__global__ void __launch_bounds__(kQuantThreads)
quantize_mxfp8_lean_kernel(const T* __restrict__ in, uint8_t* __restrict__ out,
                           uint8_t* __restrict__ packed, uint8_t* __restrict__ logical,
                           uint32_t rows, uint32_t row_chunks, uint32_t chunks,
                           int64_t pad_begin, int64_t pad_total) {
  // Decode batches are launched as programmatic dependents: the GEMM that follows may
  // start (and prefetch its weights) at once, and this kernel itself may become resident
  // while the kernel before it still runs; it reads and writes nothing before the wait.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  constexpr int kUnroll = 4;
  const uint32_t nthreads = gridDim.x * blockDim.x;
  const uint32_t tid = blockIdx.x * blockDim.x + threadIdx.x;
  const uint32_t groups = row_chunks >> 2;
  const uint32_t atoms_per_rb = groups >> 2;
  // (row, chunk in row) of this thread's current chunk, and the step of one sub-iteration.
  const uint32_t step_rows = nthreads / row_chunks;
  const uint32_t step_cols = nthreads - step_rows * row_chunks;
  uint32_t row = tid / row_chunks;
  uint32_t col = tid - row * row_chunks;
  const uint4* src = reinterpret_cast<const uint4*>(in);
  uint2* dst = reinterpret_cast<uint2*>(out);
  // Every thread runs every round (the shuffles below need whole warps).
  const uint32_t per_round = nthreads * kUnroll;
  const uint32_t rounds = (chunks + per_round - 1) / per_round;
  for (uint32_t it = 0; it < rounds; ++it) {
    const uint32_t base = it * per_round + tid;
    Vec8<T> raw[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t c = base + u * nthreads;
      raw[u].raw = make_uint4(0u, 0u, 0u, 0u);
      if (c < chunks) raw[u].raw = __ldg(src + c);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t c = base + u * nthreads;
      float v[8];
      raw[u].unpack(v);
      float amax = absmax8(v);
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      const uint32_t sbits = ue8m0_scale_bits(amax, 448.0f);
      const float inv = ue8m0_inverse(sbits);
      const uint32_t code = sbits >> 23;
      uint32_t word = code;
      word |= __shfl_down_sync(0xffffffffu, code, 4) << 8;
      word |= __shfl_down_sync(0xffffffffu, code, 8) << 16;
      word |= __shfl_down_sync(0xffffffffu, code, 12) << 24;
      if (c < chunks) {
        uint32_t w[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const uint32_t lo = __nv_cvt_float2_to_fp8x2(
              make_float2(v[4 * i] * inv, v[4 * i + 1] * inv), __NV_SATFINITE, __NV_E4M3);
          const uint32_t hi = __nv_cvt_float2_to_fp8x2(
              make_float2(v[4 * i + 2] * inv, v[4 * i + 3] * inv), __NV_SATFINITE, __NV_E4M3);
          w[i] = lo | (hi << 16);
        }
        dst[c] = make_uint2(w[0], w[1]);
        if ((threadIdx.x & 15) == 0) {
          const uint32_t g = col >> 2;  // a multiple of 4: 16 lanes = four groups of one row
          if (logical != nullptr) *reinterpret_cast<uint32_t*>(logical + (c >> 2)) = word;
          if (packed != nullptr) {
            const uint32_t offset = ((row >> 7) * atoms_per_rb + (g >> 2)) * 512u +
                                    (row & 31u) * 16u + ((row >> 5) & 3u) * 4u;
            *reinterpret_cast<uint32_t*>(packed + offset) = word;
          }
        }
      }
      row += step_rows;
      col += step_cols;
      if (col >= row_chunks) {
        col -= row_chunks;
        ++row;
      }
    }
  }
  if (packed != nullptr && pad_begin < pad_total) {
    fill_scale_padding_words(packed, static_cast<uint32_t>(pad_begin),
                             static_cast<uint32_t>(pad_total), rows, tid, nthreads);
  }
}

// One thread per 16 consecutive K values (two per scale group); the sixteen
// E3M2 codes leave as three 32-bit words (code i at bits 6i..6i+5).
template <class T>
__global__ void __launch_bounds__(kQuantThreads)
quantize_mxfp6_kernel(const T* __restrict__ in, uint8_t* __restrict__ out,
                      uint8_t* __restrict__ packed, uint8_t* __restrict__ logical, int64_t rows,
                      int k, int64_t pad_begin, int64_t pad_total) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int groups = k / kScaleVec;
  const int64_t chunks = rows * (k / 16);
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t rounds = (chunks + nthreads - 1) / nthreads;
  for (int64_t it = 0; it < rounds; ++it) {
    const int64_t c = it * nthreads + tid;
    const bool valid = c < chunks;
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = 0.0f;
    if (valid) {
      Vec8<T> a, b;
      a.raw = __ldg(reinterpret_cast<const uint4*>(in) + 2 * c);
      b.raw = __ldg(reinterpret_cast<const uint4*>(in) + 2 * c + 1);
      float lo[8], hi[8];
      a.unpack(lo);
      b.unpack(hi);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[i] = lo[i];
        v[8 + i] = hi[i];
      }
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    const uint32_t sbits = ue8m0_scale_bits(amax, 28.0f);
    const float inv = ue8m0_inverse(sbits);
    if (valid) {
      uint32_t unit[4];  // four codes -> 24 bits, code i at bits 6i..6i+5
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t p0 = __nv_cvt_float2_to_fp6x2(
            make_float2(v[4 * u] * inv, v[4 * u + 1] * inv), __NV_E3M2, cudaRoundNearest);
        const uint32_t p1 = __nv_cvt_float2_to_fp6x2(
            make_float2(v[4 * u + 2] * inv, v[4 * u + 3] * inv), __NV_E3M2, cudaRoundNearest);
        unit[u] = (p0 & 0x3fu) | (((p0 >> 8) & 0x3fu) << 6) | ((p1 & 0x3fu) << 12) |
                  (((p1 >> 8) & 0x3fu) << 18);
      }
      uint32_t* dst = reinterpret_cast<uint32_t*>(out + c * 12);
      dst[0] = unit[0] | (unit[1] << 24);
      dst[1] = (unit[1] >> 8) | (unit[2] << 16);
      dst[2] = (unit[2] >> 16) | (unit[3] << 8);
      if ((c & 1) == 0) {
        const int64_t group = c >> 1;
        const uint8_t code = static_cast<uint8_t>(sbits >> 23);
        if (logical != nullptr) logical[group] = code;
        if (packed != nullptr) {
          const int64_t row = group / groups;
          const int g = static_cast<int>(group - row * groups);
          packed[packed_scale_offset(row, g, groups)] = code;
        }
      }
    }
  }
  if (packed != nullptr && pad_begin < pad_total) {
    fill_scale_padding(packed, pad_begin, pad_total, rows, groups, tid, nthreads);
  }
}

// RMSNorm fused into the activation quantizer: one CTA per row keeps the row in registers
// (up to kNormChunks 8-value chunks per thread), so the row is read once and only the MXFP8
// bytes and scales are written.  y = round_to_T((x * rsqrt(mean(x^2) + eps)) * w) in FP32
// with one rounding (the rule of torch.nn.functional.rms_norm), then the MXFP8 rule above.
constexpr int kNormChunks = 8;  // K <= 8 * 8 * 256 = 16384

template <class T>
__device__ __forceinline__ float round_to(float v);
template <>
__device__ __forceinline__ float round_to<__nv_bfloat16>(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}
template <>
__device__ __forceinline__ float round_to<__half>(float v) {
  return __half2float(__float2half_rn(v));
}

template <class T, int kChunks>
__global__ void __launch_bounds__(kQuantThreads)
rmsnorm_quantize_mxfp8_kernel(const T* in, const T* __restrict__ residual, T* updated,
                              const T* __restrict__ weight, float eps,
                              uint8_t* __restrict__ out, uint8_t* __restrict__ packed,
                              uint8_t* __restrict__ logical, int64_t rows, int k,
                              int64_t pad_begin, int64_t pad_total, bool quad_scales) {
  __shared__ float warp_sums[kQuantThreads / 32];
  const int row_chunks = k / 8;
  const int groups = k / kScaleVec;
  const int64_t row = blockIdx.x;
  const uint4* src = reinterpret_cast<const uint4*>(in) + row * row_chunks;
  const uint4* wsrc = reinterpret_cast<const uint4*>(weight);
  Vec8<T> raw[kChunks];
  float sum = 0.0f;
#pragma unroll
  for (int u = 0; u < kChunks; ++u) {
    const int c = u * kQuantThreads + threadIdx.x;
    raw[u].raw = make_uint4(0u, 0u, 0u, 0u);
    if (c < row_chunks) raw[u].raw = src[c];
  }
  if (residual != nullptr) {
    // Residual stream: x <- round(x + r), written back (to `updated`, which may be `in`),
    // and the norm is taken of the rounded sum.
    const uint4* rsrc = reinterpret_cast<const uint4*>(residual) + row * row_chunks;
    uint4* xdst = reinterpret_cast<uint4*>(updated) + row * row_chunks;
#pragma unroll
    for (int u = 0; u < kChunks; ++u) {
      const int c = u * kQuantThreads + threadIdx.x;
      if (c < row_chunks) {
        Vec8<T> r;
        r.raw = __ldg(rsrc + c);
        float a[8], b[8];
        raw[u].unpack(a);
        r.unpack(b);
        T packed8[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) packed8[i] = static_cast<T>(a[i] + b[i]);
        raw[u].raw = *reinterpret_cast<const uint4*>(packed8);
        xdst[c] = raw[u].raw;
      }
    }
  }
#pragma unroll
  for (int u = 0; u < kChunks; ++u) {
    float v[8];
    raw[u].unpack(v);
#pragma unroll
    for (int i = 0; i < 8; ++i) sum = fmaf(v[i], v[i], sum);
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = sum;
  __syncthreads();
  float total = 0.0f;
#pragma unroll
  for (int w = 0; w < kQuantThreads / 32; ++w) total += warp_sums[w];
  const float inv_rms = rsqrtf(total / static_cast<float>(k) + eps);
#pragma unroll
  for (int u = 0; u < kChunks; ++u) {
    const int c = u * kQuantThreads + threadIdx.x;
    const bool valid = c < row_chunks;
    float v[8], g[8];
    raw[u].unpack(v);
    Vec8<T> wv;
    wv.raw = make_uint4(0u, 0u, 0u, 0u);
    if (valid) wv.raw = __ldg(wsrc + c);
    wv.unpack(g);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = round_to<T>((v[i] * inv_rms) * g[i]);
    float amax = absmax8(v);
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
      const int g_index = c >> 2;
      if (quad_scales) {
        if ((threadIdx.x & 15) == 0) {
          if (logical != nullptr)
            *reinterpret_cast<uint32_t*>(logical + row * groups + g_index) = word;
          if (packed != nullptr)
            *reinterpret_cast<uint32_t*>(packed + packed_scale_offset(row, g_index, groups)) = word;
        }
      } else if ((c & 3) == 0) {
        if (logical != nullptr) logical[row * groups + g_index] = static_cast<uint8_t>(code);
        if (packed != nullptr)
          packed[packed_scale_offset(row, g_index, groups)] = static_cast<uint8_t>(code);
      }
    }
  }
  if (packed != nullptr && pad_begin < pad_total) {
    fill_scale_padding(packed, pad_begin, pad_total, rows, groups,
                       static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x,
                       static_cast<int64_t>(gridDim.x) * blockDim.x);
  }
}

int check_args(const void* in, int dtype, int64_t rows, int64_t k, const void* values) {
  MX_REQUIRE(in != nullptr && values != nullptr, "input and output pointers must not be null");
  MX_REQUIRE(dtype == kF16 || dtype == kBF16, "input must be float16 or bfloat16");
  MX_REQUIRE(rows > 0, "M must be positive; got %lld", (long long)rows);
  MX_REQUIRE(k > 0 && k % kScaleVec == 0, "K must be a positive multiple of 32; got %lld",
             (long long)k);
  MX_REQUIRE(rows <= INT32_MAX && k <= INT32_MAX, "M and K must fit in a 32-bit integer");
  MX_REQUIRE((reinterpret_cast<uintptr_t>(in) & 15) == 0, "input must be 16-byte aligned");
  return kOk;
}

void padding_range(int64_t rows, int64_t k, int64_t* begin, int64_t* total) {
  const int64_t groups = k / kScaleVec;
  *total = packed_scale_bytes(rows, k);
  if (groups % kAtomGroups != 0) {
    *begin = 0;
  } else if (rows % kAtomRows != 0) {
    *begin = (rows / kAtomRows) * (groups / kAtomGroups) * 512;
  } else {
    *begin = *total;
  }
}

int grid_for(int64_t chunks) {
  // Enough CTAs to fill 148 SMs at 8 resident CTAs each; grid-stride beyond that.
  // Every thread takes four chunks per round.
  const int64_t want = (chunks + 4 * kQuantThreads - 1) / (4 * kQuantThreads);
  // Persistent once the GPU is full (4 CTAs of 256 threads fit an SM at 59 registers):
  // CTAs then loop over rounds instead of being relaunched, and only the last of
  // several rounds is ragged.
  const int64_t cap = 148 * 4;
  return static_cast<int>(want < 1 ? 1 : (want > cap ? cap : want));
}

}  // namespace

int quantize_mxfp8(const void* in, int dtype, int64_t rows, int64_t k, uint8_t* values,
                   uint8_t* packed, uint8_t* logical, cudaStream_t stream) {
  if (int rc = check_args(in, dtype, rows, k, values)) return rc;
  MX_REQUIRE(packed != nullptr || logical != nullptr, "at least one scale output is required");
  MX_REQUIRE((reinterpret_cast<uintptr_t>(values) & 7) == 0, "values must be 8-byte aligned");
  int64_t pad_begin = 0, pad_total = 0;
  if (packed != nullptr) padding_range(rows, k, &pad_begin, &pad_total);
  const int64_t chunks = rows * (k / 8);
  const int grid = grid_for(chunks);
  // Word-wide scale stores need whole quads of groups per row, 4-byte aligned
  // scale buffers and 32-bit group indices.
  const bool quad = (k / kScaleVec) % 4 == 0 && chunks < (int64_t(1) << 33) &&
                    (reinterpret_cast<uintptr_t>(packed) & 3) == 0 &&
                    (reinterpret_cast<uintptr_t>(logical) & 3) == 0;
  // packed offsets in 32 bits: the scale buffer is rows * groups bytes plus padding.
  if (quad && chunks < (int64_t(1) << 31) && packed_scale_bytes(rows, k) < (int64_t(1) << 31)) {
    // A batch of a few rows has more padding words to write than chunks to quantize.
    const int64_t pad_ctas = ((pad_total - pad_begin) / 4 + 4 * kQuantThreads - 1) / (4 * kQuantThreads);
    const int grid = (int)std::max<int64_t>(grid_for(chunks), std::min<int64_t>(pad_ctas, 148));
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)grid);
    config.blockDim = dim3(kQuantThreads);
    config.stream = stream;
    // Small grids only: a large quantizer that became resident early would sit on SM
    // slots of the kernel it waits for.
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = grid <= 148 ? 1 : 0;
    if (dtype == kBF16) {
      MX_CUDA(cudaLaunchKernelEx(&config, quantize_mxfp8_lean_kernel<__nv_bfloat16>,
                                 static_cast<const __nv_bfloat16*>(in), values, packed, logical,
                                 (uint32_t)rows, (uint32_t)(k / 8), (uint32_t)chunks, pad_begin,
                                 pad_total));
    } else {
      MX_CUDA(cudaLaunchKernelEx(&config, quantize_mxfp8_lean_kernel<__half>,
                                 static_cast<const __half*>(in), values, packed, logical,
                                 (uint32_t)rows, (uint32_t)(k / 8), (uint32_t)chunks, pad_begin,
                                 pad_total));
    }
    return kOk;
  }
  if (dtype == kBF16) {
    quantize_mxfp8_kernel<__nv_bfloat16><<<grid, kQuantThreads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(in), values, packed, logical, rows,
        static_cast<int>(k), pad_begin, pad_total, quad);
  } else {
    quantize_mxfp8_kernel<__half><<<grid, kQuantThreads, 0, stream>>>(
        static_cast<const __half*>(in), values, packed, logical, rows, static_cast<int>(k),
        pad_begin, pad_total, quad);
  }
  MX_CUDA(cudaGetLastError());
  return kOk;
}

int quantize_mxfp6(const void* in, int dtype, int64_t rows, int64_t k, uint8_t* values,
                   uint8_t* packed, uint8_t* logical, cudaStream_t stream) {
  if (int rc = check_args(in, dtype, rows, k, values)) return rc;
  MX_REQUIRE(packed != nullptr || logical != nullptr, "at least one scale output is required");
  MX_REQUIRE((reinterpret_cast<uintptr_t>(values) & 3) == 0, "values must be 4-byte aligned");
  int64_t pad_begin = 0, pad_total = 0;
  if (packed != nullptr) padding_range(rows, k, &pad_begin, &pad_total);
  const int64_t chunks = rows * (k / 16);
  const int grid = grid_for(chunks);
  if (dtype == kBF16) {
    quantize_mxfp6_kernel<__nv_bfloat16><<<grid, kQuantThreads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(in), values, packed, logical, rows,
        static_cast<int>(k), pad_begin, pad_total);
  } else {
    quantize_mxfp6_kernel<__half><<<grid, kQuantThreads, 0, stream>>>(
        static_cast<const __half*>(in), values, packed, logical, rows, static_cast<int>(k),
        pad_begin, pad_total);
  }
  MX_CUDA(cudaGetLastError());
  return kOk;
}

int rmsnorm_quantize_mxfp8(const void* in, const void* residual, void* updated, int dtype,
                           const void* weight, float eps, int64_t rows, int64_t k, uint8_t* values,
                           uint8_t* packed, uint8_t* logical, cudaStream_t stream) {
  if (int rc = check_args(in, dtype, rows, k, values)) return rc;
  MX_REQUIRE((residual == nullptr) == (updated == nullptr),
             "residual and updated go together");
  MX_REQUIRE(residual == nullptr || ((reinterpret_cast<uintptr_t>(residual) & 15) == 0 &&
                                     (reinterpret_cast<uintptr_t>(updated) & 15) == 0),
             "residual / updated must be 16-byte aligned");
  MX_REQUIRE(weight != nullptr && (reinterpret_cast<uintptr_t>(weight) & 15) == 0,
             "the norm weight must be a 16-byte aligned device pointer");
  MX_REQUIRE(packed != nullptr || logical != nullptr, "at least one scale output is required");
  MX_REQUIRE((reinterpret_cast<uintptr_t>(values) & 7) == 0, "values must be 8-byte aligned");
  MX_REQUIRE(k % 8 == 0 && k <= kNormChunks * 8 * kQuantThreads,
             "the fused norm keeps a row in registers: K must be at most %d; got %lld",
             kNormChunks * 8 * kQuantThreads, (long long)k);
  MX_REQUIRE(eps >= 0.0f, "eps must not be negative");
  int64_t pad_begin = 0, pad_total = 0;
  if (packed != nullptr) padding_range(rows, k, &pad_begin, &pad_total);
  // Word-wide scale stores: a row of whole quads of groups, so that 16 consecutive
  // threads hold four consecutive groups of one row.
  const bool quad = (k / kScaleVec) % 4 == 0 && (reinterpret_cast<uintptr_t>(packed) & 3) == 0 &&
                    (reinterpret_cast<uintptr_t>(logical) & 3) == 0;
  const unsigned grid = static_cast<unsigned>(rows);
  // The row lives in registers: instantiate for the number of 8-value chunks a thread holds.
  const int need = static_cast<int>((k / 8 + kQuantThreads - 1) / kQuantThreads);
#define MX_LAUNCH_NORM(T, CH)                                                                   \
  rmsnorm_quantize_mxfp8_kernel<T, CH><<<grid, kQuantThreads, 0, stream>>>(                     \
      static_cast<const T*>(in), static_cast<const T*>(residual), static_cast<T*>(updated),     \
      static_cast<const T*>(weight), eps, values, packed, logical, rows, static_cast<int>(k),   \
      pad_begin, pad_total, quad)
#define MX_DISPATCH_NORM(T)                    \
  do {                                         \
    if (need <= 1) MX_LAUNCH_NORM(T, 1);       \
    else if (need <= 2) MX_LAUNCH_NORM(T, 2);  \
    else if (need <= 3) MX_LAUNCH_NORM(T, 3);  \
    else if (need <= 4) MX_LAUNCH_NORM(T, 4);  \
    else MX_LAUNCH_NORM(T, kNormChunks);       \
  } while (0)
  if (dtype == kBF16) {
    MX_DISPATCH_NORM(__nv_bfloat16);
  } else {
    MX_DISPATCH_NORM(__half);
  }
#undef MX_DISPATCH_NORM
#undef MX_LAUNCH_NORM
  MX_CUDA(cudaGetLastError());
  return kOk;
}

}  // namespace mx
