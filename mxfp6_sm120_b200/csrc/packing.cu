// Layout utilities: E3M2 bitstream pack/unpack, 12->16 byte padding, lossless
// E3M2->E4M3 expansion, and logical <-> packed UE8M0 scale reordering.
//
// Byte formats match the reference (csrc/packing.cu:46-59 for the bitstream,
// :61-89 for the E3M2->E4M3 map, :239-283 for the scale atoms); the kernels are
// written for 16-byte vector traffic with a scalar tail.
#include "common.cuh"

namespace mx {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ uint32_t pack4(uint32_t codes) {
  return (codes & 0x3fu) | (((codes >> 8) & 0x3fu) << 6) | (((codes >> 16) & 0x3fu) << 12) |
         (((codes >> 24) & 0x3fu) << 18);
}

__device__ __forceinline__ uint32_t unpack4(uint32_t bits24) {
  return (bits24 & 0x3fu) | (((bits24 >> 6) & 0x3fu) << 8) | (((bits24 >> 12) & 0x3fu) << 16) |
         (((bits24 >> 18) & 0x3fu) << 24);
}

// Four E3M2 codes (one per byte) -> four E4M3 bytes with the same values.
// Normals: exponent rebias 3 -> 7, mantissa gains a zero bit.  Subnormals
// m * 2^-4 (m = 1, 2, 3) become the E4M3 normals 0x18, 0x20, 0x24.
__device__ __forceinline__ uint32_t e3m2x4_to_e4m3x4(uint32_t codes) {
  uint32_t out = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t c = (codes >> (8 * i)) & 0x3fu;
    const uint32_t sign = (c & 0x20u) << 2;
    const uint32_t e = (c >> 2) & 7u;
    const uint32_t m = c & 3u;
    uint32_t mag;
    if (e != 0) {
      mag = ((e + 4u) << 3) | (m << 1);
    } else {
      mag = m == 0 ? 0u : (m == 1 ? 0x18u : (m == 2 ? 0x20u : 0x24u));
    }
    out |= (sign | mag) << (8 * i);
  }
  return out;
}

__global__ void __launch_bounds__(kThreads)
pack_fp6_kernel(const uint8_t* __restrict__ codes, uint8_t* __restrict__ out, int64_t n,
                bool vector_ok) {
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t vec = vector_ok ? n / 16 : 0;
  for (int64_t c = tid; c < vec; c += nthreads) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(codes) + c);
    const uint32_t u0 = pack4(v.x), u1 = pack4(v.y), u2 = pack4(v.z), u3 = pack4(v.w);
    uint32_t* dst = reinterpret_cast<uint32_t*>(out + c * 12);
    dst[0] = u0 | (u1 << 24);
    dst[1] = (u1 >> 8) | (u2 << 16);
    dst[2] = (u2 >> 16) | (u3 << 8);
  }
  for (int64_t q = vec * 4 + tid; q < n / 4; q += nthreads) {
    const uint8_t* s = codes + q * 4;
    const uint32_t u = pack4(s[0] | (s[1] << 8) | (s[2] << 16) | (uint32_t(s[3]) << 24));
    out[q * 3] = u & 0xff;
    out[q * 3 + 1] = (u >> 8) & 0xff;
    out[q * 3 + 2] = (u >> 16) & 0xff;
  }
}

template <bool kExpand>
__global__ void __launch_bounds__(kThreads)
unpack_fp6_kernel(const uint8_t* __restrict__ packed, uint8_t* __restrict__ out, int64_t n,
                  bool vector_ok) {
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t vec = vector_ok ? n / 16 : 0;
  for (int64_t c = tid; c < vec; c += nthreads) {
    const uint32_t* src = reinterpret_cast<const uint32_t*>(packed + c * 12);
    const uint32_t w0 = __ldg(src), w1 = __ldg(src + 1), w2 = __ldg(src + 2);
    uint4 v;
    v.x = unpack4(w0 & 0xffffffu);
    v.y = unpack4((w0 >> 24) | ((w1 & 0xffffu) << 8));
    v.z = unpack4((w1 >> 16) | ((w2 & 0xffu) << 16));
    v.w = unpack4(w2 >> 8);
    if (kExpand) {
      v.x = e3m2x4_to_e4m3x4(v.x);
      v.y = e3m2x4_to_e4m3x4(v.y);
      v.z = e3m2x4_to_e4m3x4(v.z);
      v.w = e3m2x4_to_e4m3x4(v.w);
    }
    reinterpret_cast<uint4*>(out)[c] = v;
  }
  for (int64_t q = vec * 4 + tid; q < n / 4; q += nthreads) {
    const uint8_t* s = packed + q * 3;
    uint32_t v = unpack4(s[0] | (s[1] << 8) | (uint32_t(s[2]) << 16));
    if (kExpand) v = e3m2x4_to_e4m3x4(v);
    out[q * 4] = v & 0xff;
    out[q * 4 + 1] = (v >> 8) & 0xff;
    out[q * 4 + 2] = (v >> 16) & 0xff;
    out[q * 4 + 3] = (v >> 24) & 0xff;
  }
}

// Every 12 packed bytes become a 16-byte segment whose last four bytes are zero.
__global__ void __launch_bounds__(kThreads)
pad_fp6_kernel(const uint8_t* __restrict__ packed, uint8_t* __restrict__ out, int64_t segments) {
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (int64_t s = tid; s < segments; s += nthreads) {
    const uint32_t* src = reinterpret_cast<const uint32_t*>(packed + s * 12);
    reinterpret_cast<uint4*>(out)[s] = make_uint4(__ldg(src), __ldg(src + 1), __ldg(src + 2), 0u);
  }
}

__global__ void __launch_bounds__(kThreads)
pack_scales_kernel(const uint8_t* __restrict__ logical, uint8_t* __restrict__ packed,
                   int64_t rows, int groups) {
  const int64_t total = round_up64(rows, kAtomRows) * round_up64(groups, kAtomGroups);
  const int64_t atoms_per_rb = (groups + kAtomGroups - 1) / kAtomGroups;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  // One thread per destination byte: writes are fully coalesced.
  for (int64_t idx = tid; idx < total; idx += nthreads) {
    const int64_t atom = idx / 512;
    const int within = static_cast<int>(idx % 512);
    const int64_t row = (atom / atoms_per_rb) * kAtomRows + ((within % 16) / 4) * 32 + within / 16;
    const int64_t g = (atom % atoms_per_rb) * kAtomGroups + within % 4;
    packed[idx] = (row < rows && g < groups) ? __ldg(logical + row * groups + g) : kUe8m0One;
  }
}

__global__ void __launch_bounds__(kThreads)
unpack_scales_kernel(const uint8_t* __restrict__ packed, uint8_t* __restrict__ logical,
                     int64_t rows, int groups) {
  const int64_t total = rows * groups;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (int64_t idx = tid; idx < total; idx += nthreads) {
    const int64_t row = idx / groups;
    const int g = static_cast<int>(idx - row * groups);
    logical[idx] = __ldg(packed + packed_scale_offset(row, g, groups));
  }
}

// scale_offsets[e] = sum over e' < e of ceil128(rows of e'); one warp scans.
__global__ void grouped_scale_offsets_kernel(const int64_t* __restrict__ expert_offsets,
                                             int64_t* __restrict__ scale_offsets, int experts) {
  const int lane = threadIdx.x;
  int64_t carry = 0;
  for (int base = 0; base < experts; base += 32) {
    const int e = base + lane;
    int64_t padded = 0;
    if (e < experts) {
      padded = round_up64(expert_offsets[e + 1] - expert_offsets[e], kAtomRows);
    }
    int64_t incl = padded;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int64_t up = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += up;
    }
    if (e < experts) scale_offsets[e] = carry + incl - padded;
    carry += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0) scale_offsets[experts] = carry;
}

// Packed scales of a row-grouped matrix: expert e's rows start at packed row
// scale_offsets[e].  `padded_rows` bounds the destination; rows that belong to
// no expert (padding) are written as 0x7f.
__global__ void __launch_bounds__(kThreads)
pack_grouped_scales_kernel(const uint8_t* __restrict__ logical,
                           const int64_t* __restrict__ expert_offsets,
                           const int64_t* __restrict__ scale_offsets, int experts,
                           uint8_t* __restrict__ packed, int64_t padded_rows, int groups) {
  const int64_t atoms_per_rb = (groups + kAtomGroups - 1) / kAtomGroups;
  const int64_t total = padded_rows * atoms_per_rb * kAtomGroups;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (int64_t idx = tid; idx < total; idx += nthreads) {
    const int64_t atom = idx / 512;
    const int within = static_cast<int>(idx % 512);
    const int64_t prow = (atom / atoms_per_rb) * kAtomRows + ((within % 16) / 4) * 32 + within / 16;
    const int64_t g = (atom % atoms_per_rb) * kAtomGroups + within % 4;
    uint8_t value = kUe8m0One;
    if (g < groups && prow < scale_offsets[experts]) {
      // Largest e with scale_offsets[e] <= prow.
      int lo = 0, hi = experts;
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (scale_offsets[mid] <= prow) lo = mid; else hi = mid;
      }
      const int64_t local = prow - scale_offsets[lo];
      const int64_t rows_e = expert_offsets[lo + 1] - expert_offsets[lo];
      if (local < rows_e) value = __ldg(logical + (expert_offsets[lo] + local) * groups + g);
    }
    packed[idx] = value;
  }
}

int grid_for(int64_t items) {
  const int64_t want = (items + kThreads - 1) / kThreads;
  const int64_t cap = 148 * 16;
  return static_cast<int>(want < 1 ? 1 : (want > cap ? cap : want));
}

bool aligned(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

}  // namespace

int pack_fp6(const uint8_t* codes, int64_t n, uint8_t* out, cudaStream_t stream) {
  MX_REQUIRE(codes != nullptr && out != nullptr, "pointers must not be null");
  MX_REQUIRE(n > 0 && n % 4 == 0, "codes.numel() must be divisible by four; got %lld",
             (long long)n);
  const bool vec = aligned(codes, 16) && aligned(out, 4);
  pack_fp6_kernel<<<grid_for(n / 16 + 1), kThreads, 0, stream>>>(codes, out, n, vec);
  MX_CUDA(cudaGetLastError());
  return kOk;
}

int unpack_fp6(const uint8_t* packed, int64_t rows, int64_t k, uint8_t* out,
               cudaStream_t stream) {
  MX_REQUIRE(packed != nullptr && out != nullptr, "pointers must not be null");
  MX_REQUIRE(rows > 0 && k > 0 && k % 4 == 0,
             "rows must be positive and k must be divisible by four");
  const int64_t n = rows * k;
  const bool vec = aligned(packed, 4) && aligned(out, 16);
  unpack_fp6_kernel<false><<<grid_for(n / 16 + 1), kThreads, 0, stream>>>(packed, out, n, vec);
  MX_CUDA(cudaGetLastError());
  return kOk;
}

int expand_fp6_to_fp8(const uint8_t* packed, int64_t rows, int64_t k, uint8_t* out,
                      cudaStream_t stream) {
  MX_REQUIRE(packed != nullptr && out != nullptr, "pointers must not be null");
  MX_REQUIRE(rows > 0 && k > 0 && k % 16 == 0,
             "rows must be positive and k must be divisible by 16");
  const int64_t n = rows * k;
  const bool vec = aligned(packed, 4) && aligned(out, 16);
  unpack_fp6_kernel<true><<<grid_for(n / 16 + 1), kThreads, 0, stream>>>(packed, out, n, vec);
  MX_CUDA(cudaGetLastError());
  return kOk;
}

int pad_fp6(const uint8_t* packed, int64_t bytes, uint8_t* out, cudaStream_t stream) {
  MX_REQUIRE(packed != nullptr && out != nullptr, "pointers must not be null");
  MX_REQUIRE(bytes > 0 && bytes % 12 == 0, "packed size must be a positive multiple of 12");
  MX_REQUIRE(aligned(packed, 4) && aligned(out, 16), "packed/out must be 4/16-byte aligned");
  pad_fp6_kernel<<<grid_for(bytes / 12), kThreads, 0, stream>>>(packed, out, bytes / 12);
  MX_CUDA(cudaGetLastError());
  return kOk;
}

int pack_scales(const uint8_t* logical, int64_t rows, int64_t k, uint8_t* packed,
                cudaStream_t stream) {
  MX_REQUIRE(logical != nullptr && packed != nullptr, "pointers must not be null");
  MX_REQUIRE(rows > 0 && k > 0 && k % kScaleVec == 0,
             "rows must be positive and k must be divisible by 32");
  pack_scales_kernel<<<grid_for(packed_scale_bytes(rows, k)), kThreads, 0, stream>>>(
      logical, packed, rows, static_cast<int>(k / kScaleVec));
  MX_CUDA(cudaGetLastError());
  return kOk;
}

int unpack_scales(const uint8_t* packed, int64_t rows, int64_t k, uint8_t* logical,
                  cudaStream_t stream) {
  MX_REQUIRE(logical != nullptr && packed != nullptr, "pointers must not be null");
  MX_REQUIRE(rows > 0 && k > 0 && k % kScaleVec == 0,
             "rows must be positive and k must be divisible by 32");
  unpack_scales_kernel<<<grid_for(rows * (k / kScaleVec)), kThreads, 0, stream>>>(
      packed, logical, rows, static_cast<int>(k / kScaleVec));
  MX_CUDA(cudaGetLastError());
  return kOk;
}

int grouped_scale_offsets(const int64_t* expert_offsets, int experts, int64_t* scale_offsets,
                          cudaStream_t stream) {
  MX_REQUIRE(expert_offsets != nullptr && scale_offsets != nullptr, "pointers must not be null");
  MX_REQUIRE(experts > 0, "experts must be positive");
  grouped_scale_offsets_kernel<<<1, 32, 0, stream>>>(expert_offsets, scale_offsets, experts);
  MX_CUDA(cudaGetLastError());
  return kOk;
}

int pack_grouped_scales(const uint8_t* logical, const int64_t* expert_offsets,
                        const int64_t* scale_offsets, int experts, int64_t padded_rows,
                        int64_t k, uint8_t* packed, cudaStream_t stream) {
  MX_REQUIRE(logical != nullptr && packed != nullptr && expert_offsets != nullptr &&
                 scale_offsets != nullptr,
             "pointers must not be null");
  MX_REQUIRE(experts > 0 && padded_rows > 0 && padded_rows % kAtomRows == 0,
             "padded_rows must be a positive multiple of 128");
  MX_REQUIRE(k > 0 && k % kScaleVec == 0, "k must be divisible by 32");
  const int groups = static_cast<int>(k / kScaleVec);
  pack_grouped_scales_kernel<<<grid_for(padded_rows * round_up64(groups, 4)), kThreads, 0,
                               stream>>>(logical, expert_offsets, scale_offsets, experts, packed,
                                         padded_rows, groups);
  MX_CUDA(cudaGetLastError());
  return kOk;
}

}  // namespace mx
