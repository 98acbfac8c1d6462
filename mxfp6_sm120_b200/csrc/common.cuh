// Shared host/device helpers for the sm_100a W6A8 library.
//
// Formats (OCP MX): weights are E3M2 codes packed four-to-three-bytes as a
// little-endian bitstream, activations are E4M3 bytes, and both carry one
// UE8M0 scale byte per 32 consecutive K values.  Packed scales use the
// 128-row x 4-group "atom" order that tcgen05.cp moves into tensor memory.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>
#include <cstdio>
#include <cstdarg>

namespace mx {

constexpr int kScaleVec = 32;          // K values per UE8M0 scale
constexpr int kAtomRows = 128;         // rows per packed-scale atom
constexpr int kAtomGroups = 4;         // k-groups per packed-scale atom
constexpr uint8_t kUe8m0One = 0x7f;    // UE8M0 encoding of 1.0

enum Status : int {
  kOk = 0,
  kInvalidArgument = 1,
  kCudaError = 2,
  kUnsupported = 3,
  kDeviceTimeout = 4,
  kWorkspaceError = 5,
};

enum DType : int { kF16 = 0, kBF16 = 1, kF32 = 2 };

// Thread-local error text for the C ABI.
void set_error(const char* fmt, ...);
const char* last_error();

#define MX_REQUIRE(cond, ...)                         \
  do {                                                \
    if (!(cond)) {                                    \
      ::mx::set_error(__VA_ARGS__);                   \
      return ::mx::kInvalidArgument;                  \
    }                                                 \
  } while (0)

#define MX_CUDA(expr)                                                        \
  do {                                                                       \
    cudaError_t mx_err__ = (expr);                                           \
    if (mx_err__ != cudaSuccess) {                                           \
      ::mx::set_error("%s failed: %s", #expr, cudaGetErrorString(mx_err__)); \
      return ::mx::kCudaError;                                               \
    }                                                                        \
  } while (0)

// SiLU table (silu_table.cu): s = bf16(g / (1 + expf(-g))) for every BF16 bit pattern of g.
int silu_table(cudaStream_t stream, const uint16_t** out);
#ifdef __CUDACC__
// `g` must already be rounded to BF16 (its low 16 bits are zero).
__device__ __forceinline__ float silu_bf16_lookup(const uint16_t* __restrict__ table, float g) {
  return __uint_as_float(static_cast<uint32_t>(__ldg(table + (__float_as_uint(g) >> 16))) << 16);
}
#endif

__host__ __device__ __forceinline__ int64_t ceil_div64(int64_t a, int64_t b) {
  return (a + b - 1) / b;
}
__host__ __device__ __forceinline__ int64_t round_up64(int64_t a, int64_t b) {
  return ceil_div64(a, b) * b;
}

// Byte offset of the scale of (row, k_group) inside a packed-scale buffer whose
// rows hold `k_groups` groups.  Same order as the reference's
// dense_scale_offset (csrc/moe.cu:587-600) and pack_scales_kernel
// (csrc/packing.cu:239-263).
__host__ __device__ __forceinline__ int64_t packed_scale_offset(int64_t row, int k_group,
                                                                int k_groups) {
  const int64_t atoms_per_row_block = (k_groups + kAtomGroups - 1) / kAtomGroups;
  const int64_t atom = (row / kAtomRows) * atoms_per_row_block + k_group / kAtomGroups;
  const int r = static_cast<int>(row % kAtomRows);
  return atom * (kAtomRows * kAtomGroups) + (r % 32) * 16 + (r / 32) * 4 + k_group % kAtomGroups;
}

__host__ __device__ __forceinline__ int64_t packed_scale_bytes(int64_t rows, int64_t k) {
  return round_up64(rows, kAtomRows) * round_up64(k / kScaleVec, kAtomGroups);
}

#ifdef __CUDACC__
template <class T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <>
__device__ __forceinline__ float to_float<__half>(__half v) {
  return __half2float(v);
}

// Round-to-nearest-even float -> bf16 -> float.
__device__ __forceinline__ float round_bf16(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

// UE8M0 scale selection of the reference quantizer (csrc/quantization.cu:118-131):
// smallest power of two >= absmax / target_max, with a 1e-30 floor, returned as the
// FP32 bit pattern of that power of two.
//
// The reference divides (IEEE) and rounds the quotient's bits up to a power of two.
// Both targets are 1.75 * 2^s (448 = 1.75 * 2^8, 28 = 1.75 * 2^4), so with
// absmax = 1.m * 2^e the result is 2^(e - s) when 1.m <= 1.75 and 2^(e - s + 1)
// otherwise: integer work on the exponent and mantissa fields, no division.  This
// is exact for FP16/BF16 inputs: their absmax has at most 11 significant bits, so
// the quotient is never within one FP32 rounding of a power of two unless it IS
// one.  The floor ceil_pow2(1e-30) = 2^-99 is exponent field 28.
template <int kTargetShift>  // 8 for E4M3 (448), 4 for E3M2 (28)
__device__ __forceinline__ uint32_t ue8m0_scale_bits_shift(float absmax) {
  const uint32_t b = __float_as_uint(absmax);
  int code = static_cast<int>(b >> 23) - kTargetShift + ((b & 0x7fffffu) > 0x600000u ? 1 : 0);
  code = code < 28 ? 28 : code;
  return static_cast<uint32_t>(code) << 23;
}
__device__ __forceinline__ uint32_t ue8m0_scale_bits(float absmax, float target_max) {
  return target_max == 448.0f ? ue8m0_scale_bits_shift<8>(absmax)
                              : ue8m0_scale_bits_shift<4>(absmax);
}
// Exact reciprocal of the power of two whose bits are `scale_bits`.
__device__ __forceinline__ float ue8m0_inverse(uint32_t scale_bits) {
  return __uint_as_float((254u << 23) - scale_bits);
}
#endif

}  // namespace mx
