// SiLU of a BF16 value, rounded to BF16, for all 65536 BF16 bit patterns.
//
// The activation rule of this library (the reference's, csrc/moe.cu:5199-5205) rounds the
// gate to BF16 first and the SiLU result to BF16 again: s = bf16(g / (1 + expf(-g))) is a
// pure function of 16 input bits.  The table is filled ON THE DEVICE by that very formula
// (so a lookup is bit-identical to evaluating it) and replaces an expf, an IEEE division
// and a rounding per element, which made the activation kernels instruction-bound.
// 128 KB in the library image, no allocation; most lookups hit L1 because activations
// occupy a few thousand distinct codes.
#include "common.cuh"

namespace mx {
namespace {

__device__ uint16_t g_silu_table[65536];

__global__ void silu_table_kernel(uint16_t* table) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  const float g = __uint_as_float(i << 16);
  const float sv = round_bf16(__fdiv_rn(g, 1.0f + expf(-g)));
  table[i] = static_cast<uint16_t>(__float_as_uint(sv) >> 16);
}

}  // namespace

// Device pointer of the table on the current device; fills it on first use.  The first
// use outside stream capture waits for the fill once (like other one-time set-up); a use
// inside a capture records the fill into the capture instead and leaves the table marked
// unfilled, so every graph stands on its own.
int silu_table(cudaStream_t stream, const uint16_t** out) {
  static bool filled[64] = {};
  static uint16_t* address[64] = {};
  int device = 0;
  MX_CUDA(cudaGetDevice(&device));
  MX_REQUIRE(device >= 0 && device < 64, "device index %d is out of range", device);
  if (address[device] == nullptr) {
    void* p = nullptr;
    MX_CUDA(cudaGetSymbolAddress(&p, g_silu_table));
    address[device] = static_cast<uint16_t*>(p);
  }
  if (!filled[device]) {
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    MX_CUDA(cudaStreamIsCapturing(stream, &capture));
    silu_table_kernel<<<256, 256, 0, stream>>>(address[device]);
    MX_CUDA(cudaGetLastError());
    if (capture == cudaStreamCaptureStatusNone) {
      MX_CUDA(cudaStreamSynchronize(stream));
      filled[device] = true;
    }
  }
  *out = address[device];
  return kOk;
}

}  // namespace mx
