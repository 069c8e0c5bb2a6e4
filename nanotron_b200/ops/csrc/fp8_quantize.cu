// Block-scaled fp8 quantisation, 1 x 128 blocks (sm_100a): one warp per (row, 128-column block); each lane handles 4
// consecutive bf16 values, the block amax is a warp reduction, the scale is amax / fmax and the payload is written as
// 4 packed fp8 bytes per lane.  One read of the source, one write of payload + scales.
#include <cuda_fp8.h>

#include "common.cuh"

namespace {

template <bool E5M2>
__global__ void quantize_1x128_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scale, int64_t rows, int blocks_per_row) {
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= rows * blocks_per_row) return;
  const int64_t row = warp / blocks_per_row;
  const int blk = static_cast<int>(warp % blocks_per_row);
  const int64_t base = (row * blocks_per_row + blk) * 128 + lane * 4;
  const uint2 raw = *reinterpret_cast<const uint2*>(x + base);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
  const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
  float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
  amax = fmaxf(warp_max(amax), 1e-12f);
  const float fmax = E5M2 ? 57344.f : 448.f;
  const float s = amax / fmax;
  const float inv = 1.f / s;
  uint32_t packed;
  if (E5M2) {
    const __nv_fp8x4_e5m2 v(make_float4(a.x * inv, a.y * inv, b.x * inv, b.y * inv));
    packed = *reinterpret_cast<const uint32_t*>(&v);
  } else {
    const __nv_fp8x4_e4m3 v(make_float4(a.x * inv, a.y * inv, b.x * inv, b.y * inv));
    packed = *reinterpret_cast<const uint32_t*>(&v);
  }
  *reinterpret_cast<uint32_t*>(q + base) = packed;
  if (lane == 0) scale[row * blocks_per_row + blk] = s;
}

}  // namespace

// x: bf16 [rows, cols] contiguous, cols % 128 == 0.  q: fp8 bytes [rows, cols].  scale: fp32 [rows, cols / 128].
NTB_EXPORT int ntb_fp8_quantize_1x128(const void* x, void* q, float* scale, int64_t rows, int cols, int e5m2, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0 || cols % 128) return NTB_ERR_ARG;
  const int bpr = cols / 128;
  const int64_t warps = rows * bpr;
  const unsigned blocks = static_cast<unsigned>((warps * 32 + 255) / 256);
  if (e5m2) quantize_1x128_kernel<true><<<blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<uint8_t*>(q), scale, rows, bpr);
  else quantize_1x128_kernel<false><<<blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<uint8_t*>(q), scale, rows, bpr);
  return ntb_check_launch();
}
