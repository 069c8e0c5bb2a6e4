// Shared device helpers for the nanotron_b200 kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define NTB_OK 0
#define NTB_ERR_ARG 1      // unsupported shape / alignment (nothing launched)
#define NTB_ERR_LAUNCH 2   // cudaGetLastError() reported a failure
#define NTB_ERR_TIMEOUT 3  // a bounded device-side wait ran out (see status word)

#define NTB_EXPORT extern "C" __attribute__((visibility("default")))

// cuTensorMapEncodeTiled is a driver-API call and needs a CUDA context current on the CALLING THREAD.  The runtime binds the
// device's primary context to a thread at its first runtime call that needs one; a fresh thread whose first CUDA work is one
// of the tensor-map builders below has none yet (seen with autograd worker threads on device 0, where the framework skips
// cudaSetDevice because device 0 is already the thread's default): the encode call then fails and the entry point would
// report the arguments as unsupported.  Binding once per thread costs two runtime calls.
static inline void ntb_bind_context_to_thread() {
  static thread_local bool bound = false;
  if (bound) return;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess && cudaSetDevice(dev) == cudaSuccess && cudaFree(nullptr) == cudaSuccess) bound = true;
}

static inline int ntb_check_launch() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? NTB_OK : NTB_ERR_LAUNCH;
}

// dtype codes shared with the Python side
enum NtbDtype { NTB_F32 = 0, NTB_BF16 = 1, NTB_F16 = 2 };

template <typename T> struct Vec8;  // 8 elements = one or two 128-bit accesses

template <> struct Vec8<__nv_bfloat16> {
  uint4 raw;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) { raw = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ void store(__nv_bfloat16* p) const { *reinterpret_cast<uint4*>(p) = raw; }
  __device__ __forceinline__ void to_float(float (&f)[8]) const {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; i++) { float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
  }
  __device__ __forceinline__ void from_float(const float (&f)[8]) {
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; i++) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  }
};

template <> struct Vec8<__half> {
  uint4 raw;
  __device__ __forceinline__ void load(const __half* p) { raw = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ void store(__half* p) const { *reinterpret_cast<uint4*>(p) = raw; }
  __device__ __forceinline__ void to_float(float (&f)[8]) const {
    const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; i++) { float2 t = __half22float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
  }
  __device__ __forceinline__ void from_float(const float (&f)[8]) {
    __half2* h = reinterpret_cast<__half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; i++) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
  }
};

template <> struct Vec8<float> {
  float4 a, b;
  __device__ __forceinline__ void load(const float* p) { a = *reinterpret_cast<const float4*>(p); b = *reinterpret_cast<const float4*>(p + 4); }
  __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = a; *reinterpret_cast<float4*>(p + 4) = b; }
  __device__ __forceinline__ void to_float(float (&f)[8]) const { f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w; }
  __device__ __forceinline__ void from_float(const float (&f)[8]) { a = make_float4(f[0], f[1], f[2], f[3]); b = make_float4(f[4], f[5], f[6], f[7]); }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; every thread gets the result. `scratch` holds >= 32 floats. Safe to call repeatedly.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? scratch[lane] : 0.f;
  return warp_sum(r);
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? scratch[lane] : -INFINITY;
  return warp_max(r);
}

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

#define NTB_DISPATCH_DTYPE(dtype, ...)                                  \
  switch (dtype) {                                                      \
    case NTB_F32: { using T = float; __VA_ARGS__; break; }              \
    case NTB_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }     \
    case NTB_F16: { using T = __half; __VA_ARGS__; break; }             \
    default: return NTB_ERR_ARG;                                        \
  }
