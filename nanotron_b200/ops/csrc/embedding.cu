// Vocabulary-parallel embedding lookup and its backward (sm_100a).
//
// forward : out[t, :] = weight[ids[t] - min_id, :] when min_id <= ids[t] < max_id, else zeros (the other tensor-parallel ranks own the
//           row; the partial results are then summed by the reduce-scatter / all-reduce that follows).  Gather and mask are one
//           pass: no `masked_fill` of the ids, no second pass over the [T, h] output.
// backward: dweight[ids[t] - min_id, :] += dout[t, :] in fp32 straight into the main-gradient buffer (16-byte vector atomics), so no
//           bf16 weight-gradient tensor of the size of the embedding table is materialised.
#include "common.cuh"

namespace {

template <typename T>
__global__ void embedding_fwd_kernel(const int64_t* __restrict__ ids, const T* __restrict__ weight, T* __restrict__ out, int64_t n, int h8, int64_t min_id,
                                     int64_t max_id) {
  // one warp per token row, 16 bytes per lane per step
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t t = warp; t < n; t += nwarps) {
    const int64_t id = ids[t];
    uint4* dst = reinterpret_cast<uint4*>(out) + t * h8;
    if (id >= min_id && id < max_id) {
      const uint4* src = reinterpret_cast<const uint4*>(weight) + (id - min_id) * h8;
      for (int v = lane; v < h8; v += 32) dst[v] = __ldg(src + v);
    } else {
      for (int v = lane; v < h8; v += 32) dst[v] = make_uint4(0, 0, 0, 0);
    }
  }
}

template <typename T>
__global__ void embedding_bwd_kernel(const int64_t* __restrict__ ids, const T* __restrict__ dout, float* __restrict__ dweight, int64_t n, int h, int64_t min_id,
                                     int64_t max_id) {
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t t = warp; t < n; t += nwarps) {
    const int64_t id = ids[t];
    if (id < min_id || id >= max_id) continue;
    float* dst = dweight + (id - min_id) * h;
    const T* src = dout + t * h;
    for (int c = lane * 8; c < h; c += 256) {
      Vec8<T> v;
      float f[8];
      v.load(src + c);
      v.to_float(f);
      atomicAdd(reinterpret_cast<float4*>(dst + c), make_float4(f[0], f[1], f[2], f[3]));
      atomicAdd(reinterpret_cast<float4*>(dst + c + 4), make_float4(f[4], f[5], f[6], f[7]));
    }
  }
}

}  // namespace

// ids: int64 [n]; weight: [max_id - min_id, h]; out: [n, h].  h * sizeof(T) must be a multiple of 16 bytes.
NTB_EXPORT int ntb_embedding_fwd(int dtype, const int64_t* ids, const void* weight, void* out, int64_t n, int h, int64_t min_id, int64_t max_id,
                                 cudaStream_t stream) {
  if (n <= 0 || h <= 0 || max_id <= min_id) return NTB_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(out)) & 15) return NTB_ERR_ARG;
  int64_t blocks = (n + 7) / 8;
  if (blocks > 148 * 16) blocks = 148 * 16;
  NTB_DISPATCH_DTYPE(dtype, {
    const int per16 = 16 / sizeof(T);
    if (h % per16) return NTB_ERR_ARG;
    embedding_fwd_kernel<T><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(ids, (const T*)weight, (T*)out, n, h / per16, min_id, max_id);
  });
  return ntb_check_launch();
}

// dweight: fp32 [max_id - min_id, h], accumulated into.  h must be a multiple of 8.
NTB_EXPORT int ntb_embedding_bwd(int dtype, const int64_t* ids, const void* dout, float* dweight, int64_t n, int h, int64_t min_id, int64_t max_id,
                                 cudaStream_t stream) {
  if (n <= 0 || h <= 0 || h % 8 || max_id <= min_id) return NTB_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(dout) | reinterpret_cast<uintptr_t>(dweight)) & 15) return NTB_ERR_ARG;
  int64_t blocks = (n + 7) / 8;
  if (blocks > 148 * 16) blocks = 148 * 16;
  NTB_DISPATCH_DTYPE(dtype, { embedding_bwd_kernel<T><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(ids, (const T*)dout, dweight, n, h, min_id, max_id); });
  return ntb_check_launch();
}
