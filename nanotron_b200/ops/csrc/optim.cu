// Flat AdamW over fp32 master weights with fused gradient scaling and bf16 write-back, and a flat sum of squares
// (gradient norm) (sm_100a).
//
// The optimizer state of a rank is a set of equally laid out flat buffers (fp32 master, exp_avg, exp_avg_sq) whose
// element i corresponds to element i of a contiguous range of the fp32 gradient buffer and of the half-precision
// parameter buffer.  Hyper-parameters that differ per parameter group (lr, weight decay) come from a small segment
// table: segment k covers elements [seg_end[k-1], seg_end[k]).
#include "common.cuh"

namespace {

constexpr int OPT_THREADS = 256;
constexpr int OPT_ITEMS = 4;  // float4 per thread per iteration

__global__ void __launch_bounds__(OPT_THREADS) adamw_flat_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                                                                 __nv_bfloat16* __restrict__ p16, int64_t n, const int64_t* __restrict__ seg_end,
                                                                 const float* __restrict__ seg_lr, const float* __restrict__ seg_wd, int nseg, float beta1,
                                                                 float beta2, float eps, float inv_bc1, float inv_sqrt_bc2, const float* __restrict__ grad_scale) {
  const float gs = grad_scale ? *grad_scale : 1.f;
  const int64_t stride = (int64_t)gridDim.x * OPT_THREADS * OPT_ITEMS;
  for (int64_t base = ((int64_t)blockIdx.x * OPT_THREADS + threadIdx.x) * OPT_ITEMS; base < n; base += stride) {
    // segment lookup (binary search; tables are tiny and stay in L1)
    int lo = 0, hi = nseg - 1;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (seg_end[mid] > base) hi = mid; else lo = mid + 1;
    }
    const float lr = seg_lr[lo], wd = seg_wd[lo];
    float4 pv = *reinterpret_cast<const float4*>(p + base);
    const float4 gv = *reinterpret_cast<const float4*>(g + base);
    float4 mv = *reinterpret_cast<const float4*>(m + base);
    float4 vv = *reinterpret_cast<const float4*>(v + base);
    float* pp = reinterpret_cast<float*>(&pv);
    const float* gp = reinterpret_cast<const float*>(&gv);
    float* mp = reinterpret_cast<float*>(&mv);
    float* vp = reinterpret_cast<float*>(&vv);
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const float gi = gp[i] * gs;
      float pi = pp[i] * (1.f - lr * wd);
      mp[i] = beta1 * mp[i] + (1.f - beta1) * gi;
      vp[i] = beta2 * vp[i] + (1.f - beta2) * gi * gi;
      const float denom = sqrtf(vp[i]) * inv_sqrt_bc2 + eps;
      pi -= lr * inv_bc1 * mp[i] / denom;
      pp[i] = pi;
    }
    *reinterpret_cast<float4*>(p + base) = pv;
    *reinterpret_cast<float4*>(m + base) = mv;
    *reinterpret_cast<float4*>(v + base) = vv;
    if (p16) {
      __nv_bfloat162 lo2 = __floats2bfloat162_rn(pp[0], pp[1]);
      __nv_bfloat162 hi2 = __floats2bfloat162_rn(pp[2], pp[3]);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&lo2);
      pk.y = *reinterpret_cast<uint32_t*>(&hi2);
      *reinterpret_cast<uint2*>(p16 + base) = pk;
    }
  }
}

__global__ void __launch_bounds__(OPT_THREADS) sumsq_kernel(const float* __restrict__ x, int64_t n, float* __restrict__ partial) {
  __shared__ float scratch[32];
  float s = 0.f;
  const int64_t stride = (int64_t)gridDim.x * OPT_THREADS * 4;
  const int64_t n4 = (n / 4) * 4;
  for (int64_t i = ((int64_t)blockIdx.x * OPT_THREADS + threadIdx.x) * 4; i < n4; i += stride) {
    const float4 a = *reinterpret_cast<const float4*>(x + i);
    s += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
  }
  if (blockIdx.x == 0) {
    for (int64_t i = n4 + threadIdx.x; i < n; i += OPT_THREADS) s += x[i] * x[i];
  }
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

__global__ void sumsq_final_kernel(const float* __restrict__ partial, int nparts, float* __restrict__ out, int accumulate) {
  __shared__ float scratch[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) s += partial[i];
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + s : s;
}

}  // namespace

// n must be a multiple of 4 and all pointers 16-byte aligned (8-byte for p16).
NTB_EXPORT int ntb_adamw_flat(float* p, const float* g, float* m, float* v, void* p16, int64_t n, const int64_t* seg_end, const float* seg_lr,
                              const float* seg_wd, int nseg, float beta1, float beta2, float eps, float bias_correction1, float bias_correction2,
                              const float* grad_scale, cudaStream_t stream) {
  if (n <= 0 || n % 4 != 0 || nseg <= 0) return NTB_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v)) & 15) return NTB_ERR_ARG;
  if (reinterpret_cast<uintptr_t>(p16) & 7) return NTB_ERR_ARG;
  int64_t blocks = (n / OPT_ITEMS + OPT_THREADS - 1) / OPT_THREADS;
  const int64_t cap = 148 * 16;
  if (blocks > cap) blocks = cap;
  adamw_flat_kernel<<<(unsigned)blocks, OPT_THREADS, 0, stream>>>(p, g, m, v, (__nv_bfloat16*)p16, n, seg_end, seg_lr, seg_wd, nseg, beta1, beta2, eps,
                                                                   1.f / bias_correction1, rsqrtf(bias_correction2), grad_scale);
  return ntb_check_launch();
}

NTB_EXPORT int ntb_sumsq_num_partials() { return 148 * 8; }

// out[0] (+)= sum x^2.  partial: fp32 [ntb_sumsq_num_partials()].
NTB_EXPORT int ntb_sumsq(const float* x, int64_t n, float* partial, float* out, int accumulate, cudaStream_t stream) {
  if (n <= 0 || (reinterpret_cast<uintptr_t>(x) & 15)) return NTB_ERR_ARG;
  const int nparts = ntb_sumsq_num_partials();
  sumsq_kernel<<<nparts, OPT_THREADS, 0, stream>>>(x, n, partial);
  sumsq_final_kernel<<<1, 256, 0, stream>>>(partial, nparts, out, accumulate);
  return ntb_check_launch();
}
