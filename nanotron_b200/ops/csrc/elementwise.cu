// RoPE (in-place capable, strided q/k views of a fused qkv buffer) and SwiGLU forward / backward (sm_100a).
// All are one-pass streaming kernels with 128-bit accesses; the goal is DRAM speed.
#include "common.cuh"

namespace {

// x: [T, H, D] with strides (stride_t, stride_h, 1) in elements.  cos/sin: fp32 [rows, D/2]; row = positions[t] when
// `positions` is given, else t.  One thread rotates 8 pairs.
template <typename T, bool INTERLEAVED>
__global__ void rope_kernel(const T* __restrict__ x, T* __restrict__ out, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                            const int64_t* __restrict__ positions, int tokens, int heads, int dim, int64_t in_stride_t, int64_t in_stride_h,
                            int64_t out_stride_t, int64_t out_stride_h, float sin_sign) {
  const int half = dim >> 1;
  const int groups = half >> 3;  // 8 pairs per thread
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = (int64_t)tokens * heads * groups;
  if (idx >= total) return;
  const int g = (int)(idx % groups);
  const int h = (int)((idx / groups) % heads);
  const int t = (int)(idx / ((int64_t)groups * heads));
  const int64_t row = positions ? positions[t] : t;
  float c[8], s[8];
  {
    const float4* cp = reinterpret_cast<const float4*>(cos_t + row * half + g * 8);
    const float4* sp = reinterpret_cast<const float4*>(sin_t + row * half + g * 8);
    float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
    c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w; c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
    s[0] = s0.x; s[1] = s0.y; s[2] = s0.z; s[3] = s0.w; s[4] = s1.x; s[5] = s1.y; s[6] = s1.z; s[7] = s1.w;
  }
  const T* xin = x + t * in_stride_t + h * in_stride_h;
  T* xout = out + t * out_stride_t + h * out_stride_h;
  Vec8<T> a, b;
  float fa[8], fb[8], oa[8], ob[8];
  if (INTERLEAVED) {
    // 16 consecutive elements = 8 (even, odd) pairs
    a.load(xin + g * 16);
    b.load(xin + g * 16 + 8);
    a.to_float(fa);
    b.to_float(fb);
    float e[16];
#pragma unroll
    for (int i = 0; i < 8; i++) { e[i] = fa[i]; e[8 + i] = fb[i]; }
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const float x1 = e[2 * i], x2 = e[2 * i + 1], ss = s[i] * sin_sign;
      e[2 * i] = x1 * c[i] - x2 * ss;
      e[2 * i + 1] = x1 * ss + x2 * c[i];
    }
#pragma unroll
    for (int i = 0; i < 8; i++) { oa[i] = e[i]; ob[i] = e[8 + i]; }
    a.from_float(oa);
    b.from_float(ob);
    a.store(xout + g * 16);
    b.store(xout + g * 16 + 8);
  } else {
    a.load(xin + g * 8);
    b.load(xin + half + g * 8);
    a.to_float(fa);
    b.to_float(fb);
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const float ss = s[i] * sin_sign;
      oa[i] = fa[i] * c[i] - fb[i] * ss;
      ob[i] = fa[i] * ss + fb[i] * c[i];
    }
    a.from_float(oa);
    b.from_float(ob);
    a.store(xout + g * 8);
    b.store(xout + half + g * 8);
  }
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// gate_up: [rows, 2*inter] = [gate | up]; out: [rows, inter]
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int64_t rows, int inter) {
  const int per_row = inter >> 3;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * per_row) return;
  const int64_t r = idx / per_row;
  const int c = (int)(idx % per_row) * 8;
  Vec8<T> g, u, o;
  float fg[8], fu[8], fo[8];
  g.load(gate_up + r * 2 * inter + c);
  u.load(gate_up + r * 2 * inter + inter + c);
  g.to_float(fg);
  u.to_float(fu);
#pragma unroll
  for (int i = 0; i < 8; i++) fo[i] = fg[i] * sigmoidf_(fg[i]) * fu[i];
  o.from_float(fo);
  o.store(out + r * inter + c);
}

template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ gate_up, const T* __restrict__ dout, T* __restrict__ dgate_up, int64_t rows, int inter) {
  const int per_row = inter >> 3;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * per_row) return;
  const int64_t r = idx / per_row;
  const int c = (int)(idx % per_row) * 8;
  Vec8<T> g, u, d, og, ou;
  float fg[8], fu[8], fd[8], dg[8], du[8];
  g.load(gate_up + r * 2 * inter + c);
  u.load(gate_up + r * 2 * inter + inter + c);
  d.load(dout + r * inter + c);
  g.to_float(fg);
  u.to_float(fu);
  d.to_float(fd);
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const float sg = sigmoidf_(fg[i]);
    dg[i] = fd[i] * fu[i] * sg * (1.f + fg[i] * (1.f - sg));
    du[i] = fd[i] * fg[i] * sg;
  }
  og.from_float(dg);
  ou.from_float(du);
  og.store(dgate_up + r * 2 * inter + c);
  ou.store(dgate_up + r * 2 * inter + inter + c);
}

}  // namespace

NTB_EXPORT int ntb_rope(int dtype, const void* x, void* out, const float* cos_t, const float* sin_t, const int64_t* positions, int tokens, int heads,
                        int dim, int64_t in_stride_t, int64_t in_stride_h, int64_t out_stride_t, int64_t out_stride_h, int interleaved, int inverse,
                        cudaStream_t stream) {
  if (tokens <= 0 || heads <= 0 || dim % 16 != 0) return NTB_ERR_ARG;
  if (in_stride_t % 8 || in_stride_h % 8 || out_stride_t % 8 || out_stride_h % 8) return NTB_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) return NTB_ERR_ARG;
  const int64_t total = (int64_t)tokens * heads * (dim / 16);
  const int threads = 256;
  const int64_t blocks = (total + threads - 1) / threads;
  const float sign = inverse ? -1.f : 1.f;
  NTB_DISPATCH_DTYPE(dtype, {
    if (interleaved)
      rope_kernel<T, true><<<(unsigned)blocks, threads, 0, stream>>>((const T*)x, (T*)out, cos_t, sin_t, positions, tokens, heads, dim, in_stride_t, in_stride_h, out_stride_t, out_stride_h, sign);
    else
      rope_kernel<T, false><<<(unsigned)blocks, threads, 0, stream>>>((const T*)x, (T*)out, cos_t, sin_t, positions, tokens, heads, dim, in_stride_t, in_stride_h, out_stride_t, out_stride_h, sign);
  });
  return ntb_check_launch();
}

NTB_EXPORT int ntb_swiglu_fwd(int dtype, const void* gate_up, void* out, int64_t rows, int inter, cudaStream_t stream) {
  if (rows <= 0 || inter <= 0 || inter % 8 != 0) return NTB_ERR_ARG;
  const int64_t total = rows * (inter / 8);
  const int threads = 256;
  NTB_DISPATCH_DTYPE(dtype, { swiglu_fwd_kernel<T><<<(unsigned)((total + threads - 1) / threads), threads, 0, stream>>>((const T*)gate_up, (T*)out, rows, inter); });
  return ntb_check_launch();
}

NTB_EXPORT int ntb_swiglu_bwd(int dtype, const void* gate_up, const void* dout, void* dgate_up, int64_t rows, int inter, cudaStream_t stream) {
  if (rows <= 0 || inter <= 0 || inter % 8 != 0) return NTB_ERR_ARG;
  const int64_t total = rows * (inter / 8);
  const int threads = 256;
  NTB_DISPATCH_DTYPE(dtype, { swiglu_bwd_kernel<T><<<(unsigned)((total + threads - 1) / threads), threads, 0, stream>>>((const T*)gate_up, (const T*)dout, (T*)dgate_up, rows, inter); });
  return ntb_check_launch();
}
