// MoE router forward (sm_100a): logits = x W^T in fp32, softmax over experts, top-k selection and the per-expert token
// histogram, in one kernel.  x: bf16 [T, h]; W: fp32 [E, h] (E <= 128, multiple of 16).  One CTA handles 64 tokens with a
// register-tiled fp32 product: x and W stream through shared memory in chunks of 32 columns, thread (tg, eg) of the 16 x 16
// grid accumulates tokens 4 tg .. 4 tg + 3 against experts eg, eg + 16, ... (one 16-byte and E / 16 4-byte shared loads per
// 4 * E / 16 FMAs, so W is read from L2 once per 64 tokens).  Then each warp finishes eight tokens: softmax with warp
// reductions, k rounds of warp arg-max.  The histogram (tokens routed to each expert, over all k slots) is accumulated with
// one atomicAdd per selection.
#include "common.cuh"

namespace {

constexpr int R_TOK = 64;
constexpr int R_CHUNK = 32;
constexpr int R_THREADS = 256;
constexpr int R_MAX_E = 128;
constexpr int R_WPITCH = R_CHUNK + 1;

__global__ void __launch_bounds__(R_THREADS) router_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w, float* __restrict__ probs,
                                                              float* __restrict__ top_p, int* __restrict__ top_i, int* __restrict__ counts, int T, int h, int E,
                                                              int k) {
  extern __shared__ float smem[];
  float* sx = smem;                        // [R_CHUNK][R_TOK]   (column-major: four consecutive tokens = one 16-byte load)
  float* sw = sx + R_CHUNK * R_TOK;        // [E][R_WPITCH]
  float* slog = sw + E * R_WPITCH;         // [R_TOK][E]
  const int tok0 = blockIdx.x * R_TOK;
  const int tg = threadIdx.x >> 4, eg = threadIdx.x & 15;
  const int EJ = E >> 4;
  float acc[4][8];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 8; j++) acc[i][j] = 0.f;
  for (int c0 = 0; c0 < h; c0 += R_CHUNK) {
    {  // x chunk: 64 tokens x 32 columns = 256 x 8 bf16
      const int t = threadIdx.x >> 2, cg = threadIdx.x & 3;
      const int tok = tok0 + t;
      float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      if (tok < T && c0 + cg * 8 + 8 <= h) {
        const uint4 raw = *reinterpret_cast<const uint4*>(x + static_cast<int64_t>(tok) * h + c0 + cg * 8);
        const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int q = 0; q < 4; q++) {
          const float2 f = __bfloat1622float2(hh[q]);
          v[2 * q] = f.x;
          v[2 * q + 1] = f.y;
        }
      } else if (tok < T) {
        for (int q = 0; q < 8; q++)
          if (c0 + cg * 8 + q < h) v[q] = __bfloat162float(x[static_cast<int64_t>(tok) * h + c0 + cg * 8 + q]);
      }
#pragma unroll
      for (int q = 0; q < 8; q++) sx[(cg * 8 + q) * R_TOK + t] = v[q];
    }
    for (int i = threadIdx.x; i < E * (R_CHUNK / 4); i += R_THREADS) {
      const int e = i >> 3, c4 = i & 7;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      const float* src = w + static_cast<int64_t>(e) * h + c0 + c4 * 4;
      if (c0 + c4 * 4 + 4 <= h) v = *reinterpret_cast<const float4*>(src);
      else {
        if (c0 + c4 * 4 + 0 < h) v.x = src[0];
        if (c0 + c4 * 4 + 1 < h) v.y = src[1];
        if (c0 + c4 * 4 + 2 < h) v.z = src[2];
      }
      float* dst = sw + e * R_WPITCH + c4 * 4;
      dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
    }
    __syncthreads();
#pragma unroll 4
    for (int c = 0; c < R_CHUNK; c++) {
      const float4 xv = *reinterpret_cast<const float4*>(sx + c * R_TOK + tg * 4);
#pragma unroll
      for (int j = 0; j < 8; j++) {
        if (j < EJ) {
          const float wv = sw[(eg + 16 * j) * R_WPITCH + c];
          acc[0][j] = fmaf(xv.x, wv, acc[0][j]);
          acc[1][j] = fmaf(xv.y, wv, acc[1][j]);
          acc[2][j] = fmaf(xv.z, wv, acc[2][j]);
          acc[3][j] = fmaf(xv.w, wv, acc[3][j]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 8; j++)
      if (j < EJ) slog[(tg * 4 + i) * E + eg + 16 * j] = acc[i][j];
  __syncthreads();
  // each warp finishes R_TOK / 8 tokens
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int t = warp; t < R_TOK; t += R_THREADS / 32) {
    const int tok = tok0 + t;
    if (tok >= T) continue;
    float v[R_MAX_E / 32];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < R_MAX_E / 32; j++) {
      const int e = lane + 32 * j;
      v[j] = e < E ? slog[t * E + e] : -INFINITY;
      mx = fmaxf(mx, v[j]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < R_MAX_E / 32; j++) {
      v[j] = (lane + 32 * j < E) ? expf(v[j] - mx) : 0.f;
      sum += v[j];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int j = 0; j < R_MAX_E / 32; j++) {
      v[j] *= inv;
      if (lane + 32 * j < E) probs[static_cast<int64_t>(tok) * E + lane + 32 * j] = v[j];
    }
    // top-k by repeated arg-max (ties: lowest expert index)
    for (int s = 0; s < k; s++) {
      float best = -1.f;
      int best_e = 0x7fffffff;
#pragma unroll
      for (int j = 0; j < R_MAX_E / 32; j++) {
        const int e = lane + 32 * j;
        if (e < E && (v[j] > best || (v[j] == best && e < best_e))) { best = v[j]; best_e = e; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
        if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
      }
      if (lane == 0) {
        top_p[static_cast<int64_t>(tok) * k + s] = best;
        top_i[static_cast<int64_t>(tok) * k + s] = best_e;
        atomicAdd(counts + best_e, 1);
      }
#pragma unroll
      for (int j = 0; j < R_MAX_E / 32; j++)
        if (lane + 32 * j == best_e) v[j] = -2.f;  // remove the winner
    }
  }
}

}  // namespace

// counts (int32 [E]) must be zero on entry.
NTB_EXPORT int ntb_moe_router_fwd(const void* x, const float* w, float* probs, float* top_p, int* top_i, int* counts, int T, int h, int E, int k,
                                  cudaStream_t stream) {
  if (T <= 0 || h <= 0 || h % 8 || E <= 0 || E > R_MAX_E || E % 16 || k <= 0 || k > E) return NTB_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) return NTB_ERR_ARG;
  const size_t smem = sizeof(float) * (R_TOK * R_CHUNK + E * R_WPITCH + R_TOK * E);
  static bool configured = false;
  if (!configured && smem > 48 * 1024) {
    if (cudaFuncSetAttribute(router_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024) != cudaSuccess) return NTB_ERR_LAUNCH;
    configured = true;
  }
  router_fwd_kernel<<<(T + R_TOK - 1) / R_TOK, R_THREADS, smem, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), w, probs, top_p, top_i, counts, T, h, E, k);
  return ntb_check_launch();
}
