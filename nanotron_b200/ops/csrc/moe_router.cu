// MoE router forward (sm_100a): logits = x W^T in fp32, softmax over experts, top-k selection and the per-expert token
// histogram, in one kernel.  x: bf16 [T, h]; W: fp32 [E, h] (E <= 128, multiple of 32).  One CTA handles 16 tokens:
// x and W are streamed through shared memory in chunks of 128 columns, every thread accumulates 16*E/256 (token, expert)
// dot products, then each warp finishes two tokens: softmax with warp reductions, k rounds of warp arg-max.
// The histogram (tokens routed to each expert, over all k slots) is accumulated with one atomicAdd per selection.
#include "common.cuh"

namespace {

constexpr int R_TOK = 16;
constexpr int R_CHUNK = 128;
constexpr int R_THREADS = 256;
constexpr int R_MAX_E = 128;

__global__ void __launch_bounds__(R_THREADS) router_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w, float* __restrict__ probs,
                                                              float* __restrict__ top_p, int* __restrict__ top_i, int* __restrict__ counts, int T, int h, int E,
                                                              int k) {
  extern __shared__ float smem[];
  float* sx = smem;                       // [R_TOK][R_CHUNK]
  float* sw = sx + R_TOK * R_CHUNK;       // [E][R_CHUNK + 1]
  float* slog = sw + E * (R_CHUNK + 1);   // [R_TOK][E]
  const int tok0 = blockIdx.x * R_TOK;
  const int per_thread = R_TOK * E / R_THREADS;  // outputs per thread (E multiple of 16)
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; i++) acc[i] = 0.f;
  for (int c0 = 0; c0 < h; c0 += R_CHUNK) {
    for (int i = threadIdx.x; i < R_TOK * R_CHUNK; i += R_THREADS) {
      const int t = i / R_CHUNK, c = i % R_CHUNK;
      const int tok = tok0 + t;
      sx[i] = (tok < T && c0 + c < h) ? __bfloat162float(x[static_cast<int64_t>(tok) * h + c0 + c]) : 0.f;
    }
    for (int i = threadIdx.x; i < E * R_CHUNK; i += R_THREADS) {
      const int e = i / R_CHUNK, c = i % R_CHUNK;
      sw[e * (R_CHUNK + 1) + c] = (c0 + c < h) ? w[static_cast<int64_t>(e) * h + c0 + c] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int o = 0; o < 8; o++) {
      if (o < per_thread) {
        const int idx = threadIdx.x + o * R_THREADS;  // (token, expert) pair
        const int t = idx / E, e = idx % E;
        const float* xr = sx + t * R_CHUNK;
        const float* wr = sw + e * (R_CHUNK + 1);
        float s = acc[o];
#pragma unroll 8
        for (int c = 0; c < R_CHUNK; c++) s = fmaf(xr[c], wr[c], s);
        acc[o] = s;
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int o = 0; o < 8; o++)
    if (o < per_thread) slog[threadIdx.x + o * R_THREADS] = acc[o];
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
  if (T <= 0 || h <= 0 || E <= 0 || E > R_MAX_E || E % 16 || k <= 0 || k > E || (R_TOK * E) % R_THREADS || R_TOK * E / R_THREADS > 8) return NTB_ERR_ARG;
  const size_t smem = sizeof(float) * (R_TOK * R_CHUNK + E * (R_CHUNK + 1) + R_TOK * E);
  static bool configured = false;
  if (!configured && smem > 48 * 1024) {
    if (cudaFuncSetAttribute(router_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024) != cudaSuccess) return NTB_ERR_LAUNCH;
    configured = true;
  }
  router_fwd_kernel<<<(T + R_TOK - 1) / R_TOK, R_THREADS, smem, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), w, probs, top_p, top_i, counts, T, h, E, k);
  return ntb_check_launch();
}
