// Data-parallel gradient / parameter exchange over NVLink peer memory, fused with the optimizer (sm_100a).
//
// Every rank of a node-local group maps the other ranks' flat buffers (symmetric memory: same layout everywhere) and
// receives the table of peer base pointers.  Three kernels make up one ZeRO-1 optimizer step:
//
//   ntb_symm_barrier          cross-rank barrier on per-rank flag words (release store to every peer, acquire spin on
//                             the local words); every spin is bounded and reports through a status word.
//   ntb_dp_reduce_scatter     rank r pulls its shard of the fp32 gradient buffer from all peers with plain peer loads,
//                             sums in a fixed rank order (bitwise identical on every run), scales (1/dp), writes the
//                             result into its own buffer in place, and emits the partial sums of squares of the
//                             reduced shard (the gradient-norm contribution), optionally pushing the reduced values
//                             back to every peer (= all-reduce, for un-sharded optimizers).
//   ntb_dp_adamw_allgather    AdamW on the fp32 master shard with the clip coefficient read on the device, then the bf16
//                             value of every updated weight is stored straight into the parameter buffer of ALL ranks
//                             (the all-gather), 16 bytes per store.
//
// Peer loads use ld.relaxed.sys so no stale line can be served from a non-coherent cache; ordering between ranks comes
// from the barrier (release/acquire at system scope).  No multimem, no TMA: the barrier is what makes the data visible.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace {

constexpr int MAX_RANKS = 16;
constexpr int COMM_THREADS = 256;

struct PeerPtrs {
  void* p[MAX_RANKS];
};

__device__ __forceinline__ float4 ld_sys_f4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_sys_u32(uint32_t* p, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// flags[r] points at rank r's flag array (world words).  Rank `me` writes `epoch` into slot `me` of every rank, then
// waits until all its own slots reached `epoch`.  Epochs only grow, so slots never need resetting.
__global__ void symm_barrier_kernel(PeerPtrs flags, int me, int world, uint32_t epoch, unsigned long long limit_ns, int* status) {
  const int t = threadIdx.x;
  if (t >= world) return;
  __threadfence_system();
  st_sys_u32(reinterpret_cast<uint32_t*>(flags.p[t]) + me, epoch);
  const uint32_t* mine = reinterpret_cast<const uint32_t*>(flags.p[me]) + t;
  const uint64_t t0 = ptx::globaltimer();
  while (true) {
    const uint32_t v = ld_acquire_sys_u32(mine);
    if (static_cast<int32_t>(v - epoch) >= 0) break;
    if (ptx::globaltimer() - t0 > limit_ns) {
      if (status) atomicExch(status, NTB_ERR_TIMEOUT);
      break;
    }
    __nanosleep(200);
  }
  __threadfence_system();
}

// grads.p[r]: base of rank r's flat fp32 gradient buffer.  Range [start, start+n) is this rank's shard (n % 4 == 0).
// Each thread keeps U x world 16-byte loads in flight (U chosen by the host so that U * world ~ 8): peer loads cross NVLink
// with a few microseconds of latency, so the bytes in flight per SM, not the instruction rate, set the bandwidth.
template <int U, int WMAX>
__global__ void __launch_bounds__(COMM_THREADS) dp_reduce_scatter_kernel(PeerPtrs grads, int me, int world, int64_t start, int64_t n, float scale,
                                                                         int broadcast, float* __restrict__ sumsq_partial) {
  __shared__ float scratch[32];
  float* own = reinterpret_cast<float*>(grads.p[me]) + start;
  float sq = 0.f;
  const int64_t stride = (int64_t)gridDim.x * COMM_THREADS * 4;
  for (int64_t i0 = ((int64_t)blockIdx.x * COMM_THREADS + threadIdx.x) * 4; i0 < n; i0 += stride * U) {
    float4 vals[U][WMAX];
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int64_t i = i0 + u * stride;
#pragma unroll
      for (int r = 0; r < WMAX; r++)
        if (r < world && i < n) vals[u][r] = (r == me) ? *reinterpret_cast<const float4*>(own + i) : ld_sys_f4(reinterpret_cast<const float*>(grads.p[r]) + start + i);
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int64_t i = i0 + u * stride;
      if (i >= n) break;
      // fixed order 0..world-1 keeps the sum deterministic
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int r = 0; r < WMAX; r++)
        if (r < world) { acc.x += vals[u][r].x; acc.y += vals[u][r].y; acc.z += vals[u][r].z; acc.w += vals[u][r].w; }
      acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
      *reinterpret_cast<float4*>(own + i) = acc;
      if (broadcast) {
        for (int k = 1; k < world; k++) {
          const int r = (me + k) % world;  // staggered so ranks do not all hit the same peer at once
          *reinterpret_cast<float4*>(reinterpret_cast<float*>(grads.p[r]) + start + i) = acc;
        }
      }
      sq += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
    }
  }
  sq = block_sum(sq, scratch);
  if (threadIdx.x == 0) sumsq_partial[blockIdx.x] = sq;
}

__global__ void sum_partials_kernel(const float* __restrict__ partial, int nparts, float* __restrict__ out) {
  __shared__ float scratch[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) s += partial[i];
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) out[0] = s;
}

// p/m/v: this rank's flat fp32 master / state shards (n elements).  g: reduced fp32 gradient shard.  params.p[r]: base
// of rank r's flat bf16 parameter buffer; element `start + i` of every rank receives the new value.
__global__ void __launch_bounds__(COMM_THREADS) dp_adamw_allgather_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                                                                          float* __restrict__ v, PeerPtrs params, int me, int world, int64_t start, int64_t n,
                                                                          const int64_t* __restrict__ seg_end, const float* __restrict__ seg_lr,
                                                                          const float* __restrict__ seg_wd, int nseg, float beta1, float beta2, float eps,
                                                                          float inv_bc1, float inv_sqrt_bc2, const float* __restrict__ grad_scale) {
  const float gs = grad_scale ? *grad_scale : 1.f;
  const int64_t stride = (int64_t)gridDim.x * COMM_THREADS * 8;
  for (int64_t base = ((int64_t)blockIdx.x * COMM_THREADS + threadIdx.x) * 8; base < n; base += stride) {
    int lo = 0, hi = nseg - 1;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (seg_end[mid] > base) hi = mid; else lo = mid + 1;
    }
    const float lr = seg_lr[lo], wd = seg_wd[lo];
    float pv[8], gv[8], mv[8], vv[8];
    *reinterpret_cast<float4*>(pv) = *reinterpret_cast<const float4*>(p + base);
    *reinterpret_cast<float4*>(pv + 4) = *reinterpret_cast<const float4*>(p + base + 4);
    *reinterpret_cast<float4*>(gv) = *reinterpret_cast<const float4*>(g + base);
    *reinterpret_cast<float4*>(gv + 4) = *reinterpret_cast<const float4*>(g + base + 4);
    *reinterpret_cast<float4*>(mv) = *reinterpret_cast<const float4*>(m + base);
    *reinterpret_cast<float4*>(mv + 4) = *reinterpret_cast<const float4*>(m + base + 4);
    *reinterpret_cast<float4*>(vv) = *reinterpret_cast<const float4*>(v + base);
    *reinterpret_cast<float4*>(vv + 4) = *reinterpret_cast<const float4*>(v + base + 4);
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const float gi = gv[i] * gs;
      float pi = pv[i] * (1.f - lr * wd);
      mv[i] = beta1 * mv[i] + (1.f - beta1) * gi;
      vv[i] = beta2 * vv[i] + (1.f - beta2) * gi * gi;
      pi -= lr * inv_bc1 * mv[i] / (sqrtf(vv[i]) * inv_sqrt_bc2 + eps);
      pv[i] = pi;
    }
    *reinterpret_cast<float4*>(p + base) = *reinterpret_cast<float4*>(pv);
    *reinterpret_cast<float4*>(p + base + 4) = *reinterpret_cast<float4*>(pv + 4);
    *reinterpret_cast<float4*>(m + base) = *reinterpret_cast<float4*>(mv);
    *reinterpret_cast<float4*>(m + base + 4) = *reinterpret_cast<float4*>(mv + 4);
    *reinterpret_cast<float4*>(v + base) = *reinterpret_cast<float4*>(vv);
    *reinterpret_cast<float4*>(v + base + 4) = *reinterpret_cast<float4*>(vv + 4);
    uint4 pk;
    __nv_bfloat162 h0 = __floats2bfloat162_rn(pv[0], pv[1]), h1 = __floats2bfloat162_rn(pv[2], pv[3]);
    __nv_bfloat162 h2 = __floats2bfloat162_rn(pv[4], pv[5]), h3 = __floats2bfloat162_rn(pv[6], pv[7]);
    pk.x = *reinterpret_cast<uint32_t*>(&h0); pk.y = *reinterpret_cast<uint32_t*>(&h1);
    pk.z = *reinterpret_cast<uint32_t*>(&h2); pk.w = *reinterpret_cast<uint32_t*>(&h3);
    for (int k = 0; k < world; k++) {
      const int r = (me + k) % world;
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(params.p[r]) + start + base) = pk;
    }
  }
}

bool fill_peers(PeerPtrs& out, const uint64_t* host_ptrs, int world) {
  if (world < 1 || world > MAX_RANKS) return false;
  for (int r = 0; r < MAX_RANKS; r++) out.p[r] = r < world ? reinterpret_cast<void*>(host_ptrs[r]) : nullptr;
  return true;
}

}  // namespace

NTB_EXPORT int ntb_comm_max_ranks() { return MAX_RANKS; }

// flag_ptrs: host array of `world` device pointers (rank r's flag words, each array holding >= world uint32).
NTB_EXPORT int ntb_symm_barrier(const uint64_t* flag_ptrs, int me, int world, uint32_t epoch, unsigned long long limit_ns, int* status, cudaStream_t stream) {
  PeerPtrs f;
  if (!fill_peers(f, flag_ptrs, world) || me < 0 || me >= world) return NTB_ERR_ARG;
  symm_barrier_kernel<<<1, 32, 0, stream>>>(f, me, world, epoch, limit_ns, status);
  return ntb_check_launch();
}

namespace {
// Spins (bounded) until the first `world` local flag words reached `epoch`.
__global__ void symm_wait_kernel(const uint32_t* flags, int world, uint32_t epoch, unsigned long long limit_ns, int* status) {
  const int t = threadIdx.x;
  if (t >= world) return;
  const uint64_t t0 = ptx::globaltimer();
  while (true) {
    if (static_cast<int32_t>(ld_acquire_sys_u32(flags + t) - epoch) >= 0) break;
    if (ptx::globaltimer() - t0 > limit_ns) {
      if (status) atomicExch(status, NTB_ERR_TIMEOUT);
      break;
    }
    __nanosleep(200);
  }
  __threadfence_system();
}
}  // namespace

NTB_EXPORT int ntb_symm_wait(const uint32_t* flags, int world, uint32_t epoch, unsigned long long limit_ns, int* status, cudaStream_t stream) {
  if (world < 1 || world > 32) return NTB_ERR_ARG;
  symm_wait_kernel<<<1, 32, 0, stream>>>(flags, world, epoch, limit_ns, status);
  return ntb_check_launch();
}

NTB_EXPORT int ntb_dp_num_partials() { return 148 * 4; }

// sumsq_partial: fp32 [ntb_dp_num_partials()]; sumsq_out: fp32 [1] receives the sum of squares of the reduced shard.
NTB_EXPORT int ntb_dp_reduce_scatter(const uint64_t* grad_ptrs, int me, int world, int64_t start, int64_t n, float scale, int broadcast,
                                     float* sumsq_partial, float* sumsq_out, cudaStream_t stream) {
  PeerPtrs g;
  if (!fill_peers(g, grad_ptrs, world) || n <= 0 || n % 4 || start % 4) return NTB_ERR_ARG;
  const int blocks = ntb_dp_num_partials();
  if (world <= 2) dp_reduce_scatter_kernel<4, 2><<<blocks, COMM_THREADS, 0, stream>>>(g, me, world, start, n, scale, broadcast, sumsq_partial);
  else if (world <= 4) dp_reduce_scatter_kernel<2, 4><<<blocks, COMM_THREADS, 0, stream>>>(g, me, world, start, n, scale, broadcast, sumsq_partial);
  else if (world <= 8) dp_reduce_scatter_kernel<2, 8><<<blocks, COMM_THREADS, 0, stream>>>(g, me, world, start, n, scale, broadcast, sumsq_partial);
  else dp_reduce_scatter_kernel<1, MAX_RANKS><<<blocks, COMM_THREADS, 0, stream>>>(g, me, world, start, n, scale, broadcast, sumsq_partial);
  sum_partials_kernel<<<1, 256, 0, stream>>>(sumsq_partial, blocks, sumsq_out);
  return ntb_check_launch();
}

namespace {
__global__ void add_partials_kernel(const float* __restrict__ partial, int nparts, float* __restrict__ out) {
  __shared__ float scratch[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) s += partial[i];
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) out[0] += s;
}
}  // namespace

// The same reduction over one sub-range [start, start + n) of this rank's shard, for exchanges that are issued piece by piece
// while the backward pass still runs: `blocks` (1 .. ntb_dp_num_partials()) bounds the SMs the transfer may occupy next to the
// compute kernels, and the sum of squares is ADDED to sumsq_accum[0] (calls on one stream are ordered, so no atomics are needed).
NTB_EXPORT int ntb_dp_reduce_scatter_range(const uint64_t* grad_ptrs, int me, int world, int64_t start, int64_t n, float scale, int broadcast,
                                           float* sumsq_partial, float* sumsq_accum, int blocks, cudaStream_t stream) {
  PeerPtrs g;
  if (!fill_peers(g, grad_ptrs, world) || n <= 0 || n % 4 || start % 4 || blocks < 1 || blocks > ntb_dp_num_partials()) return NTB_ERR_ARG;
  if (world <= 2) dp_reduce_scatter_kernel<4, 2><<<blocks, COMM_THREADS, 0, stream>>>(g, me, world, start, n, scale, broadcast, sumsq_partial);
  else if (world <= 4) dp_reduce_scatter_kernel<2, 4><<<blocks, COMM_THREADS, 0, stream>>>(g, me, world, start, n, scale, broadcast, sumsq_partial);
  else if (world <= 8) dp_reduce_scatter_kernel<2, 8><<<blocks, COMM_THREADS, 0, stream>>>(g, me, world, start, n, scale, broadcast, sumsq_partial);
  else dp_reduce_scatter_kernel<1, MAX_RANKS><<<blocks, COMM_THREADS, 0, stream>>>(g, me, world, start, n, scale, broadcast, sumsq_partial);
  add_partials_kernel<<<1, 256, 0, stream>>>(sumsq_partial, blocks, sumsq_accum);
  return ntb_check_launch();
}

NTB_EXPORT int ntb_dp_adamw_allgather(float* p, const float* g, float* m, float* v, const uint64_t* param_ptrs, int me, int world, int64_t start, int64_t n,
                                      const int64_t* seg_end, const float* seg_lr, const float* seg_wd, int nseg, float beta1, float beta2, float eps,
                                      float bias_correction1, float bias_correction2, const float* grad_scale, cudaStream_t stream) {
  PeerPtrs pp;
  if (!fill_peers(pp, param_ptrs, world) || n <= 0 || n % 8 || start % 8 || nseg <= 0) return NTB_ERR_ARG;
  int64_t blocks = (n / 8 + COMM_THREADS - 1) / COMM_THREADS;
  if (blocks > 148 * 8) blocks = 148 * 8;
  dp_adamw_allgather_kernel<<<(unsigned)blocks, COMM_THREADS, 0, stream>>>(p, g, m, v, pp, me, world, start, n, seg_end, seg_lr, seg_wd, nseg, beta1, beta2, eps,
                                                                          1.f / bias_correction1, rsqrtf(bias_correction2), grad_scale);
  return ntb_check_launch();
}
