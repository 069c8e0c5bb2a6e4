// Mixture-of-experts token dispatch / combine over NVLink peer memory (sm_100a), with no host synchronisation.
//
// Every rank of the expert-parallel group owns E / W consecutive experts.  Tokens travel as rows of a receive buffer in the
// owner's memory laid out for the grouped GEMM: expert j of the owner holds rows [seg_off[j], seg_off[j+1]), every offset a
// multiple of 128, rows ordered by (source rank, token, slot), padding rows zero.  One layer's forward is
//
//   plan      one block: publishes this rank's per-expert counts in every peer's table (peer stores + release flag), waits
//             (bounded) for the peers' counts, then derives the padded offsets of EVERY owner, this rank's first row
//             inside each destination expert, the row-block -> expert table and the number of used row blocks.
//   rank      one warp per expert scans the top-k ids in token order (ballot + popcount), giving each (token, slot) its
//             destination row: stable, so results do not depend on scheduling.
//   dispatch  one block per token: reads the row once and stores it into the k owners' receive buffers (16-byte peer
//             stores); optionally sends the routing probability of each copy along (backward needs it at the owner).
//   zero_pad  the owner zeroes the padding rows of its receive buffer.
//   [barrier] (ntb_symm_barrier)
//   grouped GEMMs on the owner (gemm_tcgen05.cu), results in a buffer the peers can read
//   [barrier]
//   combine   one block per token: pulls its k result rows from the owners (ld.relaxed.sys), weights them with the routing
//             probabilities in fp32 and writes the bf16 output row; can also gather one fp32 scalar per copy.
//
// Backward reuses the same plan: dispatch(dOut) with the probabilities, `scale_dot` at the owner (dY_row *= p and
// dP_row = <dOut_row, Y_row>), grouped dgrad / wgrad, then combine with unit weights (dX) gathering dP.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace {

constexpr int MOE_MAX_RANKS = 8;
constexpr int MOE_MAX_EXPERTS = 256;
constexpr int MOE_MAX_K = 16;

struct MoePeers {
  void* p[MOE_MAX_RANKS];
};

__device__ __forceinline__ int ld_sys_i32(const int* p) {
  int v;
  asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float ld_sys_f32(const float* p) {
  float v;
  asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_sys_u4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// counts_all tables: [2 (epoch parity)][W][E] int32 on every rank.
__global__ void moe_plan_kernel(const int* __restrict__ counts, MoePeers tables, MoePeers flags, int me, int W, int E, uint32_t epoch,
                                unsigned long long limit_ns, int* status, int* __restrict__ seg_off, int* __restrict__ cnt_tot, int* __restrict__ dest_base,
                                int* __restrict__ tile_expert, int* __restrict__ num_m_tiles, int cap_tiles) {
  __shared__ int tot[MOE_MAX_EXPERTS];
  __shared__ int before[MOE_MAX_EXPERTS];
  __shared__ int owner_off[MOE_MAX_EXPERTS];
  __shared__ int bad;
  const int t = threadIdx.x;
  const int El = E / W;
  const int parity = epoch & 1;
  if (t == 0) bad = 0;
  if (t < E) {
    const int c = counts[t];
    for (int r = 0; r < W; r++) reinterpret_cast<int*>(tables.p[r])[(parity * W + me) * E + t] = c;
  }
  __threadfence_system();
  __syncthreads();
  if (t < W) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(reinterpret_cast<uint32_t*>(flags.p[t]) + me), "r"(epoch) : "memory");
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(flags.p[me]) + t;
    const uint64_t t0 = ptx::globaltimer();
    while (true) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if (static_cast<int32_t>(v - epoch) >= 0) break;
      if (ptx::globaltimer() - t0 > limit_ns) { bad = 1; break; }
      __nanosleep(200);
    }
  }
  __syncthreads();
  if (bad) {
    if (t == 0) {
      if (status) atomicExch(status, NTB_ERR_TIMEOUT);
      *num_m_tiles = 0;  // the grouped GEMMs then skip every tile
    }
    return;
  }
  if (t < E) {
    const int* mine = reinterpret_cast<const int*>(tables.p[me]) + parity * W * E;
    int s = 0, b = 0;
    for (int r = 0; r < W; r++) {
      const int c = ld_sys_i32(mine + r * E + t);
      if (r < me) b += c;
      s += c;
    }
    tot[t] = s;
    before[t] = b;
  }
  __syncthreads();
  if (t < W) {
    int off = 0;
    for (int j = 0; j < El; j++) {
      const int e = t * El + j;
      owner_off[e] = off;
      if (t == me) {
        seg_off[j] = off;
        cnt_tot[j] = tot[e];
      }
      off += (tot[e] + 127) & ~127;
    }
    if (t == me) {
      seg_off[El] = off;
      int tiles = off >> 7;
      if (tiles > cap_tiles) {  // cannot happen when the buffer is sized for the worst case; never run past it
        tiles = 0;
        if (status) atomicExch(status, NTB_ERR_ARG);
      }
      *num_m_tiles = tiles;
    }
  }
  __syncthreads();
  if (t < E) dest_base[t] = owner_off[t] + before[t];
  if (t < El) {
    const int lo = owner_off[me * El + t] >> 7;
    const int hi = lo + ((tot[me * El + t] + 127) >> 7);
    for (int i = lo; i < hi && i < cap_tiles; i++) tile_expert[i] = t;
  }
}

// One warp per expert: destination row of every (token, slot) routed to it, in token order.
__global__ void moe_rank_kernel(const int* __restrict__ top_i, int n, const int* __restrict__ dest_base, int E, int* __restrict__ row_of) {
  const int e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (e >= E) return;
  int running = dest_base[e];
  const unsigned lt = (1u << lane) - 1u;
  for (int i0 = 0; i0 < n; i0 += 128) {
    int v[4];
#pragma unroll
    for (int u = 0; u < 4; u++) {
      const int i = i0 + u * 32 + lane;
      v[u] = i < n ? __ldg(top_i + i) : -1;
    }
#pragma unroll
    for (int u = 0; u < 4; u++) {
      const unsigned m = __ballot_sync(0xffffffffu, v[u] == e);
      if (v[u] == e) row_of[i0 + u * 32 + lane] = running + __popc(m & lt);
      running += __popc(m);
    }
  }
}

__global__ void moe_dispatch_kernel(const uint4* __restrict__ x, const int* __restrict__ top_i, const int* __restrict__ row_of, const float* __restrict__ top_p,
                                    MoePeers recv, MoePeers p_recv, int T, int h8, int k, int El) {
  __shared__ int s_owner[MOE_MAX_K];
  __shared__ int s_row[MOE_MAX_K];
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    __syncthreads();
    if (threadIdx.x < k) {
      const int e = top_i[t * k + threadIdx.x];
      const int row = row_of[t * k + threadIdx.x];
      s_owner[threadIdx.x] = e / El;
      s_row[threadIdx.x] = row;
      if (top_p != nullptr) reinterpret_cast<float*>(p_recv.p[e / El])[row] = top_p[t * k + threadIdx.x];
    }
    __syncthreads();
    for (int v = threadIdx.x; v < h8; v += blockDim.x) {
      const uint4 val = x[static_cast<long long>(t) * h8 + v];
      for (int j = 0; j < k; j++) reinterpret_cast<uint4*>(recv.p[s_owner[j]])[static_cast<long long>(s_row[j]) * h8 + v] = val;
    }
  }
}

__global__ void moe_zero_pad_kernel(uint4* __restrict__ buf, const int* __restrict__ seg_off, const int* __restrict__ cnt_tot, int h8) {
  const int j = blockIdx.x;
  const int lo = seg_off[j] + cnt_tot[j], hi = seg_off[j + 1];
  for (int r = lo + blockIdx.y; r < hi; r += gridDim.y)
    for (int v = threadIdx.x; v < h8; v += blockDim.x) buf[static_cast<long long>(r) * h8 + v] = make_uint4(0, 0, 0, 0);
}

__global__ void moe_combine_kernel(MoePeers ybuf, const int* __restrict__ top_i, const int* __restrict__ row_of, const float* __restrict__ weights,
                                   uint4* __restrict__ out, MoePeers scalar_src, float* __restrict__ scalar_out, int T, int h8, int k, int El) {
  __shared__ int s_owner[MOE_MAX_K];
  __shared__ int s_row[MOE_MAX_K];
  __shared__ float s_w[MOE_MAX_K];
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    __syncthreads();
    if (threadIdx.x < k) {
      const int e = top_i[t * k + threadIdx.x];
      const int row = row_of[t * k + threadIdx.x];
      s_owner[threadIdx.x] = e / El;
      s_row[threadIdx.x] = row;
      s_w[threadIdx.x] = weights != nullptr ? weights[t * k + threadIdx.x] : 1.0f;
      if (scalar_out != nullptr) scalar_out[t * k + threadIdx.x] = ld_sys_f32(reinterpret_cast<const float*>(scalar_src.p[e / El]) + row);
    }
    __syncthreads();
    for (int v = threadIdx.x; v < h8; v += blockDim.x) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int j = 0; j < k; j++) {
        const uint4 raw = ld_sys_u4(reinterpret_cast<const uint4*>(ybuf.p[s_owner[j]]) + static_cast<long long>(s_row[j]) * h8 + v);
        const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&raw);
        const float w = s_w[j];
#pragma unroll
        for (int q = 0; q < 4; q++) {
          const float2 f = __bfloat1622float2(hh[q]);
          acc[2 * q] += w * f.x;
          acc[2 * q + 1] += w * f.y;
        }
      }
      uint4 o;
      __nv_bfloat162 h0 = __floats2bfloat162_rn(acc[0], acc[1]), h1 = __floats2bfloat162_rn(acc[2], acc[3]);
      __nv_bfloat162 h2 = __floats2bfloat162_rn(acc[4], acc[5]), h3 = __floats2bfloat162_rn(acc[6], acc[7]);
      o.x = *reinterpret_cast<uint32_t*>(&h0); o.y = *reinterpret_cast<uint32_t*>(&h1);
      o.z = *reinterpret_cast<uint32_t*>(&h2); o.w = *reinterpret_cast<uint32_t*>(&h3);
      out[static_cast<long long>(t) * h8 + v] = o;
    }
  }
}

// Owner side of the backward: for every used row r, dp_rows[r] = <dy[r], y[r]> and dy[r] *= p_recv[r]; padding rows become zero.
__global__ void moe_scale_dot_kernel(uint4* __restrict__ dy, const uint4* __restrict__ y, const float* __restrict__ p_recv, float* __restrict__ dp_rows,
                                     const int* __restrict__ num_m_tiles, const int* __restrict__ tile_expert, const int* __restrict__ seg_off,
                                     const int* __restrict__ cnt_tot, int h8) {
  __shared__ float red[32];
  const int rows = *num_m_tiles * 128;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const int e = tile_expert[r >> 7];
    const bool valid = r - seg_off[e] < cnt_tot[e];
    const float p = valid ? p_recv[r] : 0.f;
    float dot = 0.f;
    for (int v = threadIdx.x; v < h8; v += blockDim.x) {
      const long long idx = static_cast<long long>(r) * h8 + v;
      if (!valid) {
        dy[idx] = make_uint4(0, 0, 0, 0);
        continue;
      }
      uint4 a = dy[idx];
      const uint4 b = y[idx];
      __nv_bfloat162* ha = reinterpret_cast<__nv_bfloat162*>(&a);
      const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
      for (int q = 0; q < 4; q++) {
        const float2 fa = __bfloat1622float2(ha[q]);
        const float2 fb = __bfloat1622float2(hb[q]);
        dot += fa.x * fb.x + fa.y * fb.y;
        ha[q] = __floats2bfloat162_rn(fa.x * p, fa.y * p);
      }
      dy[idx] = a;
    }
    // block reduction of `dot`
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = dot;
    __syncthreads();
    if (threadIdx.x == 0) {
      float s = 0.f;
      for (int w = 0; w < (blockDim.x >> 5); w++) s += red[w];
      dp_rows[r] = valid ? s : 0.f;
    }
  }
}

bool fill(MoePeers& dst, const uint64_t* ptrs, int W) {
  if (W < 1 || W > MOE_MAX_RANKS) return false;
  for (int r = 0; r < MOE_MAX_RANKS; r++) dst.p[r] = (ptrs != nullptr && r < W) ? reinterpret_cast<void*>(ptrs[r]) : nullptr;
  return true;
}

}  // namespace

NTB_EXPORT int ntb_moe_max_experts() { return MOE_MAX_EXPERTS; }

// counts [E] int32 (this rank's assignments per global expert).  table_ptrs / flag_ptrs: per-rank base of the [2][W][E]
// int32 count tables and of the flag words (>= W uint32).  Outputs are local device arrays: seg_off [E/W + 1],
// cnt_tot [E/W], dest_base [E], tile_expert [cap_tiles], num_m_tiles [1].
NTB_EXPORT int ntb_moe_plan(const int* counts, const uint64_t* table_ptrs, const uint64_t* flag_ptrs, int me, int W, int E, uint32_t epoch,
                            unsigned long long limit_ns, int* status, int* seg_off, int* cnt_tot, int* dest_base, int* tile_expert, int* num_m_tiles,
                            int cap_tiles, cudaStream_t stream) {
  MoePeers tables, flags;
  if (!fill(tables, table_ptrs, W) || !fill(flags, flag_ptrs, W) || E <= 0 || E > MOE_MAX_EXPERTS || E % W || me < 0 || me >= W || cap_tiles <= 0) return NTB_ERR_ARG;
  moe_plan_kernel<<<1, 256, 0, stream>>>(counts, tables, flags, me, W, E, epoch, limit_ns, status, seg_off, cnt_tot, dest_base, tile_expert, num_m_tiles, cap_tiles);
  return ntb_check_launch();
}

// row_of[n] for the n = T * k (token, slot) pairs.
NTB_EXPORT int ntb_moe_rank(const int* top_i, int n, const int* dest_base, int E, int* row_of, cudaStream_t stream) {
  if (n <= 0 || E <= 0 || E > MOE_MAX_EXPERTS) return NTB_ERR_ARG;
  moe_rank_kernel<<<(E + 3) / 4, 128, 0, stream>>>(top_i, n, dest_base, E, row_of);
  return ntb_check_launch();
}

// x [T, h] bf16 -> rows of the owners' receive buffers; top_p (nullable) -> the owners' p_recv.
NTB_EXPORT int ntb_moe_dispatch(const void* x, const int* top_i, const int* row_of, const float* top_p, const uint64_t* recv_ptrs, const uint64_t* p_recv_ptrs,
                                int T, int h, int k, int W, int E, cudaStream_t stream) {
  MoePeers recv, precv;
  if (!fill(recv, recv_ptrs, W) || !fill(precv, p_recv_ptrs, W) || T <= 0 || h % 8 || k < 1 || k > MOE_MAX_K || E % W) return NTB_ERR_ARG;
  if (top_p != nullptr && p_recv_ptrs == nullptr) return NTB_ERR_ARG;
  const int grid = T < 148 * 8 ? T : 148 * 8;
  moe_dispatch_kernel<<<grid, 128, 0, stream>>>(reinterpret_cast<const uint4*>(x), top_i, row_of, top_p, recv, precv, T, h / 8, k, E / W);
  return ntb_check_launch();
}

NTB_EXPORT int ntb_moe_zero_pad(void* buf, const int* seg_off, const int* cnt_tot, int h, int El, cudaStream_t stream) {
  if (El <= 0 || h % 8) return NTB_ERR_ARG;
  moe_zero_pad_kernel<<<dim3(El, 16), 128, 0, stream>>>(reinterpret_cast<uint4*>(buf), seg_off, cnt_tot, h / 8);
  return ntb_check_launch();
}

// out[t] = sum_j w[t, j] * ybuf[owner(t, j)][row_of[t, j]] (w null = 1); optionally scalar_out[t, j] = scalar_src[owner][row].
NTB_EXPORT int ntb_moe_combine(const uint64_t* y_ptrs, const int* top_i, const int* row_of, const float* weights, void* out, const uint64_t* scalar_ptrs,
                               float* scalar_out, int T, int h, int k, int W, int E, cudaStream_t stream) {
  MoePeers y, sc;
  if (!fill(y, y_ptrs, W) || !fill(sc, scalar_ptrs, W) || T <= 0 || h % 8 || k < 1 || k > MOE_MAX_K || E % W) return NTB_ERR_ARG;
  if (scalar_out != nullptr && scalar_ptrs == nullptr) return NTB_ERR_ARG;
  const int grid = T < 148 * 8 ? T : 148 * 8;
  moe_combine_kernel<<<grid, 128, 0, stream>>>(y, top_i, row_of, weights, reinterpret_cast<uint4*>(out), sc, scalar_out, T, h / 8, k, E / W);
  return ntb_check_launch();
}

NTB_EXPORT int ntb_moe_scale_dot(void* dy, const void* y, const float* p_recv, float* dp_rows, const int* num_m_tiles, const int* tile_expert, const int* seg_off,
                                 const int* cnt_tot, int h, int cap_rows, cudaStream_t stream) {
  if (h % 8 || cap_rows <= 0) return NTB_ERR_ARG;
  const int grid = cap_rows < 148 * 8 ? cap_rows : 148 * 8;
  moe_scale_dot_kernel<<<grid, 128, 0, stream>>>(reinterpret_cast<uint4*>(dy), reinterpret_cast<const uint4*>(y), p_recv, dp_rows, num_m_tiles, tile_expert, seg_off,
                                                 cnt_tot, h / 8);
  return ntb_check_launch();
}
