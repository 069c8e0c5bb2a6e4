// Flash attention backward on tcgen05 / TMEM (sm_100a): head dim 128, bf16, causal or full, GQA, packed sequences.
//
// One CTA owns a tile of 128 keys of one KV head and walks every query head of its group and every 64-query tile that can
// see those keys.  All five products are issued "transposed" so that M = 128 everywhere and the key index is the TMEM
// lane:
//     S^T  = K Q^T        (128 keys x 64 queries)          dP^T = V dO^T
//     P^T  = exp2(S^T c - lse)     dS^T = P^T (dP^T - delta) * scale        (thread = key row, registers -> bf16 smem)
//     dV  += P^T dO       dK += dS^T Q       (fp32 accumulators in TMEM for the whole CTA lifetime)
//     dQ^T = K^T dS^T     (128 head-dim lanes x 64 queries) -> red.global.add.f32 into an fp32 dQ buffer; a warp's 32
//                          lanes hit 32 consecutive floats, so the reductions are coalesced.
// Warp roles: warp 0 TMA producer (K, V once; Q / dO double buffered), warp 1 MMA issuer (the scores of step n + 1 are issued
// before the three products of step n, so the softmax of the next step overlaps them; dQ^T in tensor memory and P^T / dS^T in
// shared memory are double buffered), warps 2-9 softmax (two warpgroups, 32 query columns each) + final dK / dV write-out,
// warps 10-13 dQ^T read-out.  A small pre-pass computes delta = rowsum(dO * O); a post-pass casts dQ to bf16.
// All waits are bounded (see sm100_ptx.cuh).
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace {

constexpr int HD = 128;
constexpr int BK = 128;  // keys per CTA
constexpr int BQ = 64;   // queries per step
constexpr int KV_TILE_BYTES = BK * HD * 2;   // 32 KiB (two [128][64] panels)
constexpr int KV_PANEL = BK * 64 * 2;        // 16 KiB
constexpr int Q_TILE_BYTES = BQ * HD * 2;    // 16 KiB (two [64][64] panels)
constexpr int Q_PANEL = BQ * 64 * 2;         // 8 KiB
constexpr int PT_BYTES = BK * BQ * 2;        // 16 KiB: [128 key rows][64 queries]
constexpr int BWD_THREADS = 448;  // TMA warp, MMA warp, two softmax warpgroups, one dQ read-out warpgroup
constexpr int QDO_STAGES = 3;                // Q / dO tiles in flight: products of step n, scores of step n + 1, prefetch
constexpr int BWD_HEAD_BYTES = 256 + 2048;   // barriers, then per-warp row statistics, in front of the 1024-byte aligned tiles
constexpr int BWD_TILE_BYTES = 2 * KV_TILE_BYTES + 2 * QDO_STAGES * Q_TILE_BYTES + 4 * PT_BYTES;  // 224 KiB
// With a 1024-byte aligned dynamic shared memory base this is exactly the 227 KiB a CTA may have; the kernel checks that the
// tiles fit behind the aligned offset and gives up with an error status otherwise.
constexpr int BWD_SMEM = 3072 + BWD_TILE_BYTES;

struct BwdParams {
  int num_heads, num_kv_heads, causal, window;
  float scale, scale_log2;
  const int* cu_q;
  const int* cu_k;
  const float* lse;    // [Hq, total_q]
  const float* delta;  // [Hq, total_q]
  float* dq_acc;       // [total_q, Hq, 128] fp32, zero-initialised
  __nv_bfloat16* dk;   // strided [total_k, Hkv, 128]
  __nv_bfloat16* dv;
  int64_t dk_stride_t;
  int total_q;
  int* status;
  int cp, cp_me, cp_chunk;  // context parallel: group size (0 = off), this rank, tokens per chunk
  // Split mode: one CTA per (key tile, QUERY head) instead of per (key tile, kv head).  The query heads of a group then add their
  // dK / dV into fp32 accumulators [total_k, Hkv, 128] (zero-filled by the caller, cast by a post-pass).  Used when key tiles x kv
  // heads would not fill the GPU (few kv heads per GPU under tensor parallelism, short sequences).
  int split;
  float* dk_split;
  float* dv_split;
};

constexpr int CP_MAX = 8;
struct CpBwd {
  CUtensorMap k[CP_MAX];
  CUtensorMap v[CP_MAX];
  float* dk_acc[CP_MAX];  // per owner: fp32 [batch * 2 * chunk, Hkv, 128]
  float* dv_acc[CP_MAX];
};

__global__ void delta_kernel(const __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ dout, float* __restrict__ delta, int total_q, int heads) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= total_q * heads) return;
  const int t = warp / heads, h = warp % heads;
  const __nv_bfloat16* o = out + (static_cast<int64_t>(t) * heads + h) * HD + lane * 4;
  const __nv_bfloat16* d = dout + (static_cast<int64_t>(t) * heads + h) * HD + lane * 4;
  const uint2 a = *reinterpret_cast<const uint2*>(o), b = *reinterpret_cast<const uint2*>(d);
  const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&b);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 2; i++) {
    const float2 x = __bfloat1622float2(ah[i]), y = __bfloat1622float2(bh[i]);
    s += x.x * y.x + x.y * y.y;
  }
  s = warp_sum(s);
  if (lane == 0) delta[static_cast<int64_t>(h) * total_q + t] = s;
}

__global__ void cast_dq_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, int64_t rows, int heads, int64_t dq_stride_t) {
  const int64_t idx = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
  if (idx >= rows * heads * HD) return;
  const int64_t t = idx / (heads * HD);
  const int64_t rem = idx % (heads * HD);
  float f[8];
  *reinterpret_cast<float4*>(f) = *reinterpret_cast<const float4*>(acc + idx);
  *reinterpret_cast<float4*>(f + 4) = *reinterpret_cast<const float4*>(acc + idx + 4);
  Vec8<__nv_bfloat16> v;
  v.from_float(f);
  v.store(dq + t * dq_stride_t + rem);
}

__device__ __forceinline__ void red_add_f32(float* p, float v) { asm volatile("red.global.add.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory"); }
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// packed fp32 pairs: one issue slot for two elements
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}

__global__ void __maxnreg__(128)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const BwdParams p, const __grid_constant__ CpBwd cpb) {
  extern __shared__ uint8_t smem_raw[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw);
  float* s_stats = reinterpret_cast<float*>(smem_raw + 256);  // [8 warps][32 (-lse log2 e) | 32 (delta scale)]
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + BWD_HEAD_BYTES + 1023) & ~uintptr_t(1023));
  if (smem + BWD_TILE_BYTES > smem_raw + BWD_SMEM) {  // uniform for the grid: the base was not 1024-byte aligned
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, NTB_ERR_LAUNCH);
    return;
  }
  uint8_t* sK = smem;
  uint8_t* sV = sK + KV_TILE_BYTES;
  uint8_t* sQ = sV + KV_TILE_BYTES;                   // QDO_STAGES stages
  uint8_t* sdO = sQ + QDO_STAGES * Q_TILE_BYTES;      // QDO_STAGES stages
  uint8_t* sPT = sdO + QDO_STAGES * Q_TILE_BYTES;     // 2 buffers
  uint8_t* sdST = sPT + 2 * PT_BYTES;                 // 2 buffers
  uint64_t* kv_full = bars;          // 1
  uint64_t* qdo_full = bars + 1;     // [QDO_STAGES]
  uint64_t* qdo_empty = bars + 4;    // [QDO_STAGES]
  uint64_t* sdp_full = bars + 7;     // 1
  uint64_t* pds_full = bars + 8;     // 1
  uint64_t* mma_done = bars + 9;     // [2] (dV, dK, dQ^T products of a step finished; steps alternate between the two)
  uint64_t* dq_free = bars + 11;     // [2] (dQ^T buffer read out by the four read-out warps)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Grid: x = (sequence, kv head), y = key tile.  CTAs are handed out x first, so all CTAs of key tile 0 start before any of tile 1:
  // under a causal mask the first key tiles are seen by the most queries, and starting the longest CTAs first keeps the tail of
  // the launch short (with the key tile in x, late CTAs of tile 0 ran alone at the end).
  const int group_all = p.num_heads / p.num_kv_heads;
  const int heads_x = p.split ? p.num_heads : p.num_kv_heads;
  const int b = blockIdx.x / heads_x, hx = blockIdx.x % heads_x;
  const int hk = p.split ? hx / group_all : hx;
  const int h_first = p.split ? hx : hk * group_all;  // first query head this CTA walks
  const bool cpm_on = p.cp > 0;
  const int q_begin = cpm_on ? b * 2 * p.cp_chunk : p.cu_q[b];
  const int q_len = cpm_on ? 2 * p.cp_chunk : p.cu_q[b + 1] - q_begin;
  const int k_begin = cpm_on ? 0 : p.cu_k[b];
  const int k_len = cpm_on ? 2 * p.cp * p.cp_chunk : p.cu_k[b + 1] - k_begin;
  const int k0 = blockIdx.y * BK;  // first key of the tile: local position, or the global one under context parallelism
  if (k0 >= k_len) return;
  const int shift = cpm_on ? 0 : k_len - q_len;
  const int group = p.split ? 1 : group_all;  // query heads this CTA walks
  // Runs of 64-query steps that can see at least one key of this tile: one run normally, up to two (one per local chunk) under
  // context parallelism.  seg_q0 = local position of the run's first query, seg_m0 = its position for the masks.
  int seg_q0[2] = {0, 0}, seg_m0[2] = {0, 0}, seg_n[2] = {0, 0};
  int kv_owner = 0, kv_row = k_begin + k0;
  if (!cpm_on) {
    int qt_begin = 0;
    if (p.causal) qt_begin = max(0, k0 - shift) / BQ;
    int qt_end = (q_len + BQ - 1) / BQ;
    if (p.window > 0) qt_end = min(qt_end, (k0 + BK - 1 - shift + p.window - 1) / BQ + 1);
    seg_q0[0] = seg_m0[0] = qt_begin * BQ;
    seg_n[0] = max(0, qt_end - qt_begin);
  } else {
    const int c = p.cp_chunk;
    for (int half = 0; half < 2; half++) {
      const int chunk = half == 0 ? p.cp_me : 2 * p.cp - 1 - p.cp_me;
      const int first = max(0, k0 - chunk * c) / BQ * BQ;  // first query of the chunk (relative) that sees key k0
      if (first < c) {
        seg_q0[half] = half * c + first;
        seg_m0[half] = chunk * c + first;
        seg_n[half] = (c - first) / BQ;
      }
    }
    const int kchunk = k0 / c;
    kv_owner = kchunk < p.cp ? kchunk : 2 * p.cp - 1 - kchunk;
    kv_row = b * 2 * c + (kchunk < p.cp ? 0 : c) + (k0 - kchunk * c);
  }
  const int tiles_per_head = seg_n[0] + seg_n[1];
  const int n_steps = tiles_per_head * group;
  // step index inside a head -> (local query position, mask position)
  auto step_pos = [&](int i, int& q0, int& m0) {
    if (i < seg_n[0]) { q0 = seg_q0[0] + i * BQ; m0 = seg_m0[0] + i * BQ; }
    else { q0 = seg_q0[1] + (i - seg_n[0]) * BQ; m0 = seg_m0[1] + (i - seg_n[0]) * BQ; }
  };
  const CUtensorMap* map_k = cpm_on ? &cpb.k[kv_owner] : &tmap_k;
  const CUtensorMap* map_v = cpm_on ? &cpb.v[kv_owner] : &tmap_v;

  if (threadIdx.x == 0) {
    ptx::mbar_init(kv_full, 1);
    for (int s = 0; s < QDO_STAGES; s++) {
      ptx::mbar_init(&qdo_full[s], 1);
      ptx::mbar_init(&qdo_empty[s], 1);
    }
    ptx::mbar_init(sdp_full, 1);
    ptx::mbar_init(pds_full, 8);
    ptx::mbar_init(&mma_done[0], 1);
    ptx::mbar_init(&mma_done[1], 1);
    ptx::mbar_init(&dq_free[0], 4);
    ptx::mbar_init(&dq_free[1], 4);
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tmap(&tmap_q);
    ptx::prefetch_tmap(&tmap_do);
    ptx::prefetch_tmap(&tmap_k);
    ptx::prefetch_tmap(&tmap_v);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tm_ST = tmem_base;         // 64 columns
  const uint32_t tm_dPT = tmem_base + 64;   // 64
  const uint32_t tm_dQT = tmem_base + 128;  // 2 x 64 (steps alternate)
  const uint32_t tm_dV = tmem_base + 256;   // 128
  const uint32_t tm_dK = tmem_base + 384;   // 128

  if (warp == 0) {
    if (ptx::elect_one() && n_steps > 0) {
      ptx::mbar_expect_tx(kv_full, 2 * KV_TILE_BYTES);
      ptx::tma_load_3d(sK, map_k, kv_full, 0, hk, kv_row);
      ptx::tma_load_3d(sK + KV_PANEL, map_k, kv_full, 64, hk, kv_row);
      ptx::tma_load_3d(sV, map_v, kv_full, 0, hk, kv_row);
      ptx::tma_load_3d(sV + KV_PANEL, map_v, kv_full, 64, hk, kv_row);
      for (int n = 0; n < n_steps; n++) {
        const int s = n % QDO_STAGES;
        const uint32_t ph = (n / QDO_STAGES) & 1;
        const int h = h_first + n / tiles_per_head;
        int sq0, sm0;
        step_pos(n % tiles_per_head, sq0, sm0);
        const int row = q_begin + sq0;
        if (!ptx::mbar_wait(&qdo_empty[s], ph ^ 1, abort_flag)) break;
        ptx::mbar_expect_tx(&qdo_full[s], 2 * Q_TILE_BYTES);
        ptx::tma_load_3d(sQ + s * Q_TILE_BYTES, &tmap_q, &qdo_full[s], 0, h, row);
        ptx::tma_load_3d(sQ + s * Q_TILE_BYTES + Q_PANEL, &tmap_q, &qdo_full[s], 64, h, row);
        ptx::tma_load_3d(sdO + s * Q_TILE_BYTES, &tmap_do, &qdo_full[s], 0, h, row);
        ptx::tma_load_3d(sdO + s * Q_TILE_BYTES + Q_PANEL, &tmap_do, &qdo_full[s], 64, h, row);
      }
    }
  } else if (warp == 1) {
    if (ptx::elect_one() && n_steps > 0) {
      constexpr uint32_t idesc_s = ptx::make_idesc_bf16(BK, BQ, false, false);   // K Q^T, V dO^T
      constexpr uint32_t idesc_dv = ptx::make_idesc_bf16(BK, HD, false, true);   // P^T dO, dS^T Q
      constexpr uint32_t idesc_dq = ptx::make_idesc_bf16(HD, BQ, true, true);    // K^T dS^T
      const uint32_t aK = ptx::smem_u32(sK), aV = ptx::smem_u32(sV), aPT = ptx::smem_u32(sPT), adST = ptx::smem_u32(sdST);
      bool ok = ptx::mbar_wait(kv_full, 0, abort_flag);
      auto issue_s = [&](int n) -> bool {
        const int s = n % QDO_STAGES;
        if (!ptx::mbar_wait(&qdo_full[s], (n / QDO_STAGES) & 1, abort_flag)) return false;
        ptx::tc_fence_after();
        const uint32_t aQ = ptx::smem_u32(sQ + s * Q_TILE_BYTES), adO = ptx::smem_u32(sdO + s * Q_TILE_BYTES);
#pragma unroll
        for (int k = 0; k < HD / 16; k++) {
          const uint32_t offA = (k >> 2) * KV_PANEL + (k & 3) * 32;
          const uint32_t offB = (k >> 2) * Q_PANEL + (k & 3) * 32;
          ptx::umma_f16(tm_ST, ptx::make_smem_desc(aK + offA, 16, 1024), ptx::make_smem_desc(aQ + offB, 16, 1024), idesc_s, k != 0);
        }
#pragma unroll
        for (int k = 0; k < HD / 16; k++) {
          const uint32_t offA = (k >> 2) * KV_PANEL + (k & 3) * 32;
          const uint32_t offB = (k >> 2) * Q_PANEL + (k & 3) * 32;
          ptx::umma_f16(tm_dPT, ptx::make_smem_desc(aV + offA, 16, 1024), ptx::make_smem_desc(adO + offB, 16, 1024), idesc_s, k != 0);
        }
        ptx::umma_commit(sdp_full);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int n = 0; n < n_steps && ok; n++) {
        const int s = n & 1;
        if (!ptx::mbar_wait(pds_full, n & 1, abort_flag)) { ok = false; break; }
        ptx::tc_fence_after();
        // the softmax warps hold S^T / dP^T of this step in registers: the next step's scores go first, so that its softmax
        // overlaps the three products of this step
        if (n + 1 < n_steps) {
          if (!issue_s(n + 1)) { ok = false; break; }
        }
        const int qs = n % QDO_STAGES;
        const uint32_t aQ = ptx::smem_u32(sQ + qs * Q_TILE_BYTES), adO = ptx::smem_u32(sdO + qs * Q_TILE_BYTES);
        const uint32_t aPTs = aPT + s * PT_BYTES, adSTs = adST + s * PT_BYTES;
        // dV += P^T dO ; dK += dS^T Q   (K dimension = 64 queries: 4 steps of 16 rows)
#pragma unroll
        for (int k = 0; k < BQ / 16; k++) {
          ptx::umma_f16(tm_dV, ptx::make_smem_desc(aPTs + k * 32, 16, 1024), ptx::make_smem_desc(adO + k * 16 * 128, Q_PANEL, 1024), idesc_dv, (n | k) != 0);
        }
#pragma unroll
        for (int k = 0; k < BQ / 16; k++) {
          ptx::umma_f16(tm_dK, ptx::make_smem_desc(adSTs + k * 32, 16, 1024), ptx::make_smem_desc(aQ + k * 16 * 128, Q_PANEL, 1024), idesc_dv, (n | k) != 0);
        }
        // dQ^T = K^T dS^T   (K dimension = 128 keys: 8 steps of 16 rows), into the dQ^T buffer of this step's parity, once the
        // read-out warps are done with step n - 2
        if (n >= 2) {
          if (!ptx::mbar_wait(&dq_free[s], ((n - 2) >> 1) & 1, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after();
        }
#pragma unroll
        for (int k = 0; k < BK / 16; k++) {
          ptx::umma_f16(tm_dQT + s * BQ, ptx::make_smem_desc(aK + k * 16 * 128, KV_PANEL, 1024), ptx::make_smem_desc(adSTs + k * 16 * 128, PT_BYTES, 1024), idesc_dq, k != 0);
        }
        ptx::umma_commit(&qdo_empty[qs]);
        ptx::umma_commit(&mma_done[s]);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax / dQ read-out / final write-out
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;  // key row (S^T, dV, dK) and head-dim row (dQ^T)
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const int kpos = k0 + r;
    const bool key_valid = kpos < k_len;
    bool ok = true;
    // Warps 2-9: two warpgroups split the 64 query columns of a step: warpgroup `wg` owns columns [32 wg, 32 wg + 32) of S^T /
    // dP^T / P^T / dS^T for all 128 key rows, and after the last step writes out dK (wg 0) or dV (wg 1).
    // Warps 10-13: read dQ^T (128 head-dim rows x 64 queries) of every step out of tensor memory into the fp32 dQ buffer.
    const int wg = (warp - 2) >> 2;
    if (wg == 2) {
      int hi = 0, ti = 0;
      const int64_t stride = static_cast<int64_t>(p.num_heads) * HD;
      for (int n = 0; n < n_steps && ok; n++) {
        int q0, m0;
        step_pos(ti, q0, m0);
        const int h = h_first + hi;
        if (++ti == tiles_per_head) { ti = 0; hi++; }
        if (!ptx::mbar_wait(&mma_done[n & 1], (n >> 1) & 1, abort_flag)) { ok = false; break; }
        ptx::tc_fence_after();
        // dQ^T[r = head-dim index][64 queries] -> dq_acc[(q_begin + q0 + col), h, r]: a warp's 32 lanes add 32 consecutive floats
#pragma unroll 1
        for (int c = 0; c < 2; c++) {
          float* ptr = p.dq_acc + (static_cast<int64_t>(q_begin + q0 + c * 32) * p.num_heads + h) * HD + r;
          const int nq = min(32, q_len - q0 - c * 32);
          uint32_t v[32];
          ptx::tmem_ld_32x32(tm_dQT + lane_addr + (n & 1) * BQ + c * 32, v);
          ptx::tmem_ld_wait();
          if (nq == 32) {
#pragma unroll
            for (int i = 0; i < 32; i++) red_add_f32(ptr + i * stride, __uint_as_float(v[i]));
          } else {
#pragma unroll
            for (int i = 0; i < 32; i++)
              if (i < nq) red_add_f32(ptr + i * stride, __uint_as_float(v[i]));
          }
        }
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&dq_free[n & 1]);
      }
    } else {
    // Row statistics (lse, delta) of my 32 query columns, fetched one step ahead.  Only the loads are issued here: a warp issues
    // in order, so any arithmetic on the loaded values would stall it for the whole global-memory latency.  The values are
    // turned into (-lse log2 e, delta * scale) when they are stored to shared memory at the top of the next step.
    auto fetch_stats = [&](int hi, int ti, float& raw_lse, float& raw_delta) {
      const int h = h_first + hi;
      int q0, m0;
      step_pos(ti, q0, m0);
      const int qpos = min(q0 + wg * 32 + lane, q_len - 1);  // rows past the end read the last valid row; masked at use
      const int64_t idx = static_cast<int64_t>(h) * p.total_q + q_begin + qpos;
      raw_lse = p.lse[idx];
      raw_delta = p.delta[idx];
    };
    float lse_next = 0.f, delta_next = 0.f;
    if (n_steps > 0) fetch_stats(0, 0, lse_next, delta_next);
    int hi = 0, ti = 0;
    for (int n = 0; n < n_steps && ok; n++) {
      int q0, m0;
      step_pos(ti, q0, m0);
      if (++ti == tiles_per_head) { ti = 0; hi++; }  // (hi, ti) now name the next step
      // per-warp copy of the 32 row statistics of this step (no cross-warp synchronisation needed)
      float* lse_s = s_stats + (warp - 2) * 64;
      float* delta_s = lse_s + 32;
      {
        const bool in = q0 + wg * 32 + lane < q_len;
        lse_s[lane] = in ? -lse_next * 1.4426950408889634f : -INFINITY;  // exp2(s c - lse) = 0 for rows past the end
        delta_s[lane] = in ? delta_next * p.scale : 0.f;
      }
      __syncwarp();
      if (n + 1 < n_steps) fetch_stats(hi, ti, lse_next, delta_next);  // in flight during this step
      if (!ptx::mbar_wait(sdp_full, n & 1, abort_flag)) { ok = false; break; }
      ptx::tc_fence_after();
      uint32_t pk_p[16], pk_ds[16];  // 32 bf16 each
      // query columns this key row may look at: [clo, chi).  Queries past the end of the sequence are handled by lse = +inf.
      int clo = 0, chi = key_valid ? BQ : 0;
      if (p.causal) clo = max(0, kpos - shift - m0);
      if (p.window > 0) chi = min(chi, kpos - shift + p.window - m0);
      const bool full = __all_sync(0xffffffffu, clo == 0 && chi == BQ);
      const uint64_t sl2 = pack2(p.scale_log2, p.scale_log2), sc2 = pack2(p.scale, p.scale);
      {
        uint32_t sv[32], dv[32];
        ptx::tmem_ld_32x32(tm_ST + lane_addr + wg * 32, sv);
        ptx::tmem_ld_32x32(tm_dPT + lane_addr + wg * 32, dv);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 nl = *reinterpret_cast<const float4*>(lse_s + i);    // -lse * log2(e)
          const float4 ds = *reinterpret_cast<const float4*>(delta_s + i);  // delta * scale
          float e0, e1, e2, e3, t0, t1, t2, t3;
          unpack2(fma2(pack2(__uint_as_float(sv[i]), __uint_as_float(sv[i + 1])), sl2, pack2(nl.x, nl.y)), e0, e1);
          unpack2(fma2(pack2(__uint_as_float(sv[i + 2]), __uint_as_float(sv[i + 3])), sl2, pack2(nl.z, nl.w)), e2, e3);
          float p0 = ex2_approx(e0), p1 = ex2_approx(e1), p2 = ex2_approx(e2), p3 = ex2_approx(e3);
          if (!full) {
            const int col = wg * 32 + i;
            if (col < clo || col >= chi) p0 = 0.f;
            if (col + 1 < clo || col + 1 >= chi) p1 = 0.f;
            if (col + 2 < clo || col + 2 >= chi) p2 = 0.f;
            if (col + 3 < clo || col + 3 >= chi) p3 = 0.f;
          }
          // dS = P (dP - delta) scale
          const uint64_t u01 = fma2(pack2(__uint_as_float(dv[i]), __uint_as_float(dv[i + 1])), sc2, pack2(-ds.x, -ds.y));
          const uint64_t u23 = fma2(pack2(__uint_as_float(dv[i + 2]), __uint_as_float(dv[i + 3])), sc2, pack2(-ds.z, -ds.w));
          unpack2(fma2(pack2(p0, p1), u01, 0ull), t0, t1);
          unpack2(fma2(pack2(p2, p3), u23, 0ull), t2, t3);
          __nv_bfloat162 hp0 = __floats2bfloat162_rn(p0, p1), hp1 = __floats2bfloat162_rn(p2, p3);
          __nv_bfloat162 hd0 = __floats2bfloat162_rn(t0, t1), hd1 = __floats2bfloat162_rn(t2, t3);
          pk_p[i / 2] = *reinterpret_cast<uint32_t*>(&hp0);
          pk_p[i / 2 + 1] = *reinterpret_cast<uint32_t*>(&hp1);
          pk_ds[i / 2] = *reinterpret_cast<uint32_t*>(&hd0);
          pk_ds[i / 2 + 1] = *reinterpret_cast<uint32_t*>(&hd1);
        }
      }
      // P^T / dS^T buffer of this step's parity: its last readers were the products of step n - 2.  (mma_done[b] completes one
      // phase per two steps and the products of step n cannot start before this warp's arrival below, so the barrier is never
      // more than one phase ahead of this wait.)
      if (n >= 2) {
        if (!ptx::mbar_wait(&mma_done[n & 1], ((n - 2) >> 1) & 1, abort_flag)) { ok = false; break; }
      }
      uint8_t* prow = sPT + (n & 1) * PT_BYTES + r * 128;
      uint8_t* drow = sdST + (n & 1) * PT_BYTES + r * 128;
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const int sw = ((wg * 4 + u) ^ (r & 7)) << 4;
        *reinterpret_cast<uint4*>(prow + sw) = make_uint4(pk_p[u * 4], pk_p[u * 4 + 1], pk_p[u * 4 + 2], pk_p[u * 4 + 3]);
        *reinterpret_cast<uint4*>(drow + sw) = make_uint4(pk_ds[u * 4], pk_ds[u * 4 + 1], pk_ds[u * 4 + 2], pk_ds[u * 4 + 3]);
      }
      ptx::tc_fence_before();
      ptx::fence_proxy_async();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(pds_full);
    }
    if (ok && n_steps > 0 && ptx::mbar_wait(&mma_done[(n_steps - 1) & 1], ((n_steps - 1) >> 1) & 1, abort_flag)) {
      ptx::tc_fence_after();
      // dK, dV rows of this key.  Every lane issues the warp-aligned TMEM loads; only the stores depend on key_valid.
      const int64_t off = static_cast<int64_t>(k_begin + kpos) * p.dk_stride_t + static_cast<int64_t>(hk) * HD;
      const int64_t acc_off = (static_cast<int64_t>(kv_row + r) * p.num_kv_heads + hk) * HD;  // context parallel: row in the owner's accumulators
      {
        const int which = wg;  // warpgroup 0 writes dK, warpgroup 1 dV
        __nv_bfloat16* dst = (which == 0 ? p.dk : p.dv) + off;
        float* acc = cpm_on ? (which == 0 ? cpb.dk_acc[kv_owner] : cpb.dv_acc[kv_owner]) + acc_off : nullptr;
        if (p.split) acc = (which == 0 ? p.dk_split : p.dv_split) + (static_cast<int64_t>(k_begin + kpos) * p.num_kv_heads + hk) * HD;
        const uint32_t src = (which == 0 ? tm_dK : tm_dV) + lane_addr;
#pragma unroll 1
        for (int c = 0; c < 4; c++) {
          uint32_t v[32];
          ptx::tmem_ld_32x32(src + c * 32, v);
          ptx::tmem_ld_wait();
          if (cpm_on || p.split) {
            // partial sums (of this rank's queries / of this query head): reduce into fp32 rows (16-byte reductions; under context
            // parallelism the rows belong to the key owner and may sit across NVLink)
            if (key_valid) {
#pragma unroll
              for (int u = 0; u < 8; u++)
                atomicAdd(reinterpret_cast<float4*>(acc + c * 32 + u * 4),
                          make_float4(__uint_as_float(v[u * 4]), __uint_as_float(v[u * 4 + 1]), __uint_as_float(v[u * 4 + 2]), __uint_as_float(v[u * 4 + 3])));
            }
          } else if (key_valid) {
#pragma unroll
            for (int u = 0; u < 4; u++) {
              uint4 pk;
              __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(v[u * 8 + 0]), __uint_as_float(v[u * 8 + 1]));
              __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(v[u * 8 + 2]), __uint_as_float(v[u * 8 + 3]));
              __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(v[u * 8 + 4]), __uint_as_float(v[u * 8 + 5]));
              __nv_bfloat162 h3 = __floats2bfloat162_rn(__uint_as_float(v[u * 8 + 6]), __uint_as_float(v[u * 8 + 7]));
              pk.x = *reinterpret_cast<uint32_t*>(&h0); pk.y = *reinterpret_cast<uint32_t*>(&h1);
              pk.z = *reinterpret_cast<uint32_t*>(&h2); pk.w = *reinterpret_cast<uint32_t*>(&h3);
              *reinterpret_cast<uint4*>(dst + c * 32 + u * 8) = pk;
            }
          }
        }
      }
    } else if (n_steps == 0 && key_valid && !cpm_on && !p.split) {
      // no query sees these keys: their gradients are zero
      const int64_t off = static_cast<int64_t>(k_begin + kpos) * p.dk_stride_t + static_cast<int64_t>(hk) * HD;
      for (int c = 0; c < HD; c += 8) {
        *reinterpret_cast<uint4*>(p.dk + off + c) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(p.dv + off + c) = make_uint4(0, 0, 0, 0);
      }
    }
    }  // softmax warpgroups
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, NTB_ERR_TIMEOUT);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn bwd_get_encode() {
  ntb_bind_context_to_thread();
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

bool make_map(CUtensorMap* m, const void* ptr, int64_t tokens, int heads, int64_t stride_t, int64_t stride_h, int box_rows) {
  cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)heads, (cuuint64_t)tokens};
  cuuint64_t strides[2] = {(cuuint64_t)stride_h * 2, (cuuint64_t)stride_t * 2};
  cuuint32_t box[3] = {64, 1, (cuuint32_t)box_rows};
  cuuint32_t es[3] = {1, 1, 1};
  return bwd_get_encode()(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// dout / out: [total_q, Hq, 128] contiguous.  q, k, v: strided like the forward (v shares k's strides).  delta: fp32 [Hq, total_q]
// scratch; dq_acc: fp32 [total_q, Hq, 128] zero-filled scratch.  dq / dk / dv: bf16 outputs with token strides dq_stride_t /
// dk_stride_t (head stride 128), e.g. views of one fused [T, Hq + 2 Hkv, 128] buffer.
// dkv_split: nullptr, or fp32 [2, total_k, Hkv, 128] zero-filled scratch that selects the split mode (one CTA per key tile and QUERY
// head; see BwdParams::split).  ntb_flash_attn_bwd_wants_split says when that pays.
static int flash_attn_bwd_impl(const void* dout, const void* q, const void* k, const void* v, const void* out, const float* lse, float* delta, float* dq_acc,
                               void* dq, void* dk, void* dv, float* dkv_split, const int* cu_q, const int* cu_k, int batch, int max_seqlen_q, int max_seqlen_k, int total_q,
                               int total_k, int num_heads, int num_kv_heads, int64_t q_stride_t, int64_t q_stride_h, int64_t k_stride_t, int64_t k_stride_h,
                               int64_t dq_stride_t, int64_t dk_stride_t, float softmax_scale, int causal, int window, int* status, cudaStream_t stream) {
  if (!bwd_get_encode() || batch <= 0 || total_q <= 0 || total_k <= 0 || num_heads % num_kv_heads) return NTB_ERR_ARG;
  if ((q_stride_t | q_stride_h | k_stride_t | k_stride_h | dq_stride_t | dk_stride_t) % 8) return NTB_ERR_ARG;
  CUtensorMap tq, tdo, tk, tv;
  if (!make_map(&tq, q, total_q, num_heads, q_stride_t, q_stride_h, BQ) || !make_map(&tdo, dout, total_q, num_heads, (int64_t)num_heads * HD, HD, BQ) ||
      !make_map(&tk, k, total_k, num_kv_heads, k_stride_t, k_stride_h, BK) || !make_map(&tv, v, total_k, num_kv_heads, k_stride_t, k_stride_h, BK))
    return NTB_ERR_ARG;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(flash_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM) != cudaSuccess) return NTB_ERR_LAUNCH;
    configured = true;
  }
  {
    const int64_t warps = static_cast<int64_t>(total_q) * num_heads;
    delta_kernel<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(out), reinterpret_cast<const __nv_bfloat16*>(dout), delta, total_q, num_heads);
  }
  BwdParams p;
  p.num_heads = num_heads;
  p.num_kv_heads = num_kv_heads;
  p.causal = causal;
  p.window = window;
  p.scale = softmax_scale;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.cu_q = cu_q;
  p.cu_k = cu_k;
  p.lse = lse;
  p.delta = delta;
  p.dq_acc = dq_acc;
  p.dk = reinterpret_cast<__nv_bfloat16*>(dk);
  p.dv = reinterpret_cast<__nv_bfloat16*>(dv);
  p.dk_stride_t = dk_stride_t;
  p.total_q = total_q;
  p.status = status;
  p.split = dkv_split != nullptr;
  p.dk_split = dkv_split;
  p.dv_split = dkv_split ? dkv_split + static_cast<int64_t>(total_k) * num_kv_heads * HD : nullptr;
  dim3 grid((p.split ? num_heads : num_kv_heads) * batch, (max_seqlen_k + BK - 1) / BK, 1);
  if (grid.y > 65535) return NTB_ERR_ARG;
  p.cp = 0;
  p.cp_me = 0;
  p.cp_chunk = 0;
  static const CpBwd no_cp = {};
  flash_bwd_kernel<<<grid, BWD_THREADS, BWD_SMEM, stream>>>(tq, tdo, tk, tv, p, no_cp);
  int rc = ntb_check_launch();
  if (rc) return rc;
  const int64_t n8 = static_cast<int64_t>(total_q) * num_heads * HD / 8;
  cast_dq_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, stream>>>(dq_acc, reinterpret_cast<__nv_bfloat16*>(dq), total_q, num_heads, dq_stride_t);
  if (p.split) {
    const int64_t k8 = static_cast<int64_t>(total_k) * num_kv_heads * HD / 8;
    cast_dq_kernel<<<(unsigned)((k8 + 255) / 256), 256, 0, stream>>>(p.dk_split, reinterpret_cast<__nv_bfloat16*>(dk), total_k, num_kv_heads, dk_stride_t);
    cast_dq_kernel<<<(unsigned)((k8 + 255) / 256), 256, 0, stream>>>(p.dv_split, reinterpret_cast<__nv_bfloat16*>(dv), total_k, num_kv_heads, dk_stride_t);
  }
  return ntb_check_launch();
}

NTB_EXPORT int ntb_flash_attn_bwd(const void* dout, const void* q, const void* k, const void* v, const void* out, const float* lse, float* delta, float* dq_acc,
                                  void* dq, void* dk, void* dv, const int* cu_q, const int* cu_k, int batch, int max_seqlen_q, int max_seqlen_k, int total_q,
                                  int total_k, int num_heads, int num_kv_heads, int64_t q_stride_t, int64_t q_stride_h, int64_t k_stride_t, int64_t k_stride_h,
                                  int64_t dq_stride_t, int64_t dk_stride_t, float softmax_scale, int causal, int window, int* status, cudaStream_t stream) {
  return flash_attn_bwd_impl(dout, q, k, v, out, lse, delta, dq_acc, dq, dk, dv, nullptr, cu_q, cu_k, batch, max_seqlen_q, max_seqlen_k, total_q, total_k, num_heads,
                             num_kv_heads, q_stride_t, q_stride_h, k_stride_t, k_stride_h, dq_stride_t, dk_stride_t, softmax_scale, causal, window, status, stream);
}

// 1 when (key tiles x kv heads x sequences) CTAs would leave most of the GPU idle and splitting the query heads of a group over
// CTAs (with fp32 dK / dV accumulation) gives the launch enough parallelism.
NTB_EXPORT int ntb_flash_attn_bwd_wants_split(int batch, int max_seqlen_k, int num_heads, int num_kv_heads) {
  if (num_heads == num_kv_heads) return 0;
  const int64_t ctas = static_cast<int64_t>((max_seqlen_k + BK - 1) / BK) * num_kv_heads * batch;
  return ctas < 148 + 74 ? 1 : 0;
}

NTB_EXPORT int ntb_flash_attn_bwd_split(const void* dout, const void* q, const void* k, const void* v, const void* out, const float* lse, float* delta, float* dq_acc,
                                        void* dq, void* dk, void* dv, float* dkv_split, const int* cu_q, const int* cu_k, int batch, int max_seqlen_q, int max_seqlen_k,
                                        int total_q, int total_k, int num_heads, int num_kv_heads, int64_t q_stride_t, int64_t q_stride_h, int64_t k_stride_t,
                                        int64_t k_stride_h, int64_t dq_stride_t, int64_t dk_stride_t, float softmax_scale, int causal, int window, int* status,
                                        cudaStream_t stream) {
  if (dkv_split == nullptr || (reinterpret_cast<uintptr_t>(dkv_split) & 15)) return NTB_ERR_ARG;
  return flash_attn_bwd_impl(dout, q, k, v, out, lse, delta, dq_acc, dq, dk, dv, dkv_split, cu_q, cu_k, batch, max_seqlen_q, max_seqlen_k, total_q, total_k, num_heads,
                             num_kv_heads, q_stride_t, q_stride_h, k_stride_t, k_stride_h, dq_stride_t, dk_stride_t, softmax_scale, causal, window, status, stream);
}

// Context-parallel backward (zig-zag layout, causal).  k_ptrs / v_ptrs: every rank's K / V as in ntb_flash_attn_fwd_cp; dk_acc_ptrs /
// dv_acc_ptrs: every rank's fp32 [batch * 2 * chunk, Hkv, 128] accumulators, zeroed and made visible by a barrier before this launch.
// dq (bf16, token stride dq_stride_t) is complete when the stream reaches the end of this call; dK / dV of this rank are complete in
// its accumulators only after the NEXT cross-rank barrier (peers add into them); ntb_cast_f32_to_bf16_rows then converts them.
NTB_EXPORT int ntb_flash_attn_bwd_cp(const void* dout, const void* q, const uint64_t* k_ptrs, const uint64_t* v_ptrs, const void* out, const float* lse, float* delta,
                                     float* dq_acc, void* dq, const uint64_t* dk_acc_ptrs, const uint64_t* dv_acc_ptrs, int batch, int chunk, int cp, int me,
                                     int num_heads, int num_kv_heads, int64_t q_stride_t, int64_t q_stride_h, int64_t kv_stride_t, int64_t kv_stride_h,
                                     int64_t dq_stride_t, float softmax_scale, int* status, cudaStream_t stream) {
  if (!bwd_get_encode() || batch <= 0 || chunk <= 0 || chunk % BK || cp < 1 || cp > CP_MAX || me < 0 || me >= cp || num_heads % num_kv_heads) return NTB_ERR_ARG;
  if ((q_stride_t | q_stride_h | kv_stride_t | kv_stride_h | dq_stride_t) % 8) return NTB_ERR_ARG;
  const int total = batch * 2 * chunk;
  CUtensorMap tq, tdo;
  CpBwd cpb = {};
  if (!make_map(&tq, q, total, num_heads, q_stride_t, q_stride_h, BQ) || !make_map(&tdo, dout, total, num_heads, (int64_t)num_heads * HD, HD, BQ)) return NTB_ERR_ARG;
  for (int r = 0; r < cp; r++) {
    if ((k_ptrs[r] | v_ptrs[r] | dk_acc_ptrs[r] | dv_acc_ptrs[r]) & 15) return NTB_ERR_ARG;
    if (!make_map(&cpb.k[r], reinterpret_cast<const void*>(k_ptrs[r]), total, num_kv_heads, kv_stride_t, kv_stride_h, BK) ||
        !make_map(&cpb.v[r], reinterpret_cast<const void*>(v_ptrs[r]), total, num_kv_heads, kv_stride_t, kv_stride_h, BK))
      return NTB_ERR_ARG;
    cpb.dk_acc[r] = reinterpret_cast<float*>(dk_acc_ptrs[r]);
    cpb.dv_acc[r] = reinterpret_cast<float*>(dv_acc_ptrs[r]);
  }
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(flash_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM) != cudaSuccess) return NTB_ERR_LAUNCH;
    configured = true;
  }
  {
    const int64_t warps = static_cast<int64_t>(total) * num_heads;
    delta_kernel<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(out), reinterpret_cast<const __nv_bfloat16*>(dout), delta, total, num_heads);
  }
  BwdParams p;
  p.num_heads = num_heads;
  p.num_kv_heads = num_kv_heads;
  p.causal = 1;
  p.window = 0;
  p.scale = softmax_scale;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.cu_q = nullptr;
  p.cu_k = nullptr;
  p.lse = lse;
  p.delta = delta;
  p.dq_acc = dq_acc;
  p.dk = nullptr;
  p.dv = nullptr;
  p.dk_stride_t = 0;
  p.total_q = total;
  p.status = status;
  p.cp = cp;
  p.cp_me = me;
  p.cp_chunk = chunk;
  p.split = 0;
  p.dk_split = nullptr;
  p.dv_split = nullptr;
  dim3 grid(num_kv_heads * batch, 2 * cp * chunk / BK, 1);
  if (grid.y > 65535) return NTB_ERR_ARG;
  flash_bwd_kernel<<<grid, BWD_THREADS, BWD_SMEM, stream>>>(tq, tdo, cpb.k[me], cpb.v[me], p, cpb);
  int rc = ntb_check_launch();
  if (rc) return rc;
  const int64_t n8 = static_cast<int64_t>(total) * num_heads * HD / 8;
  cast_dq_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, stream>>>(dq_acc, reinterpret_cast<__nv_bfloat16*>(dq), total, num_heads, dq_stride_t);
  return ntb_check_launch();
}

// fp32 [rows, heads, 128] -> bf16 with token stride dst_stride_t (head stride 128).
NTB_EXPORT int ntb_cast_f32_to_bf16_rows(const float* src, void* dst, int64_t rows, int heads, int64_t dst_stride_t, cudaStream_t stream) {
  if (rows <= 0 || heads <= 0 || dst_stride_t % 8) return NTB_ERR_ARG;
  const int64_t n8 = rows * heads * HD / 8;
  cast_dq_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, stream>>>(src, reinterpret_cast<__nv_bfloat16*>(dst), rows, heads, dst_stride_t);
  return ntb_check_launch();
}

