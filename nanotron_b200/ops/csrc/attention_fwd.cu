// Flash attention forward on tcgen05 / TMEM (sm_100a): head dim 128, bf16, causal or full, GQA, packed variable-length
// sequences (cu_seqlens), returns the log-sum-exp per (head, token).
//
// One CTA per (128-query tile, query head, sequence).  Warp roles:
//   warp 0     TMA producer: Q once, then K / V tiles of 128 keys through 2-stage rings (per-CTA loads, 128-byte swizzle)
//   warp 1     MMA issuer:   S = Q K^T  (128x128x128, fp32 in TMEM, double buffered so S(j+1) is computed while the
//                            softmax of tile j runs), then O += P V with P read from shared memory
//   warps 2-5  softmax:      thread r owns query row r.  Two passes over S in TMEM (row max, then exp2 / sum / bf16 P into
//                            swizzled shared memory); O in TMEM is rescaled only when some row of the warp raised its max.
// Epilogue: O / l from TMEM straight to global memory (rows past the end of the sequence are not written), LSE to global.
// Tiles hanging over the end of a packed sequence read the next sequence's keys: those columns are masked to -inf.
// All barrier waits are bounded; a timeout raises `status` and the CTA unwinds.
//
// Context-parallel mode (p.cp > 0): the sequence is split in 2 * cp chunks of `cp_chunk` tokens and rank r holds chunks r and
// 2 cp - 1 - r (zig-zag) of every batch row, one after the other.  Keys / values stay where they are: every rank's K and V live in
// peer-mapped buffers and the TMA producer of this kernel reads the tiles it needs straight from their owner (one tensor map per
// peer, per-CTA loads over NVLink), so the "ring exchange" happens tile by tile inside the attention kernel and overlaps its MMAs.
// Masking uses global positions: key tile j covers global keys [128 j, 128 j + 128) wherever it is stored.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace {

constexpr int HD = 128;          // head dim
constexpr int BM = 128;          // queries per CTA
constexpr int BN = 128;          // keys per tile
constexpr int KV_STAGES = 2;
constexpr int TILE_BYTES = 128 * HD * 2;  // 32 KiB: two 16 KiB panels of [128 rows][64 elements]
constexpr int PANEL_BYTES = 128 * 64 * 2;
constexpr int FA_THREADS = 192;
constexpr int FA_SMEM = TILE_BYTES * (1 + 2 * KV_STAGES + 1) + 1024 + 256;  // Q, K ring, V ring, P

struct FwdParams {
  int num_heads, num_kv_heads;
  int causal;
  int window;  // <= 0: none
  float scale_log2;  // softmax_scale * log2(e)
  float scale;
  const int* cu_q;
  const int* cu_k;
  __nv_bfloat16* out;  // [T, Hq, HD] contiguous
  float* lse;          // [Hq, T]
  int total_q;
  int* status;
  int cp, cp_me, cp_chunk;  // context parallel: group size (0 = off), this rank, tokens per chunk (multiple of 128)
};

constexpr int CP_MAX = 8;
struct CpMaps {
  CUtensorMap k[CP_MAX];
  CUtensorMap v[CP_MAX];
};

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]),
      "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
      "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__global__ void __launch_bounds__(FA_THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                 const FwdParams p, const __grid_constant__ CpMaps cpm) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + TILE_BYTES;
  uint8_t* sV = sK + KV_STAGES * TILE_BYTES;
  uint8_t* sP = sV + KV_STAGES * TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + TILE_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;   // [2]
  uint64_t* k_empty = bars + 3;  // [2]
  uint64_t* v_full = bars + 5;   // [2]
  uint64_t* v_empty = bars + 7;  // [2]
  uint64_t* s_full = bars + 9;   // [2]
  uint64_t* s_empty = bars + 11; // [2]
  uint64_t* p_full = bars + 13;
  uint64_t* pv_done = bars + 14;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, h = blockIdx.y;
  const bool cpm_on = p.cp > 0;
  const int q_begin = cpm_on ? b * 2 * p.cp_chunk : p.cu_q[b];
  const int q_len = cpm_on ? 2 * p.cp_chunk : p.cu_q[b + 1] - q_begin;
  const int k_begin = cpm_on ? 0 : p.cu_k[b];
  const int k_len = cpm_on ? 2 * p.cp * p.cp_chunk : p.cu_k[b + 1] - k_begin;
  // heavy (late) query tiles first: with a causal mask they have the most key tiles
  const int q_tile = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
  const int q0 = q_tile * BM;
  if (q0 >= q_len) return;  // uniform for the CTA
  // position of the tile's first query for masking: local position, or the global one under context parallelism
  int mq0 = q0;
  if (cpm_on) {
    const int half = q0 / p.cp_chunk;
    const int chunk = half == 0 ? p.cp_me : 2 * p.cp - 1 - p.cp_me;
    mq0 = chunk * p.cp_chunk + (q0 - half * p.cp_chunk);
  }
  const int shift = cpm_on ? 0 : k_len - q_len;  // bottom-right aligned causal mask
  int kv_end = k_len;
  if (p.causal) kv_end = min(k_len, mq0 + BM + shift);
  int kv_start = 0;
  if (p.window > 0) kv_start = max(0, (mq0 + shift - p.window + 1) / BN * BN);
  const int n_tiles = kv_end > kv_start ? (kv_end - kv_start + BN - 1) / BN : 0;
  const int hk = h / (p.num_heads / p.num_kv_heads);

  if (threadIdx.x == 0) {
    ptx::mbar_init(q_full, 1);
    for (int s = 0; s < 2; s++) {
      ptx::mbar_init(&k_full[s], 1);
      ptx::mbar_init(&k_empty[s], 1);
      ptx::mbar_init(&v_full[s], 1);
      ptx::mbar_init(&v_empty[s], 1);
      ptx::mbar_init(&s_full[s], 1);
      ptx::mbar_init(&s_empty[s], 4);
    }
    ptx::mbar_init(p_full, 4);
    ptx::mbar_init(pv_done, 1);
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tmap(&tmap_q);
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
  const uint32_t tmem_S = tmem_base;        // 2 x 128 columns
  const uint32_t tmem_O = tmem_base + 256;  // 128 columns

  if (warp == 0) {
    if (ptx::elect_one() && n_tiles > 0) {
      ptx::mbar_expect_tx(q_full, TILE_BYTES);
      ptx::tma_load_3d(sQ, &tmap_q, q_full, 0, h, q_begin + q0);
      ptx::tma_load_3d(sQ + PANEL_BYTES, &tmap_q, q_full, 64, h, q_begin + q0);
      for (int j = 0; j < n_tiles; j++) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        int krow = k_begin + kv_start + j * BN;
        const CUtensorMap* mk = &tmap_k;
        const CUtensorMap* mv = &tmap_v;
        if (cpm_on) {
          // global key tile -> the rank that stores it and the row inside that rank's [batch, 2 chunks] buffer
          const int gk = kv_start + j * BN;
          const int chunk = gk / p.cp_chunk;
          const int owner = chunk < p.cp ? chunk : 2 * p.cp - 1 - chunk;
          krow = b * 2 * p.cp_chunk + (chunk < p.cp ? 0 : p.cp_chunk) + (gk - chunk * p.cp_chunk);
          mk = &cpm.k[owner];
          mv = &cpm.v[owner];
        }
        if (!ptx::mbar_wait(&k_empty[s], ph ^ 1, abort_flag)) break;
        ptx::mbar_expect_tx(&k_full[s], TILE_BYTES);
        ptx::tma_load_3d(sK + s * TILE_BYTES, mk, &k_full[s], 0, hk, krow);
        ptx::tma_load_3d(sK + s * TILE_BYTES + PANEL_BYTES, mk, &k_full[s], 64, hk, krow);
        if (!ptx::mbar_wait(&v_empty[s], ph ^ 1, abort_flag)) break;
        ptx::mbar_expect_tx(&v_full[s], TILE_BYTES);
        ptx::tma_load_3d(sV + s * TILE_BYTES, mv, &v_full[s], 0, hk, krow);
        ptx::tma_load_3d(sV + s * TILE_BYTES + PANEL_BYTES, mv, &v_full[s], 64, hk, krow);
      }
    }
  } else if (warp == 1) {
    if (ptx::elect_one() && n_tiles > 0) {
      constexpr uint32_t idesc_qk = ptx::make_idesc_bf16(BM, BN, false, false);
      constexpr uint32_t idesc_pv = ptx::make_idesc_bf16(BM, HD, false, true);
      const uint32_t aQ = ptx::smem_u32(sQ), aP = ptx::smem_u32(sP);
      bool ok = ptx::mbar_wait(q_full, 0, abort_flag);
      auto issue_qk = [&](int j) -> bool {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!ptx::mbar_wait(&k_full[s], ph, abort_flag)) return false;
        if (!ptx::mbar_wait(&s_empty[s], ph ^ 1, abort_flag)) return false;
        ptx::tc_fence_after();
        const uint32_t aK = ptx::smem_u32(sK + s * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < HD / 16; k++) {
          const uint32_t off = (k >> 2) * PANEL_BYTES + (k & 3) * 32;
          ptx::umma_f16(tmem_S + s * BN, ptx::make_smem_desc(aQ + off, 16, 1024), ptx::make_smem_desc(aK + off, 16, 1024), idesc_qk, k != 0);
        }
        ptx::umma_commit(&k_empty[s]);
        ptx::umma_commit(&s_full[s]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < n_tiles && ok; j++) {
        if (j + 1 < n_tiles) {
          if (!issue_qk(j + 1)) { ok = false; break; }
        }
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!ptx::mbar_wait(&v_full[s], ph, abort_flag)) { ok = false; break; }
        if (!ptx::mbar_wait(p_full, j & 1, abort_flag)) { ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t aV = ptx::smem_u32(sV + s * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < BN / 16; k++) {
          const uint64_t adesc = ptx::make_smem_desc(aP + (k >> 2) * PANEL_BYTES + (k & 3) * 32, 16, 1024);
          const uint64_t bdesc = ptx::make_smem_desc(aV + k * 16 * 128, PANEL_BYTES, 1024);
          ptx::umma_f16(tmem_O, adesc, bdesc, idesc_pv, (j | k) != 0);
        }
        ptx::umma_commit(&v_empty[s]);
        ptx::umma_commit(pv_done);
      }
    }
  } else if (n_tiles > 0) {
    // ------------------------------------------------------------------ softmax / correction / epilogue
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;       // query row inside the tile
    const int qpos = q0 + r;                  // position inside the (local) sequence: validity and output row
    const int mpos = mq0 + r;                 // position used by the masks
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; j++) {
      const int s = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      const int k0 = kv_start + j * BN;
      if (!ptx::mbar_wait(&s_full[s], ph, abort_flag)) { ok = false; break; }
      ptx::tc_fence_after();
      const uint32_t tS = tmem_S + lane_addr + s * BN;
      // columns this row may look at: [lo, hi)
      int hi = k_len - k0;
      if (p.causal) hi = min(hi, mpos + shift - k0 + 1);
      int lo = 0;
      if (p.window > 0) lo = max(0, mpos + shift - p.window + 1 - k0);
      const bool need_mask = (hi < BN) || (lo > 0);
      // pass 1: row max
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; c++) {
        uint32_t v[32];
        ptx::tmem_ld_32x32(tS + c * 32, v);
        ptx::tmem_ld_wait();
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; i++) {
            const int col = c * 32 + i;
            if (col >= lo && col < hi) mx = fmaxf(mx, __uint_as_float(v[i]));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i++) mx = fmaxf(mx, __uint_as_float(v[i]));
        }
      }
      const float m_new = fmaxf(m_run, mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;  // fully masked row so far: keep exp2 finite
      const float alpha = exp2f((m_run - m_use) * p.scale_log2);  // 0 when m_run = -inf
      // O and the P buffer are free once the previous P*V has completed
      if (j > 0) {
        if (!ptx::mbar_wait(pv_done, (j - 1) & 1, abort_flag)) { ok = false; break; }
        ptx::tc_fence_after();
        if (__any_sync(0xffffffffu, alpha != 1.f)) {
          const uint32_t tO = tmem_O + lane_addr;
#pragma unroll 1
          for (int c = 0; c < 4; c++) {
            uint32_t v[32];
            ptx::tmem_ld_32x32(tO + c * 32, v);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i++) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tmem_st_32x32(tO + c * 32, v);
          }
          tmem_st_wait();
        }
      }
      // pass 2: probabilities -> bf16 -> shared memory (A operand of P*V), row sum
      float sum = 0.f;
      const float neg_m = -m_use * p.scale_log2;
      uint8_t* prow0 = sP + r * 128;
#pragma unroll 1
      for (int c = 0; c < 4; c++) {
        uint32_t v[32];
        ptx::tmem_ld_32x32(tS + c * 32, v);
        ptx::tmem_ld_wait();
        float e[32];
#pragma unroll
        for (int i = 0; i < 32; i++) {
          const int col = c * 32 + i;
          float x = exp2f(fmaf(__uint_as_float(v[i]), p.scale_log2, neg_m));
          if (need_mask && (col < lo || col >= hi)) x = 0.f;
          e[i] = x;
          sum += x;
        }
        uint8_t* prow = prow0 + (c >> 1) * PANEL_BYTES;
#pragma unroll
        for (int u = 0; u < 4; u++) {
          uint4 pk;
          __nv_bfloat162 h0 = __floats2bfloat162_rn(e[u * 8 + 0], e[u * 8 + 1]), h1 = __floats2bfloat162_rn(e[u * 8 + 2], e[u * 8 + 3]);
          __nv_bfloat162 h2 = __floats2bfloat162_rn(e[u * 8 + 4], e[u * 8 + 5]), h3 = __floats2bfloat162_rn(e[u * 8 + 6], e[u * 8 + 7]);
          pk.x = *reinterpret_cast<uint32_t*>(&h0); pk.y = *reinterpret_cast<uint32_t*>(&h1);
          pk.z = *reinterpret_cast<uint32_t*>(&h2); pk.w = *reinterpret_cast<uint32_t*>(&h3);
          const int unit = (c & 1) * 4 + u;
          *reinterpret_cast<uint4*>(prow + ((unit ^ (r & 7)) << 4)) = pk;
        }
      }
      l_run = l_run * alpha + sum;
      m_run = m_new;
      // S buffer read, P written: tell the MMA warp
      ptx::tc_fence_before();
      ptx::fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        ptx::mbar_arrive(&s_empty[s]);
        ptx::mbar_arrive(p_full);
      }
    }
    // ------------------------------------------------------------------ epilogue
    if (ok && ptx::mbar_wait(pv_done, (n_tiles - 1) & 1, abort_flag)) {
      ptx::tc_fence_after();
      const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
      const bool valid = qpos < q_len;
      const int64_t tok = static_cast<int64_t>(q_begin) + qpos;
      __nv_bfloat16* orow = p.out + (tok * p.num_heads + h) * HD;
      const uint32_t tO = tmem_O + lane_addr;
#pragma unroll 1
      for (int c = 0; c < 4; c++) {
        uint32_t v[32];
        ptx::tmem_ld_32x32(tO + c * 32, v);
        ptx::tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int u = 0; u < 4; u++) {
            uint4 pk;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(v[u * 8 + 0]) * inv_l, __uint_as_float(v[u * 8 + 1]) * inv_l);
            __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(v[u * 8 + 2]) * inv_l, __uint_as_float(v[u * 8 + 3]) * inv_l);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(v[u * 8 + 4]) * inv_l, __uint_as_float(v[u * 8 + 5]) * inv_l);
            __nv_bfloat162 h3 = __floats2bfloat162_rn(__uint_as_float(v[u * 8 + 6]) * inv_l, __uint_as_float(v[u * 8 + 7]) * inv_l);
            pk.x = *reinterpret_cast<uint32_t*>(&h0); pk.y = *reinterpret_cast<uint32_t*>(&h1);
            pk.z = *reinterpret_cast<uint32_t*>(&h2); pk.w = *reinterpret_cast<uint32_t*>(&h3);
            *reinterpret_cast<uint4*>(orow + c * 32 + u * 8) = pk;
          }
        }
      }
      if (valid) p.lse[static_cast<int64_t>(h) * p.total_q + tok] = (l_run > 0.f) ? m_run * p.scale + logf(l_run) : -INFINITY;
    }
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
EncodeTiledFn fa_get_encode() {
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

// [tokens, heads, 128] bf16 with element strides (stride_t, stride_h, 1): 3-D map {128, heads, tokens}, box {64, 1, 128}.
bool make_qkv_map(CUtensorMap* m, const void* ptr, int64_t tokens, int heads, int64_t stride_t, int64_t stride_h) {
  cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)heads, (cuuint64_t)tokens};
  cuuint64_t strides[2] = {(cuuint64_t)stride_h * 2, (cuuint64_t)stride_t * 2};
  cuuint32_t box[3] = {64, 1, 128};
  cuuint32_t es[3] = {1, 1, 1};
  return fa_get_encode()(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// q: [total_q, Hq, 128], k/v: [total_k, Hkv, 128] bf16 (token / head strides in elements, last dim contiguous);
// out: [total_q, Hq, 128] contiguous; lse: fp32 [Hq, total_q]; cu_q / cu_k: int32 [batch + 1] on the device.
NTB_EXPORT int ntb_flash_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, const int* cu_q, const int* cu_k, int batch,
                                  int max_seqlen_q, int total_q, int total_k, int num_heads, int num_kv_heads, int64_t q_stride_t, int64_t q_stride_h,
                                  int64_t k_stride_t, int64_t k_stride_h, int64_t v_stride_t, int64_t v_stride_h, float softmax_scale, int causal, int window,
                                  int* status, cudaStream_t stream) {
  if (!fa_get_encode() || batch <= 0 || total_q <= 0 || total_k <= 0 || num_heads % num_kv_heads) return NTB_ERR_ARG;
  if ((q_stride_t | q_stride_h | k_stride_t | k_stride_h | v_stride_t | v_stride_h) % 8) return NTB_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(out)) & 15) return NTB_ERR_ARG;
  CUtensorMap tq, tk, tv;
  if (!make_qkv_map(&tq, q, total_q, num_heads, q_stride_t, q_stride_h) || !make_qkv_map(&tk, k, total_k, num_kv_heads, k_stride_t, k_stride_h) ||
      !make_qkv_map(&tv, v, total_k, num_kv_heads, v_stride_t, v_stride_h))
    return NTB_ERR_ARG;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(flash_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FA_SMEM) != cudaSuccess) return NTB_ERR_LAUNCH;
    configured = true;
  }
  FwdParams p;
  p.num_heads = num_heads;
  p.num_kv_heads = num_kv_heads;
  p.causal = causal;
  p.window = window;
  p.scale = softmax_scale;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.cu_q = cu_q;
  p.cu_k = cu_k;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.total_q = total_q;
  p.status = status;
  p.cp = 0;
  p.cp_me = 0;
  p.cp_chunk = 0;
  static const CpMaps no_cp = {};
  dim3 grid((max_seqlen_q + BM - 1) / BM, num_heads, batch);
  flash_fwd_kernel<<<grid, FA_THREADS, FA_SMEM, stream>>>(tq, tk, tv, p, no_cp);
  return ntb_check_launch();
}

// Context-parallel forward.  q: this rank's [batch * 2 * chunk, Hq, 128] (chunk r then chunk 2 cp - 1 - r of every batch row);
// k_ptrs / v_ptrs: device addresses of every rank's [batch * 2 * chunk, Hkv, 128] K and V (peer-mapped, same strides everywhere,
// filled and made visible by a cross-rank barrier before this launch).  Causal only.  out / lse as in ntb_flash_attn_fwd.
NTB_EXPORT int ntb_flash_attn_fwd_cp(const void* q, const uint64_t* k_ptrs, const uint64_t* v_ptrs, void* out, float* lse, int batch, int chunk, int cp, int me,
                                     int num_heads, int num_kv_heads, int64_t q_stride_t, int64_t q_stride_h, int64_t kv_stride_t, int64_t kv_stride_h,
                                     float softmax_scale, int* status, cudaStream_t stream) {
  if (!fa_get_encode() || batch <= 0 || chunk <= 0 || chunk % BM || cp < 1 || cp > CP_MAX || me < 0 || me >= cp || num_heads % num_kv_heads) return NTB_ERR_ARG;
  if ((q_stride_t | q_stride_h | kv_stride_t | kv_stride_h) % 8) return NTB_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out)) & 15) return NTB_ERR_ARG;
  const int total = batch * 2 * chunk;
  CUtensorMap tq;
  CpMaps maps = {};
  if (!make_qkv_map(&tq, q, total, num_heads, q_stride_t, q_stride_h)) return NTB_ERR_ARG;
  for (int r = 0; r < cp; r++) {
    if ((k_ptrs[r] | v_ptrs[r]) & 15) return NTB_ERR_ARG;
    if (!make_qkv_map(&maps.k[r], reinterpret_cast<const void*>(k_ptrs[r]), total, num_kv_heads, kv_stride_t, kv_stride_h) ||
        !make_qkv_map(&maps.v[r], reinterpret_cast<const void*>(v_ptrs[r]), total, num_kv_heads, kv_stride_t, kv_stride_h))
      return NTB_ERR_ARG;
  }
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(flash_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FA_SMEM) != cudaSuccess) return NTB_ERR_LAUNCH;
    configured = true;
  }
  FwdParams p;
  p.num_heads = num_heads;
  p.num_kv_heads = num_kv_heads;
  p.causal = 1;
  p.window = 0;
  p.scale = softmax_scale;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.cu_q = nullptr;
  p.cu_k = nullptr;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.total_q = total;
  p.status = status;
  p.cp = cp;
  p.cp_me = me;
  p.cp_chunk = chunk;
  dim3 grid(2 * chunk / BM, num_heads, batch);
  flash_fwd_kernel<<<grid, FA_THREADS, FA_SMEM, stream>>>(tq, maps.k[me], maps.v[me], p, maps);
  return ntb_check_launch();
}
