// Flash attention forward on tcgen05 / TMEM (sm_100a), two query tiles per CTA: head dim 128, bf16, causal or full, sliding
// window, GQA, packed variable-length sequences (cu_seqlens); returns the log-sum-exp per (head, token).
//
// One CTA per (256 queries = two 128-row tiles, query head, sequence); all 512 TMEM columns: S0 | S1 | O0 | O1.
//   warp 0      TMA producer: both Q tiles once, then K / V tiles of 128 keys through rings (128-byte swizzle)
//   warp 1      MMA issuer, one elected thread.  Steady state per key tile j:
//                   O0 += P0(j) V(j);  S0 = Q0 K(j+1)^T;  O1 += P1(j) V(j);  S1 = Q1 K(j+1)^T
//               so while the softmax of one query tile runs, the tensor core works on the other tile.
//               P is the A operand FROM TENSOR MEMORY: the softmax warps overwrite part of S_t with the bf16 probabilities
//               (two per 32-bit column), so P never goes through shared memory and S_t / P_t share storage.
//               MMAs of one thread execute in issue order, which is what makes the reuse of S_t safe without a barrier:
//               S_t(j+1) is issued after the P_t(j) V(j) product that reads the same columns.
//   warps 2-17  softmax: warps 2-9 serve query tile 0, warps 10-17 tile 1; inside a tile two warps share 32 query rows (a TMEM
//               lane quarter), one per half of the key columns (64 scores each, read 32 at a time) and per half of O's columns.
//               In steady state there is NO row maximum: the exponentials are taken relative to the reference maximum of the
//               earlier tiles and the row sum (needed anyway) shows whether that was good enough; if not (a half row sums to
//               more than 1024, or is not finite) both warps of the rows compute the exact maximum (halves exchanged through
//               shared memory behind a two-arrival mbarrier with a bounded wait), rescale O and l, and recompute the tile: P is only stored
//               after that decision, so the scores can be read again.  The final O / l is exact either way.  P_t is stored
//               over columns 0-31 and 64-95 of S_t (each warp inside its own half).
//               `s_full[t]` firing also means P_t(j-1) V(j-1) has completed (a commit covers every earlier MMA of the thread),
//               so O_t may be rescaled as soon as S_t(j) can be read.
// Epilogue: O_t / l from TMEM straight to global memory (rows past the end of the sequence are not written), LSE to global.
// Tiles hanging over the end of a packed sequence read the next sequence's keys: those columns are masked.
// All barrier waits are bounded; a timeout raises `status` and the CTA unwinds.
#include <cstdlib>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace {

constexpr int HD = 128;
constexpr int BM = 128;  // queries per tile (two tiles per CTA)
constexpr int BN = 128;  // keys per tile
constexpr int K_STAGES = 2;
constexpr int V_STAGES = 2;
constexpr int TILE_BYTES = 128 * HD * 2;
constexpr int PANEL_BYTES = 128 * 64 * 2;
constexpr int F2_THREADS = 576;  // TMA warp, MMA warp, 16 softmax warps (two per 32 query rows of each tile)
constexpr int XCH_BYTES = 2 * 2 * 4 * 2 * 32 * 4 + 256;  // [slot][tile][quarter][half][lane] floats + flags
constexpr int F2_SMEM = TILE_BYTES * (2 + K_STAGES + V_STAGES) + 1024 + 256 + XCH_BYTES;
constexpr float SUM_LIMIT = 1024.f;  // a tile's row sum above this moves the reference maximum

struct Fwd2Params {
  int num_heads, num_kv_heads;
  int causal;
  int window;  // <= 0: none
  float scale_log2;
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
struct Cp2Maps {
  CUtensorMap k[CP_MAX];
  CUtensorMap v[CP_MAX];
};

__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]),
      "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]),
      "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
      "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait2() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[tmem] * B[smem]: the A operand (128 rows x 16 bf16 = 8 columns of 32 bits per instruction) is read from tensor memory.
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// packed fp32 pairs (one issue slot for two elements) and the three-input maximum
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
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// 2^x for a pair of arguments on the FMA / integer pipes (the special-function unit is the scarce resource of this kernel):
// n = round(x) by the magic-number addition, f = x - n in [-0.5, 0.5], degree-3 polynomial for 2^f (relative error 1e-4, well
// under the bf16 rounding of the probabilities), n added into the exponent field.
__device__ __forceinline__ void exp2_poly_pair(float y0, float y1, float& x0, float& x1) {
  y0 = fmaxf(y0, -126.f);
  y1 = fmaxf(y1, -126.f);
  const uint64_t y2 = pack2(y0, y1);
  const uint64_t t2 = add2(y2, pack2(12582912.f, 12582912.f));
  const uint64_t n2 = add2(t2, pack2(-12582912.f, -12582912.f));
  const uint64_t f2 = fma2(n2, pack2(-1.f, -1.f), y2);
  uint64_t p2 = fma2(pack2(0.05592203512787819f, 0.05592203512787819f), f2, pack2(0.24264007806777954f, 0.24264007806777954f));
  p2 = fma2(p2, f2, pack2(0.6931210160255432f, 0.6931210160255432f));
  p2 = fma2(p2, f2, pack2(0.9999244809150696f, 0.9999244809150696f));
  float t0, t1, p0, p1;
  unpack2(t2, t0, t1);
  unpack2(p2, p0, p1);
  x0 = __uint_as_float(__float_as_uint(p0) + (__float_as_uint(t0) << 23));
  x1 = __uint_as_float(__float_as_uint(p1) + (__float_as_uint(t1) << 23));
}

// POLY_PAIRS: of every four element pairs, how many take exp2_poly_pair instead of the special-function unit.
template <int POLY_PAIRS>
__global__ void __maxnreg__(96)
flash_fwd2_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                  const Fwd2Params p, const __grid_constant__ Cp2Maps cpm) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;  // two tiles
  uint8_t* sK = sQ + 2 * TILE_BYTES;
  uint8_t* sV = sK + K_STAGES * TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + V_STAGES * TILE_BYTES);
  uint64_t* q_full = bars;                      // [1]
  uint64_t* k_full = bars + 1;                  // [K_STAGES]
  uint64_t* k_empty = k_full + K_STAGES;        // [K_STAGES]
  uint64_t* v_full = k_empty + K_STAGES;        // [V_STAGES]
  uint64_t* v_empty = v_full + V_STAGES;        // [V_STAGES]
  uint64_t* s_full = v_empty + V_STAGES;        // [2] per query tile
  uint64_t* p_full = s_full + 2;                // [2]
  uint64_t* o_done = p_full + 2;                // [2]
  uint64_t* pair_sync = o_done + 2;             // [2 tiles][4 quarters]: the two warps that share 32 query rows
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pair_sync + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* xch = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 256);            // [2 slots][2][4][2][32]
  volatile int* xflag = reinterpret_cast<volatile int*>(xch + 2 * 2 * 4 * 2 * 32);          // [2 slots][2][4][2]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // grid: x = (sequence, head), y = query-tile pair.  Blocks are handed out x-fastest, so all (sequence, head) instances of the
  // heaviest pair start first and the light ones fill the tail
  const int b = blockIdx.x / p.num_heads, h = blockIdx.x % p.num_heads;
  // Context-parallel mode (p.cp > 0): the sequence is split in 2 * cp chunks and this rank holds chunks cp_me and 2 cp - 1 - cp_me
  // of every batch row, one after the other.  Keys / values stay with their owners (peer-mapped buffers, one tensor map per rank)
  // and are read tile by tile over NVLink by the TMA producer; masks use global positions.
  const bool cpm_on = p.cp > 0;
  const int q_begin = cpm_on ? b * 2 * p.cp_chunk : p.cu_q[b];
  const int q_len = cpm_on ? 2 * p.cp_chunk : p.cu_q[b + 1] - q_begin;
  const int k_begin = cpm_on ? 0 : p.cu_k[b];
  const int k_len = cpm_on ? 2 * p.cp * p.cp_chunk : p.cu_k[b + 1] - k_begin;
  // heavy (late) query tiles first: with a causal mask they have the most key tiles
  const int pair = static_cast<int>(gridDim.y) - 1 - static_cast<int>(blockIdx.y);
  const int q0 = pair * 2 * BM;
  if (q0 >= q_len) return;  // uniform for the CTA
  const int shift = cpm_on ? 0 : k_len - q_len;  // bottom-right aligned causal mask
  // position of a query tile's first row for the masks: the local one, or the global one under context parallelism
  auto mask_pos = [&](int qt) -> int {
    if (!cpm_on) return qt;
    const int half = qt / p.cp_chunk;
    const int chunk = half == 0 ? p.cp_me : 2 * p.cp - 1 - p.cp_me;
    return chunk * p.cp_chunk + (qt - half * p.cp_chunk);
  };
  // key range of the CTA: from the first key tile query tile 0 may see to the last one query tile 1 may see
  int kv_start = 0;
  if (p.window > 0) kv_start = max(0, (mask_pos(q0) + shift - p.window + 1) / BN * BN);
  auto tiles_of = [&](int t) -> int {
    const int qt = q0 + t * BM;
    int kv_end = k_len;
    if (p.causal) kv_end = min(k_len, mask_pos(qt) + BM + shift);
    return (qt < q_len && kv_end > kv_start) ? (kv_end - kv_start + BN - 1) / BN : 0;
  };
  const int n_t0 = tiles_of(0), n_t1 = tiles_of(1);
  const int n_max = max(n_t0, n_t1);
  const int hk = h / (p.num_heads / p.num_kv_heads);

  if (threadIdx.x == 0) {
    ptx::mbar_init(q_full, 1);
    for (int s = 0; s < K_STAGES; s++) {
      ptx::mbar_init(&k_full[s], 1);
      ptx::mbar_init(&k_empty[s], 1);
    }
    for (int s = 0; s < V_STAGES; s++) {
      ptx::mbar_init(&v_full[s], 1);
      ptx::mbar_init(&v_empty[s], 1);
    }
    for (int t = 0; t < 2; t++) {
      ptx::mbar_init(&s_full[t], 1);
      ptx::mbar_init(&p_full[t], 8);
      ptx::mbar_init(&o_done[t], 1);
      for (int q = 0; q < 4; q++) ptx::mbar_init(&pair_sync[t * 4 + q], 2);
    }
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
  // S_t at columns t * 128 (P_t aliases its first 64 columns), O_t at 256 + t * 128

  if (warp == 0) {
    if (ptx::elect_one() && n_max > 0) {
      const int q_tiles = n_t1 > 0 ? 2 : 1;  // tile 0 is valid whenever the CTA runs
      ptx::mbar_expect_tx(q_full, q_tiles * TILE_BYTES);
      for (int t = 0; t < q_tiles; t++) {
        ptx::tma_load_3d(sQ + t * TILE_BYTES, &tmap_q, q_full, 0, h, q_begin + q0 + t * BM);
        ptx::tma_load_3d(sQ + t * TILE_BYTES + PANEL_BYTES, &tmap_q, q_full, 64, h, q_begin + q0 + t * BM);
      }
      for (int j = 0; j < n_max; j++) {
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
        const int ks = j % K_STAGES, vs = j % V_STAGES;
        if (!ptx::mbar_wait(&k_empty[ks], ((j / K_STAGES) & 1) ^ 1, abort_flag)) break;
        ptx::mbar_expect_tx(&k_full[ks], TILE_BYTES);
        ptx::tma_load_3d(sK + ks * TILE_BYTES, mk, &k_full[ks], 0, hk, krow);
        ptx::tma_load_3d(sK + ks * TILE_BYTES + PANEL_BYTES, mk, &k_full[ks], 64, hk, krow);
        if (!ptx::mbar_wait(&v_empty[vs], ((j / V_STAGES) & 1) ^ 1, abort_flag)) break;
        ptx::mbar_expect_tx(&v_full[vs], TILE_BYTES);
        ptx::tma_load_3d(sV + vs * TILE_BYTES, mv, &v_full[vs], 0, hk, krow);
        ptx::tma_load_3d(sV + vs * TILE_BYTES + PANEL_BYTES, mv, &v_full[vs], 64, hk, krow);
      }
    }
  } else if (warp == 1) {
    if (ptx::elect_one() && n_max > 0) {
      constexpr uint32_t idesc_qk = ptx::make_idesc_bf16(BM, BN, false, false);
      constexpr uint32_t idesc_pv = ptx::make_idesc_bf16(BM, HD, false, true);
      bool ok = ptx::mbar_wait(q_full, 0, abort_flag);
      auto issue_qk = [&](int t, int j) -> bool {
        const int ks = j % K_STAGES;
        if (!ptx::mbar_wait(&k_full[ks], (j / K_STAGES) & 1, abort_flag)) return false;
        ptx::tc_fence_after();
        const uint32_t aQ = ptx::smem_u32(sQ + t * TILE_BYTES);
        const uint32_t aK = ptx::smem_u32(sK + ks * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < HD / 16; k++) {
          const uint32_t off = (k >> 2) * PANEL_BYTES + (k & 3) * 32;
          ptx::umma_f16(tmem_base + t * BN, ptx::make_smem_desc(aQ + off, 16, 1024), ptx::make_smem_desc(aK + off, 16, 1024), idesc_qk, k != 0);
        }
        ptx::umma_commit(&s_full[t]);
        return true;
      };
      auto issue_pv = [&](int t, int j) -> bool {
        const int vs = j % V_STAGES;
        if (!ptx::mbar_wait(&v_full[vs], (j / V_STAGES) & 1, abort_flag)) return false;
        if (!ptx::mbar_wait(&p_full[t], j & 1, abort_flag)) return false;
        ptx::tc_fence_after();
        const uint32_t aV = ptx::smem_u32(sV + vs * TILE_BYTES);
        const uint32_t tP = tmem_base + t * BN;
        const uint32_t tO = tmem_base + 256 + t * HD;
#pragma unroll
        for (int k = 0; k < BN / 16; k++) {
          const uint64_t bdesc = ptx::make_smem_desc(aV + k * 16 * 128, PANEL_BYTES, 1024);
          umma_f16_ts(tO, tP + (k < 4 ? k * 8 : 64 + (k - 4) * 8), bdesc, idesc_pv, (j | k) != 0);
        }
        if (j == (t ? n_t1 : n_t0) - 1) ptx::umma_commit(&o_done[t]);
        return true;
      };
      for (int t = 0; t < 2 && ok; t++)
        if ((t ? n_t1 : n_t0) > 0) ok = issue_qk(t, 0);
      if (ok) ptx::umma_commit(&k_empty[0]);
      for (int j = 0; j < n_max && ok; j++) {
        for (int t = 0; t < 2 && ok; t++) {
          const int nt = t ? n_t1 : n_t0;
          if (j < nt) ok = issue_pv(t, j);
          if (ok && j + 1 < nt) ok = issue_qk(t, j + 1);
        }
        if (!ok) break;
        ptx::umma_commit(&v_empty[j % V_STAGES]);
        if (j + 1 < n_max) ptx::umma_commit(&k_empty[(j + 1) % K_STAGES]);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax / correction / epilogue
    // warp -> (query tile t, half h of the key columns and of the head dim, TMEM lane quarter): two warps share 32 query rows
    const int t = (warp - 2) >> 3;
    const int hh = ((warp - 2) >> 2) & 1;
    const int n_tiles = t ? n_t1 : n_t0;
    if (n_tiles > 0) {
      const int quarter = warp & 3;            // TMEM lane quarter this warp may access
      const int r = quarter * 32 + lane;       // query row inside the tile
      const int qpos = q0 + t * BM + r;        // position inside the (local) sequence: validity and output row
      const int mpos = mask_pos(q0 + t * BM) + r;  // position used by the masks
      const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
      const uint32_t tS = tmem_base + lane_addr + t * BN + hh * 64;       // my 64 score columns; my P goes to their first 32
      const uint32_t tO = tmem_base + lane_addr + 256 + t * HD + hh * 64; // my 64 columns of O
      // Rendezvous of the two warps of these rows: an mbarrier with two arrivals and a bounded wait (a named barrier would hang
      // the partner if one warp gave up on a timeout).  Both warps take the same branches, so they count the same phases.
      uint64_t* pair_bar = &pair_sync[t * 4 + quarter];
      uint32_t pair_phase = 0;
      auto pair_rendezvous = [&]() -> bool {
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(pair_bar);
        const bool done = ptx::mbar_wait(pair_bar, pair_phase & 1, abort_flag);
        pair_phase++;
        return done;
      };
      auto xslot = [&](int slot, int half) -> float* { return xch + ((((slot * 2 + t) * 4 + quarter) * 2 + half) * 32) + lane; };
      auto fslot = [&](int slot, int half) -> volatile int* { return xflag + (((slot * 2 + t) * 4 + quarter) * 2 + half); };
      float m_ref = -INFINITY, l_run = 0.f;  // m_ref: the maximum the stored probabilities and O are relative to (same in both warps)
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; j++) {
        const int k0 = kv_start + j * BN + hh * 64;
        if (!ptx::mbar_wait(&s_full[t], j & 1, abort_flag)) { ok = false; break; }
        ptx::tc_fence_after();
        int hi = k_len - k0;
        if (p.causal) hi = min(hi, mpos + shift - k0 + 1);
        int lo = 0;
        if (p.window > 0) lo = max(0, mpos + shift - p.window + 1 - k0);
        const bool need_mask = (hi < 64) || (lo > 0);
        // one 32-column chunk of my half of the score row at a time (register budget: 18 warps share the register file)
        auto load_chunk = [&](int c, uint32_t (&v)[32]) {
          ptx::tmem_ld_32x32(tS + c * 32, v);
          ptx::tmem_ld_wait();
          if (need_mask) {
#pragma unroll
            for (int i = 0; i < 32; i++) {
              const int col = c * 32 + i;
              if (col < lo || col >= hi) v[i] = 0xff800000u;  // -inf: exp2 gives 0
            }
          }
        };
        // Fast path: exponentials relative to the reference maximum m_ref of the earlier tiles, no row maximum at all.  The row
        // sum (needed anyway) tells whether that was good enough: if some row of either warp sums to more than SUM_LIMIT (or is
        // not finite), both warps take the slow path once for this tile: exact row maximum (scores read again: P is only
        // stored after the decision; the two halves exchanged through shared memory), new reference, O and l rescaled,
        // exponentials recomputed.  The result is exact either way.
        float alpha = 1.f, sum = 0.f;
        uint32_t pk[2][16];
        bool slow = (j == 0) || __any_sync(0xffffffffu, m_ref == -INFINITY);
#pragma unroll 1
        for (int attempt = 0; attempt < 2; attempt++) {
          if (slow) {
            float mine = -INFINITY;
#pragma unroll 1
            for (int c = 0; c < 2; c++) {
              uint32_t v[32];
              load_chunk(c, v);
              float m0 = fmaxf(__uint_as_float(v[0]), __uint_as_float(v[1])), m1 = fmaxf(__uint_as_float(v[2]), __uint_as_float(v[3]));
#pragma unroll
              for (int i = 4; i < 32; i += 4) {
                m0 = max3(m0, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
                m1 = max3(m1, __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
              }
              mine = max3(mine, m0, m1);
            }
            *xslot(j & 1, hh) = mine;
            if (!pair_rendezvous()) { ok = false; break; }
            const float m_new = fmaxf(m_ref, fmaxf(mine, *xslot(j & 1, hh ^ 1)));
            const float m_fin = (m_new == -INFINITY) ? 0.f : m_new;
            alpha = (m_ref == -INFINITY) ? 0.f : ex2((m_ref - m_fin) * p.scale_log2);
            if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
              // my half of O_t holds the sum over earlier tiles relative to the old reference (its last P*V completed before S_t(j))
#pragma unroll 1
              for (int c = 0; c < 2; c++) {
                uint32_t o[32];
                ptx::tmem_ld_32x32(tO + c * 32, o);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                tmem_st_32x32b(tO + c * 32, o);
              }
            }
            m_ref = m_new;
          }
          const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
          const float neg_m = -m_use * p.scale_log2;
          const uint64_t sl2 = pack2(p.scale_log2, p.scale_log2), nm2 = pack2(neg_m, neg_m);
          uint64_t acc2[2];
#pragma unroll
          for (int c = 0; c < 2; c++) {
            uint32_t v[32];
            load_chunk(c, v);
            acc2[c] = 0ull;
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              float y0, y1;
              unpack2(fma2(pack2(__uint_as_float(v[i]), __uint_as_float(v[i + 1])), sl2, nm2), y0, y1);
              float x0, x1;
              if (((i >> 1) & 3) < POLY_PAIRS) {
                exp2_poly_pair(y0, y1, x0, x1);
              } else {
                x0 = ex2(y0);
                x1 = ex2(y1);
              }
              acc2[c] = add2(acc2[c], pack2(x0, x1));
              __nv_bfloat162 hb = __floats2bfloat162_rn(x0, x1);
              pk[c][i >> 1] = *reinterpret_cast<uint32_t*>(&hb);
            }
          }
          float s0, s1, s2, s3;
          unpack2(acc2[0], s0, s1);
          unpack2(acc2[1], s2, s3);
          sum = (s0 + s1) + (s2 + s3);
          if (slow) break;
          // both warps of these rows must take the same decision
          const bool bad = __any_sync(0xffffffffu, !(sum <= SUM_LIMIT));
          if (lane == 0) *fslot(j & 1, hh) = bad ? 1 : 0;
          if (!pair_rendezvous()) { ok = false; break; }
          if (!(bad || *fslot(j & 1, hh ^ 1) != 0)) break;
          slow = true;
        }
        if (!ok) break;
        // the scores are not needed any more: P over the first 32 columns of my half
        tmem_st_32x16(tS, pk[0]);
        tmem_st_32x16(tS + 16, pk[1]);
        tmem_st_wait2();
        l_run = l_run * alpha + sum;
        // my half of P written (and of O rescaled): tell the MMA warp
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&p_full[t]);
      }
      // ---------------------------------------------------------------- epilogue: my 64 columns of O
      if (ok && ptx::mbar_wait(&o_done[t], 0, abort_flag)) {
        ptx::tc_fence_after();
        *xslot(n_tiles & 1, hh) = l_run;
        const bool met = pair_rendezvous();
        const float l_tot = l_run + *xslot(n_tiles & 1, hh ^ 1);
        const float inv_l = l_tot > 0.f ? 1.f / l_tot : 0.f;
        const bool valid = met && qpos < q_len;
        const int64_t tok = static_cast<int64_t>(q_begin) + qpos;
        __nv_bfloat16* orow = p.out + (tok * p.num_heads + h) * HD + hh * 64;
#pragma unroll 1
        for (int c = 0; c < 2; c++) {
          uint32_t v[32];
          ptx::tmem_ld_32x32(tO + c * 32, v);
          ptx::tmem_ld_wait();
          if (valid) {
#pragma unroll
            for (int u = 0; u < 4; u++) {
              uint4 o4;
              __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(v[u * 8 + 0]) * inv_l, __uint_as_float(v[u * 8 + 1]) * inv_l);
              __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(v[u * 8 + 2]) * inv_l, __uint_as_float(v[u * 8 + 3]) * inv_l);
              __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(v[u * 8 + 4]) * inv_l, __uint_as_float(v[u * 8 + 5]) * inv_l);
              __nv_bfloat162 h3 = __floats2bfloat162_rn(__uint_as_float(v[u * 8 + 6]) * inv_l, __uint_as_float(v[u * 8 + 7]) * inv_l);
              o4.x = *reinterpret_cast<uint32_t*>(&h0); o4.y = *reinterpret_cast<uint32_t*>(&h1);
              o4.z = *reinterpret_cast<uint32_t*>(&h2); o4.w = *reinterpret_cast<uint32_t*>(&h3);
              *reinterpret_cast<uint4*>(orow + c * 32 + u * 8) = o4;
            }
          }
        }
        if (valid && hh == 0) p.lse[static_cast<int64_t>(h) * p.total_q + tok] = (l_tot > 0.f) ? m_ref * p.scale + logf(l_tot) : -INFINITY;
      }
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

typedef CUresult (*EncodeTiledFn2)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn2 f2_get_encode() {
  ntb_bind_context_to_thread();
  static EncodeTiledFn2 fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn2>(ptr);
  }
  return fn;
}

// [tokens, heads, 128] bf16 with element strides (stride_t, stride_h, 1): 3-D map {128, heads, tokens}, box {64, 1, 128}.
bool f2_make_map(CUtensorMap* m, const void* ptr, int64_t tokens, int heads, int64_t stride_t, int64_t stride_h) {
  cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)heads, (cuuint64_t)tokens};
  cuuint64_t strides[2] = {(cuuint64_t)stride_h * 2, (cuuint64_t)stride_t * 2};
  cuuint32_t box[3] = {64, 1, 128};
  cuuint32_t es[3] = {1, 1, 1};
  return f2_get_encode()(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int f2_launch(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const Fwd2Params& p, const Cp2Maps& maps, dim3 grid, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(flash_fwd2_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, F2_SMEM) != cudaSuccess) return NTB_ERR_LAUNCH;
    configured = true;
  }
  if (grid.y > 65535) return NTB_ERR_ARG;
  flash_fwd2_kernel<0><<<grid, F2_THREADS, F2_SMEM, stream>>>(tq, tk, tv, p, maps);
  return ntb_check_launch();
}

}  // namespace

// Same contract as ntb_flash_attn_fwd.  q: [total_q, Hq, 128], k/v: [total_k, Hkv, 128] bf16 (token / head strides in elements,
// last dim contiguous); out: [total_q, Hq, 128] contiguous; lse: fp32 [Hq, total_q]; cu_q / cu_k: int32 [batch + 1] on the device.
NTB_EXPORT int ntb_flash_attn_fwd2(const void* q, const void* k, const void* v, void* out, float* lse, const int* cu_q, const int* cu_k, int batch,
                                   int max_seqlen_q, int total_q, int total_k, int num_heads, int num_kv_heads, int64_t q_stride_t, int64_t q_stride_h,
                                   int64_t k_stride_t, int64_t k_stride_h, int64_t v_stride_t, int64_t v_stride_h, float softmax_scale, int causal, int window,
                                   int* status, cudaStream_t stream) {
  if (!f2_get_encode() || batch <= 0 || total_q <= 0 || total_k <= 0 || num_heads % num_kv_heads) return NTB_ERR_ARG;
  if ((q_stride_t | q_stride_h | k_stride_t | k_stride_h | v_stride_t | v_stride_h) % 8) return NTB_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(out)) & 15) return NTB_ERR_ARG;
  CUtensorMap tq, tk, tv;
  if (!f2_make_map(&tq, q, total_q, num_heads, q_stride_t, q_stride_h) || !f2_make_map(&tk, k, total_k, num_kv_heads, k_stride_t, k_stride_h) ||
      !f2_make_map(&tv, v, total_k, num_kv_heads, v_stride_t, v_stride_h))
    return NTB_ERR_ARG;
  Fwd2Params p;
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
  static const Cp2Maps no_cp = {};
  return f2_launch(tq, tk, tv, p, no_cp, dim3(num_heads * batch, (max_seqlen_q + 2 * BM - 1) / (2 * BM), 1), stream);
}

// Context-parallel forward.  q: this rank's [batch * 2 * chunk, Hq, 128] (chunk r then chunk 2 cp - 1 - r of every batch row);
// k_ptrs / v_ptrs: device addresses of every rank's [batch * 2 * chunk, Hkv, 128] K and V (peer-mapped, same strides everywhere,
// filled and made visible by a cross-rank barrier before this launch).  Causal only.  out / lse as in ntb_flash_attn_fwd2.
NTB_EXPORT int ntb_flash_attn_fwd2_cp(const void* q, const uint64_t* k_ptrs, const uint64_t* v_ptrs, void* out, float* lse, int batch, int chunk, int cp, int me,
                                      int num_heads, int num_kv_heads, int64_t q_stride_t, int64_t q_stride_h, int64_t kv_stride_t, int64_t kv_stride_h,
                                      float softmax_scale, int* status, cudaStream_t stream) {
  if (!f2_get_encode() || batch <= 0 || chunk <= 0 || chunk % BM || cp < 1 || cp > CP_MAX || me < 0 || me >= cp || num_heads % num_kv_heads) return NTB_ERR_ARG;
  if ((q_stride_t | q_stride_h | kv_stride_t | kv_stride_h) % 8) return NTB_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out)) & 15) return NTB_ERR_ARG;
  const int total = batch * 2 * chunk;
  CUtensorMap tq;
  Cp2Maps maps = {};
  if (!f2_make_map(&tq, q, total, num_heads, q_stride_t, q_stride_h)) return NTB_ERR_ARG;
  for (int r = 0; r < cp; r++) {
    if ((k_ptrs[r] | v_ptrs[r]) & 15) return NTB_ERR_ARG;
    if (!f2_make_map(&maps.k[r], reinterpret_cast<const void*>(k_ptrs[r]), total, num_kv_heads, kv_stride_t, kv_stride_h) ||
        !f2_make_map(&maps.v[r], reinterpret_cast<const void*>(v_ptrs[r]), total, num_kv_heads, kv_stride_t, kv_stride_h))
      return NTB_ERR_ARG;
  }
  Fwd2Params p;
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
  return f2_launch(tq, maps.k[me], maps.v[me], p, maps, dim3(num_heads * batch, (2 * chunk + 2 * BM - 1) / (2 * BM), 1), stream);
}
