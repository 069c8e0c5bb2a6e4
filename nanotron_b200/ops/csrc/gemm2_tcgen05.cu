// bf16 GEMM on CTA pairs (tcgen05 cta_group::2 + TMEM + TMA), persistent and warp-specialised (sm_100a).
//
//   D[M,N] (=|+=) sum_k A(m,k) * B(n,k)          same operand-storage and output conventions as gemm_tcgen05.cu
//
// Two CTAs of a cluster (one per SM of a pair) work on one 256 x 256 output tile.  Each CTA keeps in its own shared memory the
// 128 rows of A that it owns and HALF of the B tile (128 of the 256 output columns); one thread of the leader CTA issues
// tcgen05.mma.cta_group::2 (256 x 256 x 16), the hardware reads both halves of B for both SMs, and each CTA's TMEM receives its
// 128 rows x 256 columns of accumulators.  Per MMA each SM reads 8 KB of operands instead of the 12 KB of the one-CTA 128 x 256
// tile, and its shared memory holds 32 KB per stage instead of 48, so six stages fit.
//
// Warp roles per CTA: warp 0 TMA producer (own A rows + own half of B into the CTA's own shared memory; the loads are the
// cta_group::2 form of cp.async.bulk.tensor, whose completion bytes are counted on the LEADER's stage barrier, so the leader's MMA
// thread waits on one barrier for both halves); warp 1: the MMA issuer in the leader, idle in the peer; warps 2..5 epilogue
// (tcgen05.ld -> swizzled staging -> TMA store / reduce-add of the CTA's own rows).
// Cross-CTA signals besides the loads are plain remote mbarrier arrives: the leader's producer forwards every "stage free" to the
// peer's producer, one leader epilogue warp forwards "accumulator ready" to the peer's epilogue, and the peer's epilogue warps hand
// accumulators back to the leader's MMA thread.  All waits are bounded; the two CTAs meet in a cluster barrier before TMEM is freed.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace {

constexpr int P_BLOCK_M = 128;   // rows per CTA (256 per pair)
constexpr int P_BLOCK_N = 256;   // columns per pair; each CTA stages 128 of them
constexpr int P_HALF_N = 128;
constexpr int P_BLOCK_K = 64;
constexpr int P_UMMA_K = 16;
constexpr int P_MAX_STAGES = 6;
constexpr int P_A_BYTES = P_BLOCK_M * P_BLOCK_K * 2;  // 16 KiB
constexpr int P_B_BYTES = P_HALF_N * P_BLOCK_K * 2;   // 16 KiB
constexpr int P_STAGE_BYTES = P_A_BYTES + P_B_BYTES;
constexpr int P_EPI_WARPS = 4;
constexpr int P_EPI_BUF = 32 * 128;
constexpr int P_EPI_BYTES = P_EPI_WARPS * 2 * P_EPI_BUF;
constexpr int P_THREADS = 32 * (2 + P_EPI_WARPS);
constexpr int P_SMEM = P_MAX_STAGES * P_STAGE_BYTES + P_EPI_BYTES + 1024 + 512;

enum POut { P_OUT_BF16 = 0, P_OUT_F32 = 1, P_OUT_F32_ACCUM = 2, P_OUT_PEER_BF16 = 3 };

// Tensor-parallel fusion on the pair kernel (same protocol as the one-CTA kernel in gemm_tcgen05.cu; all off when world == 0):
//  * all-gather -> GEMM: A is a gathered buffer of `world` row blocks of `ag_rows` rows that peers fill with plain stores;
//    block r is valid once ag_flags[r] >= epoch.  Each CTA's TMA producer polls the word of the block its 128 rows belong to
//    (bounded) before its first load from it; tile rows are visited starting with this rank's own block.
//  * GEMM -> reduce-scatter (P_OUT_PEER_BF16): the epilogue TMA-stores every bf16 chunk into slot `me` of the staging area of the
//    rank that owns those rows (one tensor map per owner); the last CTA of the grid to finish raises rs_flags[owner][me] everywhere.
constexpr int P_TP_MAX = 8;
struct PFuse {
  int world = 0, me = 0;
  uint32_t epoch = 0;
  int m_rot = 0;                        // rotation of the tile rows, in 256-row pair tiles
  const uint32_t* ag_flags = nullptr;   // local flag words [world]
  int ag_rows = 0;                      // rows per gathered block (multiple of 128)
  int ag_local = 0;                     // 1: this rank's own block is read through tmap_al (its source tensor) and needs no flag
  uint32_t* rs_flags[P_TP_MAX] = {};    // per-owner flag words [world]
  int rs_rows = 0;                      // rows per owner (multiple of 32)
  unsigned int* done_counter = nullptr; // local counter, zero before launch
};
struct PPeerMaps {
  CUtensorMap m[P_TP_MAX];
};

// Work units of a launch.  Tiles are dealt to the CTA pairs round robin; when the last round would leave most pairs idle, the
// tiles of that round are cut along K into `split` chunks each, one unit per chunk, so the tail of the launch is shared by all
// pairs.  A chunk stores its fp32 partial sums into a slab of its own in a workspace (no zero fill, no atomics); a small pass
// then sums the slabs of a tile in chunk order and writes D (bf16 / fp32 store, or fp32 accumulate), so the result does not
// depend on which chunk finished first.
struct PSched {
  int total_units = 0;  // grid-stride loop bound
  int full_units = 0;   // units [0, full_units) are whole tiles with the same index
  int split = 1;        // chunks per tile of the last round (1: nothing is split)
  int kb_per = 0;       // k-blocks per chunk
};
struct PUnit {
  int tile, kb0, kbs, ws;  // ws: workspace slab of this chunk (unit index within the last round), -1 for a whole tile
};
__device__ __forceinline__ PUnit decode_unit(int u, const PSched& sc, int k_blocks) {
  if (u < sc.full_units || sc.split <= 1) return {u, 0, k_blocks, -1};
  const int v = u - sc.full_units;
  const int rt = v / sc.split, ch = v - rt * sc.split;
  const int kb0 = ch * sc.kb_per;
  return {sc.full_units + rt, kb0, min(sc.kb_per, k_blocks - kb0), v};
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cta address of this CTA -> shared::cluster address of the same location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(local_addr), "r"(rank));
  return a;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Forwarding a hardware completion (nothing this thread wrote has to become visible): no release fence on the hot path.
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ptx::smem_u32(smem_dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma2_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive on the barrier at shared::cluster address `addr` once every tcgen05.mma issued so far by this thread has completed
__device__ __forceinline__ void umma2_commit(uint32_t addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(addr) : "memory");
}

// Tiled loads whose mbarrier may live in the other CTA of the pair (`bar_cluster_addr` is a shared::cluster address).
__device__ __forceinline__ void tma2_load_2d(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(ptx::smem_u32(smem_dst)),
               "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma2_load_3d(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(ptx::smem_u32(smem_dst)),
               "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z)
               : "memory");
}

struct PTile {
  int m_blk, n_blk;  // in units of 256 x 256 pair tiles
};
// Tiles are visited column by column inside bands of `BAND` tile rows: the band's rows of A stay in L2 while B streams through
// once per band.  The host picks the band so that its A rows take about a third of L2, i.e. B is re-read as rarely as possible.
__device__ __forceinline__ PTile pair_tile(int t, int tiles_m, int tiles_n, int BAND) {
  const int band_size = BAND * tiles_n;
  const int band = t / band_size;
  const int first_m = band * BAND;
  const int rows = min(BAND, tiles_m - first_m);
  const int r = t - band * band_size;
  return {first_m + r % rows, r / rows};
}

template <bool A_MN, bool B_MN, int OUT, int P_STAGES>
__global__ void __launch_bounds__(P_THREADS, 1)
gemm2_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const __grid_constant__ CUtensorMap tmap_d,
                     int M, int N, int K, int band, int* __restrict__ status, const __grid_constant__ PFuse fuse, const __grid_constant__ PPeerMaps pmaps,
                     const __grid_constant__ PSched sched, const __grid_constant__ CUtensorMap tmap_ws, const __grid_constant__ CUtensorMap tmap_al) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_smem = smem + P_MAX_STAGES * P_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + P_EPI_BYTES);
  uint64_t* full_bar = bars;                       // [STAGES]  (leader) both CTAs' loads of the stage have landed
  uint64_t* empty_bar = bars + 2 * P_MAX_STAGES;       // [STAGES]  the MMAs that read this stage are done
  uint64_t* tmem_full = bars + 3 * P_MAX_STAGES;       // [2]
  uint64_t* tmem_empty = tmem_full + 2;            // [2]  (leader) both CTAs' epilogues have drained the accumulator
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();  // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int tiles_m = (M + 2 * P_BLOCK_M - 1) / (2 * P_BLOCK_M);
  const int tiles_n = (N + P_BLOCK_N - 1) / P_BLOCK_N;
  const int k_blocks = (K + P_BLOCK_K - 1) / P_BLOCK_K;

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; s++) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; b++) {
      ptx::mbar_init(&tmem_full[b], 1);  // leader: the MMA commit; peer: the remote arrive that forwards it
      ptx::mbar_init(&tmem_empty[b], 2 * P_EPI_WARPS);
    }
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tmap(&tmap_a);
    ptx::prefetch_tmap(&tmap_b);
    ptx::prefetch_tmap(&tmap_d);
  }
  if (warp == 1) {
    tmem_alloc2(tmem_base_slot, 512);
    tmem_relinquish2();
  }
  ptx::tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before any remote arrive or commit can reach them
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (ptx::elect_one()) {
      int it = 0;
      bool ok = true;
      uint32_t ag_ready = 0;
      for (int u = pair; u < sched.total_units && ok; u += num_pairs) {
        const PUnit un = decode_unit(u, sched, k_blocks);
        if (un.kbs <= 0) continue;
        PTile tc = pair_tile(un.tile, tiles_m, tiles_n, band);
        tc.m_blk = (tc.m_blk + fuse.m_rot) % tiles_m;
        const int m0 = (tc.m_blk * 2 + static_cast<int>(cta)) * P_BLOCK_M;           // this CTA's rows of A
        const int n0 = tc.n_blk * P_BLOCK_N + static_cast<int>(cta) * P_HALF_N;      // this CTA's half of B
        bool a_local = false;
        if (fuse.ag_flags != nullptr && m0 < M) {
          const int src = min(fuse.world - 1, m0 / fuse.ag_rows);  // ag_rows is a multiple of 128: one source per CTA row block
          if (fuse.ag_local && src == fuse.me) {
            a_local = true;  // own rows come straight from the tensor they were pushed from: nothing to wait for
          } else if (!(ag_ready & (1u << src))) {
            const uint64_t t0 = ptx::globaltimer();
            while (true) {
              uint32_t v;
              asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(fuse.ag_flags + src) : "memory");
              if (static_cast<int32_t>(v - fuse.epoch) >= 0) { ag_ready |= 1u << src; break; }
              if (*abort_flag || ptx::globaltimer() - t0 > NTB_WAIT_LIMIT_NS) { *abort_flag = 1; ok = false; break; }
              __nanosleep(100);
            }
            if (!ok) break;
            // the block was written by peers with generic stores: make it visible to the async (TMA) proxy
            asm volatile("fence.proxy.async.global;" ::: "memory");
          }
        }
        for (int kb = un.kb0; kb < un.kb0 + un.kbs; kb++, it++) {
          const int s = it % P_STAGES;
          const uint32_t ph = (it / P_STAGES) & 1;
          if (!ptx::mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, 200)) { ok = false; break; }
          uint8_t* sa = smem + s * P_STAGE_BYTES;
          uint8_t* sb = sa + P_A_BYTES;
          if (cta == 0) {
            // the stage is free in both CTAs (the MMAs that read it are complete): tell the peer's producer, then expect both halves
            if (it >= P_STAGES) mbar_arrive_cluster_relaxed(map_to_cta(ptx::smem_u32(&empty_bar[s]), 1));
            ptx::mbar_expect_tx(&full_bar[s], 2 * P_STAGE_BYTES);
          }
          const uint32_t fb = map_to_cta(ptx::smem_u32(&full_bar[s]), 0);  // bytes of both CTAs are counted on the leader's barrier
          if (A_MN) tma2_load_3d(sa, &tmap_a, fb, 0, kb * P_BLOCK_K, m0 / 64);
          else if (a_local) tma2_load_2d(sa, &tmap_al, fb, kb * P_BLOCK_K, m0 - fuse.me * fuse.ag_rows);
          else      tma2_load_2d(sa, &tmap_a, fb, kb * P_BLOCK_K, m0);
          if (B_MN) tma2_load_3d(sb, &tmap_b, fb, 0, kb * P_BLOCK_K, n0 / 64);
          else      tma2_load_2d(sb, &tmap_b, fb, kb * P_BLOCK_K, n0);
        }
      }
      if (!ok && cta == 1) {
        // this CTA's loads in flight are counted on the leader's barrier: give them time to land before the shared memory goes away
        const uint64_t t0 = ptx::globaltimer();
        while (ptx::globaltimer() - t0 < 100000ull) {}
      }
      if (!ok && cta == 0) {
        const uint64_t t0 = ptx::globaltimer();
        for (int s = 0; s < P_STAGES; s++) {
          const int last = it - 1 - ((it - 1 - s) % P_STAGES + P_STAGES) % P_STAGES;
          if (it == 0 || last < 0) continue;
          const uint32_t ph = (last / P_STAGES) & 1;
          while (!ptx::mbar_try_wait(&full_bar[s], ph) && ptx::globaltimer() - t0 < NTB_WAIT_LIMIT_NS) {}
        }
      }
    }
  } else if (warp == 1) {
    if (ptx::elect_one()) {
      if (cta == 0) {
        // ---------------------------------------------------------------- MMA issuer (leader)
        constexpr uint32_t idesc = ptx::make_idesc_bf16(2 * P_BLOCK_M, P_BLOCK_N, A_MN, B_MN);
        int it = 0, tile_it = 0;
        bool ok = true;
        for (int u = pair; u < sched.total_units && ok; u += num_pairs) {
          const PUnit un = decode_unit(u, sched, k_blocks);
          if (un.kbs <= 0) continue;
          const int acc = tile_it & 1;
          const uint32_t acc_ph = (tile_it >> 1) & 1;
          tile_it++;
          if (!ptx::mbar_wait(&tmem_empty[acc], acc_ph ^ 1, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t tmem_d = tmem_base + acc * P_BLOCK_N;
          for (int kb = 0; kb < un.kbs; kb++, it++) {
            const int s = it % P_STAGES;
            const uint32_t ph = (it / P_STAGES) & 1;
            if (!ptx::mbar_wait(&full_bar[s], ph, abort_flag)) { ok = false; break; }
            ptx::tc_fence_after();
            const uint32_t sa = ptx::smem_u32(smem + s * P_STAGE_BYTES);
            const uint32_t sb = sa + P_A_BYTES;
#pragma unroll
            for (int k = 0; k < P_BLOCK_K / P_UMMA_K; k++) {
              const uint64_t adesc = A_MN ? ptx::make_smem_desc(sa + k * P_UMMA_K * 128, P_BLOCK_K * 128, 1024) : ptx::make_smem_desc(sa + k * P_UMMA_K * 2, 16, 1024);
              const uint64_t bdesc = B_MN ? ptx::make_smem_desc(sb + k * P_UMMA_K * 128, P_BLOCK_K * 128, 1024) : ptx::make_smem_desc(sb + k * P_UMMA_K * 2, 16, 1024);
              umma2_f16(tmem_d, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
            }
            umma2_commit(ptx::smem_u32(&empty_bar[s]));  // the stage is free once these MMAs (in both SMs) have read it
          }
          if (ok) umma2_commit(ptx::smem_u32(&tmem_full[acc]));
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps (both CTAs, own 128 rows)
    const int q = warp & 3;
    uint8_t* my_epi = epi_smem + (warp - 2) * 2 * P_EPI_BUF;
    constexpr bool BF16_OUT = (OUT == P_OUT_BF16 || OUT == P_OUT_PEER_BF16);
    int tile_it = 0, buf = 0;
    bool ok = true;
    for (int u = pair; u < sched.total_units && ok; u += num_pairs) {
      const PUnit un = decode_unit(u, sched, k_blocks);
      if (un.kbs <= 0) continue;
      PTile tc = pair_tile(un.tile, tiles_m, tiles_n, band);
      tc.m_blk = (tc.m_blk + fuse.m_rot) % tiles_m;
      const int acc = tile_it & 1;
      const uint32_t acc_ph = (tile_it >> 1) & 1;
      tile_it++;
      // a chunk of a split tile leaves as fp32 partial sums in its workspace slab, whatever the type of D
      const bool to_ws = un.ws >= 0;
      const bool bf16_path = BF16_OUT && !to_ws;
      const int CHUNK_COLS = bf16_path ? 64 : 32;
      const int CHUNKS = P_BLOCK_N / CHUNK_COLS;
      if (!ptx::mbar_wait(&tmem_full[acc], acc_ph, abort_flag, 1000)) { ok = false; break; }
      if (cta == 0 && warp == 2 && lane == 0) mbar_arrive_cluster(map_to_cta(ptx::smem_u32(&tmem_full[acc]), 1));  // forward to the peer's epilogue
      ptx::tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * P_BLOCK_N;
      const int row0 = (tc.m_blk * 2 + static_cast<int>(cta)) * P_BLOCK_M + q * 32;
#pragma unroll 1
      for (int c = 0; c < CHUNKS; c++) {
        uint8_t* stage_buf = my_epi + buf * P_EPI_BUF;
        if (lane == 0) ptx::tma_wait_group_read<1>();
        __syncwarp();
        uint8_t* my_row = stage_buf + lane * 128;
        if (bf16_path) {
          uint32_t r0[32], r1[32];
          ptx::tmem_ld_32x32(taddr + c * 64, r0);
          ptx::tmem_ld_32x32(taddr + c * 64 + 32, r1);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; j++) {
            const uint32_t* src = (j < 4) ? &r0[j * 8] : &r1[(j - 4) * 8];
            uint4 pk;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(src[0]), __uint_as_float(src[1]));
            __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(src[2]), __uint_as_float(src[3]));
            __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(src[4]), __uint_as_float(src[5]));
            __nv_bfloat162 h3 = __floats2bfloat162_rn(__uint_as_float(src[6]), __uint_as_float(src[7]));
            pk.x = *reinterpret_cast<uint32_t*>(&h0);
            pk.y = *reinterpret_cast<uint32_t*>(&h1);
            pk.z = *reinterpret_cast<uint32_t*>(&h2);
            pk.w = *reinterpret_cast<uint32_t*>(&h3);
            *reinterpret_cast<uint4*>(my_row + ((j ^ (lane & 7)) << 4)) = pk;
          }
        } else {
          uint32_t r0[32];
          ptx::tmem_ld_32x32(taddr + c * 32, r0);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; j++) {
            uint4 pk = make_uint4(r0[j * 4], r0[j * 4 + 1], r0[j * 4 + 2], r0[j * 4 + 3]);
            *reinterpret_cast<uint4*>(my_row + ((j ^ (lane & 7)) << 4)) = pk;
          }
        }
        ptx::fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          const int x = tc.n_blk * P_BLOCK_N + c * CHUNK_COLS;
          if (to_ws) {
            ptx::tma_store_2d(&tmap_ws, stage_buf, c * 32, un.ws * (2 * P_BLOCK_M) + static_cast<int>(cta) * P_BLOCK_M + q * 32);
          } else if (x < N && row0 < M) {
            if (OUT == P_OUT_PEER_BF16) {
              const int owner = row0 / fuse.rs_rows;  // rs_rows is a multiple of 32: the 32 rows of this warp share an owner
              ptx::tma_store_2d(&pmaps.m[owner], stage_buf, x, fuse.me * fuse.rs_rows + (row0 - owner * fuse.rs_rows));
            } else if (OUT == P_OUT_F32_ACCUM) ptx::tma_reduce_add_2d(&tmap_d, stage_buf, x, row0);
            else ptx::tma_store_2d(&tmap_d, stage_buf, x, row0);
          }
          ptx::tma_commit_group();
        }
        buf ^= 1;
      }
      // accumulator fully read: hand it back to the leader's MMA thread (a remote arrive from the peer CTA)
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (cta == 0) ptx::mbar_arrive(&tmem_empty[acc]);
        else mbar_arrive_cluster(map_to_cta(ptx::smem_u32(&tmem_empty[acc]), 0));
      }
    }
    if (lane == 0) {
      ptx::tma_wait_group<0>();
      if (OUT == P_OUT_PEER_BF16) {
        // the peer stores were made by the async proxy: order them before the generic-proxy flag store that follows the CTA barrier
        asm volatile("fence.proxy.async.global;" ::: "memory");
        __threadfence_system();
      }
    }
    __syncwarp();
  }

  ptx::tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the leader's MMAs write the peer's TMEM and read its shared memory: nobody leaves or frees before both are done
  if (warp == 1) {
    ptx::tc_fence_after();
    tmem_dealloc2(tmem_base, 512);
  }
  if (OUT == P_OUT_PEER_BF16 && fuse.done_counter != nullptr && threadIdx.x == 0) {
    // every store of this CTA is complete and fenced (epilogue warps, before the barrier above); the last CTA of the grid to get
    // here tells every owner that this rank's partial sums are in place
    __threadfence_system();
    const unsigned int prev = atomicAdd(fuse.done_counter, 1u);
    if (prev == gridDim.x - 1) {
      __threadfence_system();
      for (int r = 0; r < fuse.world; r++)
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(fuse.rs_flags[r] + fuse.me), "r"(fuse.epoch) : "memory");
      *fuse.done_counter = 0;
    }
  }
  if (threadIdx.x == 0 && *abort_flag && status) atomicExch(status, NTB_ERR_TIMEOUT);
}

// Split tiles: D tile = (D tile +) the sum, in chunk order, of the tile's workspace slabs (256 x 256 fp32 each, complete once the
// GEMM kernel has finished).  One block per split tile and 32-row group.  OUT as in the GEMM kernel.
template <int OUT>
__global__ void gemm2_split_fixup_kernel(const float* __restrict__ ws, void* __restrict__ d_, int64_t ldd, int M, int N, int k_blocks, PSched sched, int tiles_m,
                                         int tiles_n, int band, int m_rot) {
  const int rt = blockIdx.x >> 3, rg = blockIdx.x & 7;
  PTile tc = pair_tile(sched.full_units + rt, tiles_m, tiles_n, band);
  tc.m_blk = (tc.m_blk + m_rot) % tiles_m;
  const int chunks = min(sched.split, (k_blocks + sched.kb_per - 1) / sched.kb_per);  // chunks past the end of K wrote nothing
  const int64_t slab = static_cast<int64_t>(2 * P_BLOCK_M) * P_BLOCK_N;
  const float* src = ws + static_cast<int64_t>(rt) * sched.split * slab + static_cast<int64_t>(rg) * 32 * P_BLOCK_N;
  for (int i = threadIdx.x; i < 32 * P_BLOCK_N / 8; i += blockDim.x) {
    const int r = i / (P_BLOCK_N / 8), c8 = (i % (P_BLOCK_N / 8)) * 8;
    const int row = tc.m_blk * 2 * P_BLOCK_M + rg * 32 + r, col = tc.n_blk * P_BLOCK_N + c8;
    if (row >= M || col >= N) continue;  // N is a multiple of 8 and rows of D start 16-byte aligned (checked by the host)
    float f[8];
    if (OUT == P_OUT_F32_ACCUM) {
      const float* dp = reinterpret_cast<const float*>(d_) + static_cast<int64_t>(row) * ldd + col;
      *reinterpret_cast<float4*>(f) = *reinterpret_cast<const float4*>(dp);
      *reinterpret_cast<float4*>(f + 4) = *reinterpret_cast<const float4*>(dp + 4);
    } else {
#pragma unroll
      for (int j = 0; j < 8; j++) f[j] = 0.f;
    }
    for (int ch = 0; ch < chunks; ch++) {
      const float* p = src + ch * slab + r * P_BLOCK_N + c8;
      const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
      f[0] += a.x; f[1] += a.y; f[2] += a.z; f[3] += a.w;
      f[4] += b.x; f[5] += b.y; f[6] += b.z; f[7] += b.w;
    }
    if (OUT == P_OUT_BF16) {
      Vec8<__nv_bfloat16> o;
      o.from_float(f);
      o.store(reinterpret_cast<__nv_bfloat16*>(d_) + static_cast<int64_t>(row) * ldd + col);
    } else {
      float* dp = reinterpret_cast<float*>(d_) + static_cast<int64_t>(row) * ldd + col;
      *reinterpret_cast<float4*>(dp) = *reinterpret_cast<float4*>(f);
      *reinterpret_cast<float4*>(dp + 4) = *reinterpret_cast<float4*>(f + 4);
    }
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Per-device fp32 workspace for split tiles (caller-owned, ws_tiles slabs of 256 x 256 floats); see ntb_gemm2_set_workspace.
static float* g_p_ws[64] = {};
static int g_p_ws_tiles[64] = {};
static cudaStream_t g_p_ws_stream[64] = {};
static int g_p_split_enabled = 0;  // off by default: measured within +-5 % of whole tiles on Llama shapes (the step is power-bound, not round-bound)

// How the tiles of a launch are dealt out (see PSched).  `ws_tiles`: workspace slabs available (0: never split).
static PSched p_schedule(int num_tiles, int pairs_max, int k_blocks, int ws_tiles) {
  PSched sc;
  sc.total_units = sc.full_units = num_tiles;
  sc.split = 1;
  sc.kb_per = k_blocks;
  if (!g_p_split_enabled || ws_tiles <= 0 || num_tiles <= 0) return sc;
  const int rounds = num_tiles / pairs_max, rem = num_tiles % pairs_max;
  if (rem == 0 || rem * 100 >= pairs_max * 85) return sc;  // the last round is (nearly) full already
  int split = pairs_max / rem;
  if (split > k_blocks / 4) split = k_blocks / 4;  // at least four k-blocks per chunk
  if (split < 2) return sc;
  if (rem * split > ws_tiles) return sc;
  sc.full_units = rounds * pairs_max;
  sc.split = split;
  sc.kb_per = (k_blocks + split - 1) / split;
  sc.total_units = sc.full_units + rem * split;
  return sc;
}

EncodeTiledFn p_get_encode() {
  ntb_bind_context_to_thread();
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

bool p_map_kmajor(CUtensorMap* m, const void* ptr, int64_t rows, int64_t k, int64_t ld) {
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64, 128};
  cuuint32_t es[2] = {1, 1};
  return p_get_encode()(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
bool p_map_mnmajor(CUtensorMap* m, const void* ptr, int64_t mn, int64_t k, int64_t ld) {
  cuuint64_t dims[3] = {64, (cuuint64_t)k, (cuuint64_t)((mn + 63) / 64)};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, 128};
  cuuint32_t box[3] = {64, (cuuint32_t)P_BLOCK_K, 2};
  cuuint32_t es[3] = {1, 1, 1};
  return p_get_encode()(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
bool p_map_out(CUtensorMap* m, void* ptr, int64_t rows, int64_t cols, int64_t ld, bool f32) {
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * (f32 ? 4 : 2)};
  cuuint32_t box[2] = {(cuuint32_t)(f32 ? 32 : 64), 32};
  cuuint32_t es[2] = {1, 1};
  return p_get_encode()(m, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ptr, dims, strides, box, es,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <bool A_MN, bool B_MN, int OUT, int ST = P_MAX_STAGES>
int p_launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td, int M, int N, int K, int* status, int num_sms, cudaStream_t stream,
             const PFuse& fuse = PFuse(), const PPeerMaps* pmaps = nullptr, void* d_out = nullptr, int64_t ldd = 0, const CUtensorMap* tal = nullptr) {
  static const PPeerMaps no_maps = {};
  const PPeerMaps& pm = pmaps ? *pmaps : no_maps;
  auto kern = gemm2_tcgen05_kernel<A_MN, B_MN, OUT, ST>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM) != cudaSuccess) return NTB_ERR_LAUNCH;
    configured = true;
  }
  const long long tiles = static_cast<long long>((M + 2 * P_BLOCK_M - 1) / (2 * P_BLOCK_M)) * ((N + P_BLOCK_N - 1) / P_BLOCK_N);
  const int k_blocks = (K + P_BLOCK_K - 1) / P_BLOCK_K;
  // every output mode but the peer stores of the reduce-scatter mode may cut the tiles of its last round along K, if a workspace
  // was registered for this device and stream and D is known as a plain pointer (16-byte aligned rows for the fix-up pass)
  int dev = 0, ws_tiles = 0;
  float* ws = nullptr;
  if (OUT != P_OUT_PEER_BF16 && d_out != nullptr && N % 8 == 0 && (OUT == P_OUT_BF16 || (ldd % 4 == 0 && (reinterpret_cast<uintptr_t>(d_out) & 15) == 0)) &&
      cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64 && g_p_ws[dev] != nullptr && g_p_ws_stream[dev] == stream) {
    ws = g_p_ws[dev];
    ws_tiles = g_p_ws_tiles[dev];
  }
  const PSched sched = p_schedule(static_cast<int>(tiles), num_sms / 2, k_blocks, tiles > (1 << 30) ? 0 : ws_tiles);
  CUtensorMap tws = td;  // placeholder when nothing goes through the workspace
  const bool uses_ws = sched.split > 1;
  if (uses_ws && !p_map_out(&tws, ws, static_cast<int64_t>(ws_tiles) * 2 * P_BLOCK_M, P_BLOCK_N, P_BLOCK_N, true)) return NTB_ERR_ARG;
  long long pairs = num_sms / 2;
  if (sched.total_units < pairs) pairs = sched.total_units;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs), 1, 1);
  cfg.blockDim = dim3(P_THREADS, 1, 1);
  cfg.dynamicSmemBytes = P_SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // rows of A (256 per tile row, K deep, bf16) that should stay resident in the 126 MB L2 while B streams: about 40 MB
  int band = static_cast<int>(40000000ll / (512ll * (K > 0 ? K : 1)));
  const int tiles_m = (M + 2 * P_BLOCK_M - 1) / (2 * P_BLOCK_M);
  if (band < 2) band = 2;
  if (band > tiles_m) band = tiles_m;
  if (cudaLaunchKernelEx(&cfg, kern, ta, tb, td, M, N, K, band, status, fuse, pm, sched, tws, tal ? *tal : ta) != cudaSuccess) {
    cudaGetLastError();
    return NTB_ERR_LAUNCH;
  }
  if (uses_ws) {
    const int split_tiles = static_cast<int>(tiles) - sched.full_units;
    const int tiles_n = (N + P_BLOCK_N - 1) / P_BLOCK_N;
    gemm2_split_fixup_kernel<OUT><<<split_tiles * 8, 256, 0, stream>>>(ws, d_out, ldd, M, N, k_blocks, sched, tiles_m, tiles_n, band, fuse.m_rot);
  }
  return ntb_check_launch();
}

}  // namespace

// Same contract as ntb_gemm_bf16 (gemm_tcgen05.cu); additionally M-major / N-major operands need M % 128 == 0 / N % 128 == 0 is NOT
// required: edges are clipped by TMA.  a_mn / b_mn: 0 = K-major, 1 = MN-major.  out_mode: 0 bf16 store, 1 fp32 store, 2 fp32 accumulate.
// Which argument check rejected the last ntb_gemm2_bf16 call of this thread (0: none; for error messages).
static thread_local int g_p_reject = 0;
NTB_EXPORT int ntb_gemm2_last_reject() { return g_p_reject; }

NTB_EXPORT int ntb_gemm2_bf16(const void* a, const void* b, void* d, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldd, int a_mn, int b_mn, int out_mode,
                              int* status, int num_sms, cudaStream_t stream) {
  g_p_reject = 0;
#define NTB_P_REJECT(code) do { g_p_reject = (code); return NTB_ERR_ARG; } while (0)
  if (M <= 0 || N <= 0 || K <= 0) NTB_P_REJECT(1);
  if (!p_get_encode()) NTB_P_REJECT(2);
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(d)) & 15) NTB_P_REJECT(3);
  if (a_mn ? (lda % 64 || M % 64) : (lda % 8)) NTB_P_REJECT(4);
  if (b_mn ? (ldb % 64 || N % 64) : (ldb % 8)) NTB_P_REJECT(5);
  if (out_mode == P_OUT_BF16 ? (ldd % 8) : (ldd % 4)) NTB_P_REJECT(6);
  if (num_sms <= 1) num_sms = 148;
  CUtensorMap ta, tb, td;
  if (!(a_mn ? p_map_mnmajor(&ta, a, M, K, lda) : p_map_kmajor(&ta, a, M, K, lda))) NTB_P_REJECT(7);
  if (!(b_mn ? p_map_mnmajor(&tb, b, N, K, ldb) : p_map_kmajor(&tb, b, N, K, ldb))) NTB_P_REJECT(8);
  if (!p_map_out(&td, d, M, N, ldd, out_mode != P_OUT_BF16)) NTB_P_REJECT(9);
#define NTB_P_CASE(AM, BM, OM) \
  if (a_mn == AM && b_mn == BM && out_mode == OM) return p_launch<AM != 0, BM != 0, OM>(ta, tb, td, M, N, K, status, num_sms, stream, PFuse(), nullptr, d, ldd);
  NTB_P_CASE(0, 0, 0) NTB_P_CASE(0, 0, 1) NTB_P_CASE(0, 0, 2)
  NTB_P_CASE(0, 1, 0) NTB_P_CASE(0, 1, 1) NTB_P_CASE(0, 1, 2)
  NTB_P_CASE(1, 1, 0) NTB_P_CASE(1, 1, 1) NTB_P_CASE(1, 1, 2)
  NTB_P_CASE(1, 0, 0) NTB_P_CASE(1, 0, 1) NTB_P_CASE(1, 0, 2)
#undef NTB_P_CASE
  NTB_P_REJECT(10);
#undef NTB_P_REJECT
}

// D = gathered_A @ B^T (or @ B when b_mn) where gathered_A = [world * ag_rows, K] is filled by ntb_tp_allgather_push on every rank
// (same contract as ntb_gemm_bf16_ag; ag_rows must be a multiple of 128 here).
static int p_gemm_ag(const void* a_gathered, const void* a_local, int64_t lda_local, const void* b, void* d, int M, int N, int K, int64_t lda, int64_t ldb,
                     int64_t ldd, int b_mn, const uint32_t* ag_flags, int ag_rows, int me, int world, uint32_t epoch, int* status, int num_sms,
                     cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || !p_get_encode() || world < 1 || world > P_TP_MAX || ag_rows <= 0 || ag_rows % P_BLOCK_M || ag_flags == nullptr) return NTB_ERR_ARG;
  if (me < 0 || me >= world || static_cast<int64_t>(ag_rows) * world != M) return NTB_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(a_gathered) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(d) | reinterpret_cast<uintptr_t>(a_local)) & 15) return NTB_ERR_ARG;
  if (lda % 8 || (b_mn ? (ldb % 64 || N % 64) : (ldb % 8)) || ldd % 8 || (a_local != nullptr && lda_local % 8)) return NTB_ERR_ARG;
  if (num_sms <= 1) num_sms = 148;
  CUtensorMap ta, tb, td, tal;
  if (!p_map_kmajor(&ta, a_gathered, M, K, lda)) return NTB_ERR_ARG;
  if (a_local != nullptr && !p_map_kmajor(&tal, a_local, ag_rows, K, lda_local)) return NTB_ERR_ARG;
  if (!(b_mn ? p_map_mnmajor(&tb, b, N, K, ldb) : p_map_kmajor(&tb, b, N, K, ldb))) return NTB_ERR_ARG;
  if (!p_map_out(&td, d, M, N, ldd, false)) return NTB_ERR_ARG;
  PFuse f;
  f.world = world;
  f.me = me;
  f.epoch = epoch;
  f.ag_flags = ag_flags;
  f.ag_rows = ag_rows;
  f.ag_local = a_local != nullptr ? 1 : 0;
  const int tiles_m = (M + 2 * P_BLOCK_M - 1) / (2 * P_BLOCK_M);
  f.m_rot = ((me * ag_rows) / (2 * P_BLOCK_M)) % tiles_m;  // start with the rows this rank contributed itself
  const CUtensorMap* pl = a_local != nullptr ? &tal : nullptr;
  return b_mn ? p_launch<false, true, P_OUT_BF16>(ta, tb, td, M, N, K, status, num_sms, stream, f, nullptr, d, ldd, pl)
              : p_launch<false, false, P_OUT_BF16>(ta, tb, td, M, N, K, status, num_sms, stream, f, nullptr, d, ldd, pl);
}

// D = gathered_A @ B^T (or @ B when b_mn) where gathered_A = [world * ag_rows, K] is filled by ntb_tp_allgather_push on every rank.
NTB_EXPORT int ntb_gemm2_bf16_ag(const void* a_gathered, const void* b, void* d, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldd, int b_mn,
                                 const uint32_t* ag_flags, int ag_rows, int me, int world, uint32_t epoch, int* status, int num_sms, cudaStream_t stream) {
  return p_gemm_ag(a_gathered, nullptr, 0, b, d, M, N, K, lda, ldb, ldd, b_mn, ag_flags, ag_rows, me, world, epoch, status, num_sms, stream);
}

// Same product, but rows [me * ag_rows, (me + 1) * ag_rows) are read from `a_local` (the tensor this rank pushes, row pitch
// lda_local) instead of from the gather buffer.  The launch then depends on no kernel of its own GPU, so the caller may run this
// rank's push on another stream at the same time; only the peers' blocks are waited for (bounded).
NTB_EXPORT int ntb_gemm2_bf16_ag_local(const void* a_gathered, const void* a_local, int64_t lda_local, const void* b, void* d, int M, int N, int K, int64_t lda,
                                       int64_t ldb, int64_t ldd, int b_mn, const uint32_t* ag_flags, int ag_rows, int me, int world, uint32_t epoch, int* status,
                                       int num_sms, cudaStream_t stream) {
  if (a_local == nullptr) return NTB_ERR_ARG;
  return p_gemm_ag(a_gathered, a_local, lda_local, b, d, M, N, K, lda, ldb, ldd, b_mn, ag_flags, ag_rows, me, world, epoch, status, num_sms, stream);
}

// Registers (ws != nullptr) or removes the fp32 workspace that lets launches on the CURRENT device cut the tiles of
// their last round along K: `tiles` slabs of 256 x 256 floats (contents do not matter), owned by the caller for as long as it is
// registered.  Only launches on `stream` use it (launches on other streams run unsplit), so two launches never write it at once.
// Returns 0, or NTB_ERR_ARG.
NTB_EXPORT int ntb_gemm2_set_workspace(float* ws, int tiles, cudaStream_t stream) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || (ws != nullptr && (tiles <= 0 || (reinterpret_cast<uintptr_t>(ws) & 127)))) return NTB_ERR_ARG;
  g_p_ws[dev] = ws;
  g_p_ws_tiles[dev] = ws ? tiles : 0;
  g_p_ws_stream[dev] = stream;
  return NTB_OK;
}

// Non-zero switches the split of the last round on for every launch that has a workspace, 0 (the default) off.
NTB_EXPORT void ntb_gemm2_enable_split(int on) { g_p_split_enabled = on != 0; }

// Partial product A @ B^T (or A @ B when b_mn) whose rows [r*rs_rows, (r+1)*rs_rows) are stored (bf16) into rank r's staging slot `me`
// (same contract as ntb_gemm_bf16_rs).
NTB_EXPORT int ntb_gemm2_bf16_rs(const void* a, const void* b, int M, int N, int K, int64_t lda, int64_t ldb, int b_mn, const uint64_t* staging_ptrs,
                                 const uint64_t* flag_ptrs, int rs_rows, int me, int world, uint32_t epoch, unsigned int* done_counter, int* status, int num_sms,
                                 cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || !p_get_encode() || world < 1 || world > P_TP_MAX || rs_rows * world != M || rs_rows % 32 || N % 8 || done_counter == nullptr) return NTB_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) return NTB_ERR_ARG;
  if (lda % 8 || (b_mn ? (ldb % 64 || N % 64) : (ldb % 8))) return NTB_ERR_ARG;
  if (num_sms <= 1) num_sms = 148;
  CUtensorMap ta, tb;
  if (!p_map_kmajor(&ta, a, M, K, lda)) return NTB_ERR_ARG;
  if (!(b_mn ? p_map_mnmajor(&tb, b, N, K, ldb) : p_map_kmajor(&tb, b, N, K, ldb))) return NTB_ERR_ARG;
  PFuse f;
  f.world = world;
  f.me = me;
  f.epoch = epoch;
  f.rs_rows = rs_rows;
  f.done_counter = done_counter;
  PPeerMaps pm = {};
  for (int r = 0; r < world; r++) {
    if (staging_ptrs[r] & 15) return NTB_ERR_ARG;
    if (!p_map_out(&pm.m[r], reinterpret_cast<void*>(staging_ptrs[r]), static_cast<int64_t>(world) * rs_rows, N, N, false)) return NTB_ERR_ARG;
    f.rs_flags[r] = reinterpret_cast<uint32_t*>(flag_ptrs[r]);
  }
  const int tiles_m = (M + 2 * P_BLOCK_M - 1) / (2 * P_BLOCK_M);
  f.m_rot = ((((me + 1) % world) * rs_rows) / (2 * P_BLOCK_M)) % tiles_m;  // the next rank's rows first, our own last
  return b_mn ? p_launch<false, true, P_OUT_PEER_BF16>(ta, tb, ta, M, N, K, status, num_sms, stream, f, &pm)
              : p_launch<false, false, P_OUT_PEER_BF16>(ta, tb, ta, M, N, K, status, num_sms, stream, f, &pm);
}
