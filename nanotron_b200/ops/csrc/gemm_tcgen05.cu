// bf16 GEMM on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), persistent and warp-specialised (sm_100a).
//
//   D[M,N] (=|+=) sum_k A(m,k) * B(n,k)
//
// Operand storage is selected per operand, so the three products of a linear layer need no transposed copies:
//   K-major  : element (m,k) at  ptr[m*ld + k]   (reduction index contiguous)   -- forward:  x[M,K], W[N,K]
//   MN-major : element (m,k) at  ptr[k*ld + m]   (output index contiguous)      -- dgrad: B = W[N_red, K_out];  wgrad: both
// Output modes: bf16 store, fp32 store, fp32 accumulate (TMA reduce-add into the fp32 main-gradient buffer).
//
// One CTA per SM walks output tiles of 128 x 256.  Warp roles:
//   warp 0     : TMA producer  (one elected lane; 4-stage ring of {A 128x64, B 256x64} bf16 tiles, 128-byte swizzle)
//   warp 1     : MMA issuer    (one elected lane; tcgen05.mma 128x256x16, fp32 accumulators in TMEM, double buffered:
//                               2 x 256 columns, so the epilogue of tile i overlaps the main loop of tile i+1)
//   warps 2..5 : epilogue      (tcgen05.ld 32 lanes x 32 columns at a time -> convert -> swizzled smem staging ->
//                               TMA store / reduce-add, double buffered per warp)
// Synchronisation is mbarrier-only (full/empty per stage, tmem_full/tmem_empty per accumulator).  All waits are bounded;
// on expiry the kernel raises a flag in `status`, drains what it issued, frees TMEM and returns.
// TMA clips stores and zero-fills loads at the M/N/K edges, so any M, N and K are accepted as long as the row pitches are
// multiples of 16 bytes (and 128 bytes for MN-major operands).
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_N = 256;
constexpr int BLOCK_K = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_TILE_BYTES = BLOCK_M * BLOCK_K * 2;  // 16 KiB
constexpr int B_TILE_BYTES = BLOCK_N * BLOCK_K * 2;  // 32 KiB
constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
constexpr int EPI_WARPS = 4;
constexpr int EPI_BUF_BYTES = 32 * 128;  // 32 rows x 128 bytes per warp per buffer
constexpr int EPI_BYTES = EPI_WARPS * 2 * EPI_BUF_BYTES;
constexpr int TMEM_COLS = 512;
constexpr int GEMM_THREADS = 32 * (2 + EPI_WARPS);
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;

enum OutMode { OUT_BF16 = 0, OUT_F32 = 1, OUT_F32_ACCUM = 2, OUT_PEER_BF16 = 3 };

// Tensor-parallel fusion hooks (all disabled when world == 0):
//  * all-gather -> GEMM: the A operand is a gathered buffer of `world` row blocks of `ag_rows` rows that peers fill with
//    plain stores; block r is valid once `ag_flags[r] >= epoch`.  The TMA producer polls that word (bounded) before its
//    first load from a block, and row blocks are visited starting with this rank's own, so the GEMM on blocks that
//    already arrived overlaps the NVLink transfer of the others.
//  * GEMM -> reduce-scatter (OUT_PEER_BF16): the epilogue TMA-stores each bf16 tile straight into the staging buffer of the
//    rank that owns those rows (one tensor map per owner over its [world * rs_rows, N] staging area, slot `me`), visiting
//    row blocks starting with the next rank's.  The last CTA to finish publishes `epoch` in every owner's `rs_flags[me]`;
//    owners then sum the `world` slots.
constexpr int TP_MAX = 8;
struct TpFuse {
  int world = 0, me = 0;
  uint32_t epoch = 0;
  int m_rot = 0;                      // tile-row rotation (in 128-row tiles)
  const uint32_t* ag_flags = nullptr; // local flag words [world]
  int ag_rows = 0;                    // rows per gathered block
  uint32_t* rs_flags[TP_MAX] = {};    // per-owner flag words [world]
  int rs_rows = 0;                    // rows per owner
  long long rs_slot_elems = 0;
  unsigned int* done_counter = nullptr;  // local counter, zero before launch
};

// Per-owner output maps of the GEMM -> reduce-scatter epilogue (unused otherwise).
struct PeerMaps {
  CUtensorMap m[TP_MAX];
};

struct TileCoord {
  int m_blk, n_blk;
};

// Grouped (mixture-of-experts) products.  Token rows live in a padded layout: expert e owns rows [seg_off[e], seg_off[e+1]),
// every offset a multiple of 128, so a 128-row block never mixes experts and the reduction range of a weight gradient is a
// whole number of 64-row k-blocks.  Offsets, the block -> expert table and the number of used blocks are DEVICE data
// (written by the dispatch kernels), so no launch parameter depends on the routing.
//   GROUP 1 (forward / dgrad): D[rows, N] = A[rows, K] x B[e(row block)]; blocks at or beyond *num_m_tiles are skipped.
//   GROUP 2 (wgrad):           D[e][M, N] = sum over the rows r of expert e of A[r, m] * B[r, n]  (both operands MN-major).
struct GroupArgs {
  const int* tile_expert = nullptr;  // GROUP 1: expert of each 128-row block
  const int* num_m_tiles = nullptr;  // GROUP 1: number of used 128-row blocks
  const int* seg_off = nullptr;      // GROUP 2: [E + 1] padded row offsets
  int E = 0;
};

struct Tile {
  int m_blk, n_blk, e, kb0, kbs;
  bool skip;
};

// Tiles are visited in column-major order inside bands of 8 tile-rows so that CTAs running at the same time share B
// tiles (and a few A tiles) through L2.
__device__ __forceinline__ TileCoord tile_coord(int t, int tiles_m, int tiles_n) {
  constexpr int BAND = 8;
  const int band_size = BAND * tiles_n;
  const int band = t / band_size;
  const int first_m = band * BAND;
  const int rows = min(BAND, tiles_m - first_m);
  const int r = t - band * band_size;
  return {first_m + r % rows, r / rows};
}

template <int GROUP>
__device__ __forceinline__ Tile decode_tile(int t, int tiles_m, int tiles_n, int k_blocks, const TpFuse& fuse, const GroupArgs& grp) {
  Tile r;
  if (GROUP == 2) {
    const int per = tiles_m * tiles_n;
    r.e = t / per;
    const TileCoord tc = tile_coord(t - r.e * per, tiles_m, tiles_n);
    r.m_blk = tc.m_blk;
    r.n_blk = tc.n_blk;
    const int lo = __ldg(grp.seg_off + r.e), hi = __ldg(grp.seg_off + r.e + 1);
    r.kb0 = lo / BLOCK_K;
    r.kbs = (hi - lo) / BLOCK_K;
    r.skip = r.kbs <= 0;
  } else {
    const TileCoord tc = tile_coord(t, tiles_m, tiles_n);
    r.m_blk = (tc.m_blk + fuse.m_rot) % tiles_m;
    r.n_blk = tc.n_blk;
    r.kb0 = 0;
    r.kbs = k_blocks;
    r.e = 0;
    r.skip = false;
    if (GROUP == 1) {
      r.skip = r.m_blk >= __ldg(grp.num_m_tiles);
      if (!r.skip) r.e = __ldg(grp.tile_expert + r.m_blk);
    }
  }
  return r;
}

template <bool A_MN, bool B_MN, int OUT, int GROUP>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const __grid_constant__ CUtensorMap tmap_d,
                    int M, int N, int K, int* __restrict__ status, const __grid_constant__ TpFuse fuse, const __grid_constant__ GroupArgs grp,
                    const __grid_constant__ PeerMaps pmaps) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_smem = smem + STAGES * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + EPI_BYTES);
  uint64_t* full_bar = bars;                 // [STAGES]
  uint64_t* empty_bar = bars + STAGES;       // [STAGES]
  uint64_t* tmem_full = bars + 2 * STAGES;   // [2]
  uint64_t* tmem_empty = tmem_full + 2;      // [2]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (M + BLOCK_M - 1) / BLOCK_M;
  const int tiles_n = (N + BLOCK_N - 1) / BLOCK_N;
  const int num_tiles = tiles_m * tiles_n * (GROUP == 2 ? grp.E : 1);
  const int k_blocks = (K + BLOCK_K - 1) / BLOCK_K;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; b++) {
      ptx::mbar_init(&tmem_full[b], 1);
      ptx::mbar_init(&tmem_empty[b], EPI_WARPS);
    }
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tmap(&tmap_a);
    ptx::prefetch_tmap(&tmap_b);
    ptx::prefetch_tmap(&tmap_d);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_base_slot, TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (ptx::elect_one()) {
      int it = 0;
      bool ok = true;
      uint32_t ag_ready = 0;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const Tile tc = decode_tile<GROUP>(t, tiles_m, tiles_n, k_blocks, fuse, grp);
        if (tc.skip) continue;
        if (fuse.ag_flags != nullptr) {
          // rows [m_blk*128, +128) may span two gathered blocks when ag_rows is not a multiple of 128
          const int first = (tc.m_blk * BLOCK_M) / fuse.ag_rows;
          const int last = min(fuse.world - 1, (min(M, (tc.m_blk + 1) * BLOCK_M) - 1) / fuse.ag_rows);
          for (int src = first; src <= last && ok; src++) {
            if (ag_ready & (1u << src)) continue;
            const uint64_t t0 = ptx::globaltimer();
            while (true) {
              uint32_t v;
              asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(fuse.ag_flags + src) : "memory");
              if (static_cast<int32_t>(v - fuse.epoch) >= 0) { ag_ready |= 1u << src; break; }
              if (*abort_flag || ptx::globaltimer() - t0 > NTB_WAIT_LIMIT_NS) { *abort_flag = 1; ok = false; break; }
              __nanosleep(100);
            }
          }
          if (!ok) break;
          // data written by peers with generic stores must be visible to the async (TMA) proxy
          asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        for (int kb = 0; kb < tc.kbs; kb++, it++) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!ptx::mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, 64)) { ok = false; break; }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_TILE_BYTES;
          const int kx = (tc.kb0 + kb) * BLOCK_K;
          ptx::mbar_expect_tx(&full_bar[s], STAGE_BYTES);
          if (A_MN) ptx::tma_load_3d(sa, &tmap_a, &full_bar[s], 0, kx, tc.m_blk * (BLOCK_M / 64));
          else      ptx::tma_load_2d(sa, &tmap_a, &full_bar[s], kx, tc.m_blk * BLOCK_M);
          if (GROUP == 1) {  // the B operand of this row block is the weight of its expert (outermost map dimension)
            if (B_MN) ptx::tma_load_4d(sb, &tmap_b, &full_bar[s], 0, kx, tc.n_blk * (BLOCK_N / 64), tc.e);
            else      ptx::tma_load_3d(sb, &tmap_b, &full_bar[s], kx, tc.n_blk * BLOCK_N, tc.e);
          } else {
            if (B_MN) ptx::tma_load_3d(sb, &tmap_b, &full_bar[s], 0, kx, tc.n_blk * (BLOCK_N / 64));
            else      ptx::tma_load_2d(sb, &tmap_b, &full_bar[s], kx, tc.n_blk * BLOCK_N);
          }
        }
      }
      if (!ok) {
        // let copies already in flight land before the CTA's shared memory goes away (bounded by the same limit)
        const uint64_t t0 = ptx::globaltimer();
        for (int s = 0; s < STAGES; s++) {
          const int last = it - 1 - ((it - 1 - s) % STAGES + STAGES) % STAGES;  // last iteration that used stage s
          if (it == 0 || last < 0) continue;
          const uint32_t ph = (last / STAGES) & 1;
          while (!ptx::mbar_try_wait(&full_bar[s], ph) && ptx::globaltimer() - t0 < NTB_WAIT_LIMIT_NS) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (ptx::elect_one()) {
      constexpr uint32_t idesc = ptx::make_idesc_bf16(BLOCK_M, BLOCK_N, A_MN, B_MN);
      int it = 0, tile_it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const Tile tc = decode_tile<GROUP>(t, tiles_m, tiles_n, k_blocks, fuse, grp);
        if (tc.skip) continue;
        const int acc = tile_it & 1;
        const uint32_t acc_ph = (tile_it >> 1) & 1;
        tile_it++;
        if (!ptx::mbar_wait(&tmem_empty[acc], acc_ph ^ 1, abort_flag)) { ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BLOCK_N;
        for (int kb = 0; kb < tc.kbs; kb++, it++) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!ptx::mbar_wait(&full_bar[s], ph, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t sa = ptx::smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + A_TILE_BYTES;
#pragma unroll
          for (int k = 0; k < BLOCK_K / UMMA_K; k++) {
            const uint64_t adesc = A_MN ? ptx::make_smem_desc(sa + k * UMMA_K * 128, BLOCK_K * 128, 1024) : ptx::make_smem_desc(sa + k * UMMA_K * 2, 16, 1024);
            const uint64_t bdesc = B_MN ? ptx::make_smem_desc(sb + k * UMMA_K * 128, BLOCK_K * 128, 1024) : ptx::make_smem_desc(sb + k * UMMA_K * 2, 16, 1024);
            ptx::umma_f16(tmem_d, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          ptx::umma_commit(&empty_bar[s]);  // frees the stage once these MMAs have read it
        }
        if (ok) ptx::umma_commit(&tmem_full[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    uint8_t* my_epi = epi_smem + (warp - 2) * 2 * EPI_BUF_BYTES;
    constexpr bool BF16_OUT = (OUT == OUT_BF16 || OUT == OUT_PEER_BF16);
    constexpr int CHUNK_COLS = BF16_OUT ? 64 : 32;  // 128 bytes of output per row
    constexpr int CHUNKS = BLOCK_N / CHUNK_COLS;
    int tile_it = 0, buf = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      const Tile tc = decode_tile<GROUP>(t, tiles_m, tiles_n, k_blocks, fuse, grp);
      if (tc.skip) continue;
      const int acc = tile_it & 1;
      const uint32_t acc_ph = (tile_it >> 1) & 1;
      tile_it++;
      if (!ptx::mbar_wait(&tmem_full[acc], acc_ph, abort_flag, 256)) { ok = false; break; }
      ptx::tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BLOCK_N;
      const int row0 = tc.m_blk * BLOCK_M + q * 32;
#pragma unroll 1
      for (int c = 0; c < CHUNKS; c++) {
        uint8_t* stage_buf = my_epi + buf * EPI_BUF_BYTES;
        // the TMA store that last read this staging buffer must be done reading it
        if (lane == 0) ptx::tma_wait_group_read<1>();
        __syncwarp();
        uint8_t* my_row = stage_buf + lane * 128;
        if (BF16_OUT) {
          uint32_t r0[32], r1[32];
          ptx::tmem_ld_32x32(taddr + c * 64, r0);
          ptx::tmem_ld_32x32(taddr + c * 64 + 32, r1);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; j++) {  // 8 x 16 bytes = 64 bf16
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
            *reinterpret_cast<uint4*>(my_row + ((j ^ (lane & 7)) << 4)) = pk;  // 128-byte swizzle
          }
        } else {
          uint32_t r0[32];
          ptx::tmem_ld_32x32(taddr + c * 32, r0);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; j++) {  // 8 x 16 bytes = 32 fp32
            uint4 pk = make_uint4(r0[j * 4], r0[j * 4 + 1], r0[j * 4 + 2], r0[j * 4 + 3]);
            *reinterpret_cast<uint4*>(my_row + ((j ^ (lane & 7)) << 4)) = pk;
          }
        }
        ptx::fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          const int x = tc.n_blk * BLOCK_N + c * CHUNK_COLS;
          if (OUT == OUT_PEER_BF16) {
            if (x < N && row0 < M) {
              const int owner = row0 / fuse.rs_rows;  // rs_rows is a multiple of 32: the 32 rows of this warp share an owner
              ptx::tma_store_2d(&pmaps.m[owner], stage_buf, x, fuse.me * fuse.rs_rows + (row0 - owner * fuse.rs_rows));
            }
          } else if (x < N && row0 < M) {
            if (GROUP == 2) {  // one weight-gradient matrix per expert: outermost map dimension
              if (OUT == OUT_F32_ACCUM) ptx::tma_reduce_add_3d(&tmap_d, stage_buf, x, row0, tc.e);
              else ptx::tma_store_3d(&tmap_d, stage_buf, x, row0, tc.e);
            } else {
              if (OUT == OUT_F32_ACCUM) ptx::tma_reduce_add_2d(&tmap_d, stage_buf, x, row0);
              else ptx::tma_store_2d(&tmap_d, stage_buf, x, row0);
            }
          }
          ptx::tma_commit_group();
        }
        buf ^= 1;
      }
      // accumulator fully read: hand it back to the MMA warp
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&tmem_empty[acc]);
    }
    if (lane == 0) {
      ptx::tma_wait_group<0>();  // all stores complete before the CTA exits
      if (OUT == OUT_PEER_BF16) {
        // the peer stores were made by the async proxy: order them before the generic-proxy flag store that follows the CTA barrier
        asm volatile("fence.proxy.async.global;" ::: "memory");
        __threadfence_system();
      }
    }
    __syncwarp();
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (OUT == OUT_PEER_BF16 && fuse.done_counter != nullptr && threadIdx.x == 0) {
    // all stores of this CTA (made by the epilogue warps before the barrier above) become visible system-wide, then the
    // last CTA to get here tells every owner that this rank's partial sums are complete
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

// ---------------------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
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

// K-major operand [rows, k] with pitch ld (elements): 2-D map {k, rows}, box {64, box_rows}.
bool make_map_kmajor(CUtensorMap* m, const void* ptr, int64_t rows, int64_t k, int64_t ld, int box_rows) {
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t es[2] = {1, 1};
  return get_encode()(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// MN-major operand stored [k, mn] with pitch ld: 3-D map {64, k, mn/64} so one copy lands as [mn/64][k][64] in shared memory.
bool make_map_mnmajor(CUtensorMap* m, const void* ptr, int64_t mn, int64_t k, int64_t ld, int box_mn) {
  cuuint64_t dims[3] = {64, (cuuint64_t)k, (cuuint64_t)((mn + 63) / 64)};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, 128};
  cuuint32_t box[3] = {64, (cuuint32_t)BLOCK_K, (cuuint32_t)(box_mn / 64)};
  cuuint32_t es[3] = {1, 1, 1};
  return get_encode()(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool make_map_out(CUtensorMap* m, void* ptr, int64_t rows, int64_t cols, int64_t ld, bool f32) {
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * (f32 ? 4 : 2)};
  cuuint32_t box[2] = {(cuuint32_t)(f32 ? 32 : 64), 32};
  cuuint32_t es[2] = {1, 1};
  return get_encode()(m, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ptr, dims, strides, box, es,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <bool A_MN, bool B_MN, int OUT, int GROUP = 0>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td, int M, int N, int K, int* status, int num_sms, cudaStream_t stream,
           const TpFuse& fuse = TpFuse(), const GroupArgs& grp = GroupArgs(), const PeerMaps* pmaps = nullptr) {
  auto kern = gemm_tcgen05_kernel<A_MN, B_MN, OUT, GROUP>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return NTB_ERR_LAUNCH;
    configured = true;
  }
  const long long tiles = static_cast<long long>((M + BLOCK_M - 1) / BLOCK_M) * ((N + BLOCK_N - 1) / BLOCK_N) * (GROUP == 2 ? grp.E : 1);
  const int grid = tiles < num_sms ? static_cast<int>(tiles) : num_sms;
  static const PeerMaps no_maps = {};
  kern<<<grid, GEMM_THREADS, SMEM_BYTES, stream>>>(ta, tb, td, M, N, K, status, fuse, grp, pmaps ? *pmaps : no_maps);
  return ntb_check_launch();
}

}  // namespace

// a_mn / b_mn: 0 = K-major ([rows, K] row-major), 1 = MN-major ([K, rows] row-major).  lda / ldb / ldd are row pitches in
// elements.  out_mode: 0 bf16 store, 1 fp32 store, 2 fp32 accumulate.  `status` (device int, may be null) receives
// NTB_ERR_TIMEOUT if a bounded wait expired.
NTB_EXPORT int ntb_gemm_bf16(const void* a, const void* b, void* d, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldd, int a_mn, int b_mn,
                             int out_mode, int* status, int num_sms, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || !get_encode()) return NTB_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(d)) & 15) return NTB_ERR_ARG;
  if (a_mn ? (lda % 64 || M % 64) : (lda % 8)) return NTB_ERR_ARG;
  if (b_mn ? (ldb % 64 || N % 64) : (ldb % 8)) return NTB_ERR_ARG;
  if (out_mode == OUT_BF16 ? (ldd % 8) : (ldd % 4)) return NTB_ERR_ARG;
  if (num_sms <= 0) num_sms = 148;
  CUtensorMap ta, tb, td;
  bool ok = a_mn ? make_map_mnmajor(&ta, a, M, K, lda, BLOCK_M) : make_map_kmajor(&ta, a, M, K, lda, BLOCK_M);
  ok = ok && (b_mn ? make_map_mnmajor(&tb, b, N, K, ldb, BLOCK_N) : make_map_kmajor(&tb, b, N, K, ldb, BLOCK_N));
  ok = ok && make_map_out(&td, d, M, N, ldd, out_mode != OUT_BF16);
  if (!ok) return NTB_ERR_ARG;
#define NTB_GEMM_CASE(AM, BM, OM) \
  if (a_mn == AM && b_mn == BM && out_mode == OM) return launch<AM != 0, BM != 0, OM>(ta, tb, td, M, N, K, status, num_sms, stream);
  NTB_GEMM_CASE(0, 0, 0) NTB_GEMM_CASE(0, 0, 1) NTB_GEMM_CASE(0, 0, 2)
  NTB_GEMM_CASE(0, 1, 0) NTB_GEMM_CASE(0, 1, 1) NTB_GEMM_CASE(0, 1, 2)
  NTB_GEMM_CASE(1, 1, 0) NTB_GEMM_CASE(1, 1, 1) NTB_GEMM_CASE(1, 1, 2)
  NTB_GEMM_CASE(1, 0, 0) NTB_GEMM_CASE(1, 0, 1) NTB_GEMM_CASE(1, 0, 2)
#undef NTB_GEMM_CASE
  return NTB_ERR_ARG;
}


// ---------------------------------------------------------------------------------------------- grouped (mixture-of-experts) entry points
namespace {

// Expert weights, K-major: [E, rows, k] contiguous -> 3-D map {k, rows, E}, box {64, 256, 1}.
bool make_map_kmajor_batched(CUtensorMap* m, const void* ptr, int64_t rows, int64_t k, int64_t ld, int64_t E, int box_rows) {
  cuuint64_t dims[3] = {(cuuint64_t)k, (cuuint64_t)rows, (cuuint64_t)E};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)ld * 2 * (cuuint64_t)rows};
  cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
  cuuint32_t es[3] = {1, 1, 1};
  return get_encode()(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Expert weights, MN-major: [E, k, mn] contiguous -> 4-D map {64, k, mn/64, E}.
bool make_map_mnmajor_batched(CUtensorMap* m, const void* ptr, int64_t mn, int64_t k, int64_t ld, int64_t E, int box_mn) {
  cuuint64_t dims[4] = {64, (cuuint64_t)k, (cuuint64_t)((mn + 63) / 64), (cuuint64_t)E};
  cuuint64_t strides[3] = {(cuuint64_t)ld * 2, 128, (cuuint64_t)ld * 2 * (cuuint64_t)k};
  cuuint32_t box[4] = {64, (cuuint32_t)BLOCK_K, (cuuint32_t)(box_mn / 64), 1};
  cuuint32_t es[4] = {1, 1, 1, 1};
  return get_encode()(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Per-expert output [E, rows, cols] contiguous -> 3-D map {cols, rows, E}.
bool make_map_out_batched(CUtensorMap* m, void* ptr, int64_t rows, int64_t cols, int64_t E, bool f32) {
  const cuuint64_t esz = f32 ? 4 : 2;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)E};
  cuuint64_t strides[2] = {(cuuint64_t)cols * esz, (cuuint64_t)cols * esz * (cuuint64_t)rows};
  cuuint32_t box[3] = {(cuuint32_t)(f32 ? 32 : 64), 32, 1};
  cuuint32_t es[3] = {1, 1, 1};
  return get_encode()(m, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, ptr, dims, strides, box, es,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// Rows of `a` [rows_cap, K] (bf16, padded expert layout) times the weight of each row block's expert:
//   b_mn = 0: b is [E, N, K] (d = a @ b[e]^T, e.g. dgrad against [E, K_in, N_out] weights seen as [E, N, K]);
//   b_mn = 1: b is [E, K, N] (d = a @ b[e], the forward of [E, in, out] weights).
// d is [rows_cap, N] bf16.  tile_expert[rows_cap / 128] and num_m_tiles[1] are device data.
NTB_EXPORT int ntb_gemm_bf16_grouped(const void* a, const void* b, void* d, int rows_cap, int N, int K, int b_mn, int E, const int* tile_expert,
                                     const int* num_m_tiles, int* status, int num_sms, cudaStream_t stream) {
  if (rows_cap <= 0 || rows_cap % BLOCK_M || N <= 0 || K <= 0 || E <= 0 || !get_encode() || !tile_expert || !num_m_tiles) return NTB_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(d)) & 15) return NTB_ERR_ARG;
  if (K % 8 || N % 8 || (b_mn && N % 64)) return NTB_ERR_ARG;
  CUtensorMap ta, tb, td;
  bool ok = make_map_kmajor(&ta, a, rows_cap, K, K, BLOCK_M);
  ok = ok && (b_mn ? make_map_mnmajor_batched(&tb, b, N, K, N, E, BLOCK_N) : make_map_kmajor_batched(&tb, b, N, K, K, E, BLOCK_N));
  ok = ok && make_map_out(&td, d, rows_cap, N, N, false);
  if (!ok) return NTB_ERR_ARG;
  GroupArgs g;
  g.tile_expert = tile_expert;
  g.num_m_tiles = num_m_tiles;
  g.E = E;
  if (num_sms <= 0) num_sms = 148;
  return b_mn ? launch<false, true, OUT_BF16, 1>(ta, tb, td, rows_cap, N, K, status, num_sms, stream, TpFuse(), g)
              : launch<false, false, OUT_BF16, 1>(ta, tb, td, rows_cap, N, K, status, num_sms, stream, TpFuse(), g);
}

// Weight gradients of every expert in one launch: dw[e][m, n] (=|+=) sum over rows r in [seg_off[e], seg_off[e+1]) of x[r, m] * dy[r, n].
// x is [rows_cap, M], dy is [rows_cap, N] (bf16; rows in padding must be zero), dw is [E, M, N] (out_mode 0 bf16, 1 fp32, 2 fp32 +=).
// Experts without rows are skipped: in the store modes the caller provides a zeroed `dw`.
NTB_EXPORT int ntb_gemm_bf16_grouped_wgrad(const void* x, const void* dy, void* dw, int rows_cap, int M, int N, int E, const int* seg_off, int out_mode,
                                           int* status, int num_sms, cudaStream_t stream) {
  if (rows_cap <= 0 || rows_cap % BLOCK_M || M <= 0 || N <= 0 || E <= 0 || !get_encode() || !seg_off || out_mode < 0 || out_mode > 2) return NTB_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dw)) & 15) return NTB_ERR_ARG;
  if (M % 64 || N % 64) return NTB_ERR_ARG;
  CUtensorMap ta, tb, td;
  bool ok = make_map_mnmajor(&ta, x, M, rows_cap, M, BLOCK_M);
  ok = ok && make_map_mnmajor(&tb, dy, N, rows_cap, N, BLOCK_N);
  ok = ok && make_map_out_batched(&td, dw, M, N, E, out_mode != OUT_BF16);
  if (!ok) return NTB_ERR_ARG;
  GroupArgs g;
  g.seg_off = seg_off;
  g.E = E;
  if (num_sms <= 0) num_sms = 148;
  if (out_mode == OUT_BF16) return launch<true, true, OUT_BF16, 2>(ta, tb, td, M, N, rows_cap, status, num_sms, stream, TpFuse(), g);
  if (out_mode == OUT_F32) return launch<true, true, OUT_F32, 2>(ta, tb, td, M, N, rows_cap, status, num_sms, stream, TpFuse(), g);
  return launch<true, true, OUT_F32_ACCUM, 2>(ta, tb, td, M, N, rows_cap, status, num_sms, stream, TpFuse(), g);
}


// ---------------------------------------------------------------------------------------------- tensor-parallel fused entry points
namespace {

struct PushPeers {
  void* dst[TP_MAX];
  uint32_t* flags[TP_MAX];
};

// Copies this rank's block into slot `me` of every rank's gather buffer (16-byte peer stores), then the last CTA publishes
// `epoch` in every rank's flag word `me`.
__global__ void ag_push_kernel(const uint4* __restrict__ src, PushPeers peers, int me, int world, long long n16, long long slot16, uint32_t epoch,
                               unsigned int* done_counter) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n16; i += stride) {
    const uint4 v = src[i];
    for (int k = 0; k < world; k++) {
      const int r = (me + k) % world;
      reinterpret_cast<uint4*>(peers.dst[r])[me * slot16 + i] = v;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(done_counter, 1u);
    if (prev == gridDim.x - 1) {
      __threadfence_system();
      for (int r = 0; r < world; r++) asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peers.flags[r] + me), "r"(epoch) : "memory");
      *done_counter = 0;
    }
  }
}

// out[i] = sum over slots (fixed order) of staging[slot][i], after every slot's flag reached `epoch`.
__global__ void rs_reduce_kernel(const __nv_bfloat16* __restrict__ staging, __nv_bfloat16* __restrict__ out, const uint32_t* __restrict__ flags, int world,
                                 long long n, long long slot_elems, uint32_t epoch, unsigned long long limit_ns, int* status) {
  __shared__ int bad;
  if (threadIdx.x == 0) {
    bad = 0;
    const uint64_t t0 = ptx::globaltimer();
    for (int r = 0; r < world; r++) {
      while (true) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + r) : "memory");
        if (static_cast<int32_t>(v - epoch) >= 0) break;
        if (ptx::globaltimer() - t0 > limit_ns) { bad = 1; break; }
        __nanosleep(100);
      }
      if (bad) break;
    }
  }
  __syncthreads();
  if (bad) {
    if (threadIdx.x == 0 && status) atomicExch(status, NTB_ERR_TIMEOUT);
    return;
  }
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 8;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8; i < n; i += stride) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r = 0; r < world; r++) {
      uint4 raw;
      asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(raw.x), "=r"(raw.y), "=r"(raw.z), "=r"(raw.w) : "l"(staging + r * slot_elems + i) : "memory");
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    Vec8<__nv_bfloat16> o;
    o.from_float(acc);
    o.store(out + i);
  }
}

}  // namespace

// Push this rank's [rows, K] bf16 block into slot `me` of every rank's gather buffer and raise flag `me` everywhere.
NTB_EXPORT int ntb_tp_allgather_push(const void* src, const uint64_t* gather_ptrs, const uint64_t* flag_ptrs, int me, int world, long long elems,
                                     uint32_t epoch, unsigned int* done_counter, cudaStream_t stream) {
  if (world < 1 || world > TP_MAX || elems <= 0 || elems % 8 || (reinterpret_cast<uintptr_t>(src) & 15)) return NTB_ERR_ARG;
  PushPeers peers;
  for (int r = 0; r < TP_MAX; r++) {
    peers.dst[r] = r < world ? reinterpret_cast<void*>(gather_ptrs[r]) : nullptr;
    peers.flags[r] = r < world ? reinterpret_cast<uint32_t*>(flag_ptrs[r]) : nullptr;
  }
  const long long n16 = elems / 8;
  int blocks = static_cast<int>((n16 + 255) / 256);
  if (blocks > 148 * 2) blocks = 148 * 2;
  ag_push_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const uint4*>(src), peers, me, world, n16, n16, epoch, done_counter);
  return ntb_check_launch();
}

// D = gathered_A @ B^T where gathered_A = [world * ag_rows, K] is filled by ntb_tp_allgather_push on every rank.
NTB_EXPORT int ntb_gemm_bf16_ag(const void* a_gathered, const void* b, void* d, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldd, int b_mn,
                                const uint32_t* ag_flags, int ag_rows, int me, int world, uint32_t epoch, int* status, int num_sms, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || !get_encode() || world < 1 || world > TP_MAX || ag_rows % BLOCK_M) return NTB_ERR_ARG;
  if (lda % 8 || (b_mn ? (ldb % 64 || N % 64) : (ldb % 8)) || ldd % 8) return NTB_ERR_ARG;
  CUtensorMap ta, tb, td;
  bool ok = make_map_kmajor(&ta, a_gathered, M, K, lda, BLOCK_M);
  ok = ok && (b_mn ? make_map_mnmajor(&tb, b, N, K, ldb, BLOCK_N) : make_map_kmajor(&tb, b, N, K, ldb, BLOCK_N));
  ok = ok && make_map_out(&td, d, M, N, ldd, false);
  if (!ok) return NTB_ERR_ARG;
  TpFuse f;
  f.world = world;
  f.me = me;
  f.epoch = epoch;
  f.ag_flags = ag_flags;
  f.ag_rows = ag_rows;
  f.m_rot = (me * ag_rows) / BLOCK_M;  // start with the rows this rank contributed itself
  if (num_sms <= 0) num_sms = 148;
  return b_mn ? launch<false, true, OUT_BF16>(ta, tb, td, M, N, K, status, num_sms, stream, f) : launch<false, false, OUT_BF16>(ta, tb, td, M, N, K, status, num_sms, stream, f);
}

// Partial product A @ B^T whose rows [r*rs_rows, (r+1)*rs_rows) are stored (bf16) into rank r's staging slot `me`.
NTB_EXPORT int ntb_gemm_bf16_rs(const void* a, const void* b, int M, int N, int K, int64_t lda, int64_t ldb, int b_mn, const uint64_t* staging_ptrs,
                                const uint64_t* flag_ptrs, int rs_rows, int me, int world, uint32_t epoch, unsigned int* done_counter, int* status, int num_sms,
                                cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || !get_encode() || world < 1 || world > TP_MAX || rs_rows * world != M || rs_rows % 32 || N % 8) return NTB_ERR_ARG;
  if (lda % 8 || (b_mn ? (ldb % 64 || N % 64) : (ldb % 8))) return NTB_ERR_ARG;
  CUtensorMap ta, tb, td;
  bool ok = make_map_kmajor(&ta, a, M, K, lda, BLOCK_M);
  ok = ok && (b_mn ? make_map_mnmajor(&tb, b, N, K, ldb, BLOCK_N) : make_map_kmajor(&tb, b, N, K, ldb, BLOCK_N));
  if (!ok) return NTB_ERR_ARG;
  td = ta;  // unused in this mode
  TpFuse f;
  f.world = world;
  f.me = me;
  f.epoch = epoch;
  f.rs_rows = rs_rows;
  f.rs_slot_elems = static_cast<long long>(rs_rows) * N;
  PeerMaps pm = {};
  for (int r = 0; r < world; r++) {
    if (staging_ptrs[r] & 15) return NTB_ERR_ARG;
    if (!make_map_out(&pm.m[r], reinterpret_cast<void*>(staging_ptrs[r]), static_cast<int64_t>(world) * rs_rows, N, N, false)) return NTB_ERR_ARG;
    f.rs_flags[r] = reinterpret_cast<uint32_t*>(flag_ptrs[r]);
  }
  f.done_counter = done_counter;
  const int tiles_m = (M + BLOCK_M - 1) / BLOCK_M;
  f.m_rot = ((((me + 1) % world) * rs_rows) / BLOCK_M) % tiles_m;  // the next rank's rows first, our own last
  if (num_sms <= 0) num_sms = 148;
  return b_mn ? launch<false, true, OUT_PEER_BF16>(ta, tb, td, M, N, K, status, num_sms, stream, f, GroupArgs(), &pm)
              : launch<false, false, OUT_PEER_BF16>(ta, tb, td, M, N, K, status, num_sms, stream, f, GroupArgs(), &pm);
}

// out[rs_rows, N] = sum of the `world` staging slots once every peer published `epoch`.
NTB_EXPORT int ntb_tp_reduce_slots(const void* staging, void* out, const uint32_t* flags, int world, long long elems, uint32_t epoch,
                                   unsigned long long limit_ns, int* status, cudaStream_t stream) {
  if (world < 1 || world > TP_MAX || elems <= 0 || elems % 8) return NTB_ERR_ARG;
  long long blocks = (elems / 8 + 255) / 256;
  if (blocks > 148 * 4) blocks = 148 * 4;
  rs_reduce_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(staging), reinterpret_cast<__nv_bfloat16*>(out), flags, world,
                                                                       elems, elems, epoch, limit_ns, status);
  return ntb_check_launch();
}
