// Block-scaled fp8 GEMM on the 5th-generation tensor cores (tcgen05 kind::f8f6f4 + TMEM + TMA), sm_100a.
//
//   D[M,N] (=|+=) sum over 128-wide k-blocks kb of  sa(m, kb) * sb(n, kb) * ( A8[m, kb-block] . B8[n, kb-block] )
//
// A8 / B8 are fp8 payloads (e4m3 or e5m2, chosen per operand), both K-major ([rows, K] with K contiguous).  sa is one fp32
// scale per row per k-block (1 x 128 quantisation); sb is either one scale per 128 rows per k-block (128 x 128 weight blocks)
// or one per row per k-block (operands quantised along the reduction dimension, as the weight gradient needs).
//
// The tensor core cannot apply per-k-block scales itself, so each k-block's product is formed on its own in TMEM
// (accumulate flag off on its first instruction) and promoted by the epilogue warps: tcgen05.ld -> multiply by the two scales
// -> add into fp32 registers.  Two 256-column TMEM buffers alternate, so the MMAs of k-block i+1 run while k-block i is promoted.
// Warp roles: warp 0 TMA producer (4-stage ring of {A 128x128 B, B 256x128 B}), warp 1 MMA issuer (four 128x256x32 MMAs per
// k-block), then the promotion + write-out warps: 8 (two per TMEM lane quarter, 128 columns and 128 fp32 accumulators per thread;
// the default) or 16 (four per quarter, 64 columns each).  All waits are bounded; on expiry the kernel raises `status`, drains,
// frees TMEM and returns.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace {

constexpr int F8_BLOCK_M = 128;
constexpr int F8_BLOCK_N = 256;
constexpr int F8_BLOCK_K = 128;  // one 128-byte swizzle row of fp8 = one scaling block
constexpr int F8_UMMA_K = 32;
constexpr int F8_STAGES = 4;
constexpr int F8_A_BYTES = F8_BLOCK_M * F8_BLOCK_K;
constexpr int F8_B_BYTES = F8_BLOCK_N * F8_BLOCK_K;
constexpr int F8_STAGE_BYTES = F8_A_BYTES + F8_B_BYTES;  // 48 KiB
constexpr int F8_SB_SMEM = 4 * F8_BLOCK_N * 4;  // per-warp staging of its per-row B scales (4 lane quarters x 256 columns)
constexpr int F8_SMEM_BYTES = F8_STAGES * F8_STAGE_BYTES + F8_SB_SMEM + 1024 + 256;

enum F8Out { F8_OUT_BF16 = 0, F8_OUT_F32_ACCUM = 2 };

struct F8Scales {
  const float* sa;   // [M, KB]
  const float* sb;   // [ceil(N / 128), KB] (SB_ROW false) or [N, KB] (SB_ROW true)
  int kb_total;
};

__host__ __device__ constexpr uint32_t make_idesc_fp8(int m, int n, int a_e5m2, int b_e5m2) {
  return (1u << 4) | (static_cast<uint32_t>(a_e5m2) << 7) | (static_cast<uint32_t>(b_e5m2) << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <bool SB_ROW, int OUT, int F8_EPI_WARPS>
__global__ void __launch_bounds__(32 * (2 + F8_EPI_WARPS), 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, void* __restrict__ d, int64_t ldd, int M, int N, int K,
                F8Scales sc, uint32_t idesc, int* __restrict__ status) {
  constexpr int F8_WCOLS = F8_BLOCK_N / (F8_EPI_WARPS / 4);  // columns per promotion warp: 128 (8 warps) or 64 (16 warps)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* sb_smem = reinterpret_cast<float*>(smem + F8_STAGES * F8_STAGE_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + F8_STAGES * F8_STAGE_BYTES + F8_SB_SMEM);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + F8_STAGES;
  uint64_t* part_full = bars + 2 * F8_STAGES;   // [2]
  uint64_t* part_empty = part_full + 2;         // [2]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(part_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + F8_BLOCK_M - 1) / F8_BLOCK_M;
  const int tiles_n = (N + F8_BLOCK_N - 1) / F8_BLOCK_N;
  const int num_tiles = tiles_m * tiles_n;
  const int k_blocks = (K + F8_BLOCK_K - 1) / F8_BLOCK_K;

  if (threadIdx.x == 0) {
    for (int s = 0; s < F8_STAGES; s++) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; b++) {
      ptx::mbar_init(&part_full[b], 1);
      ptx::mbar_init(&part_empty[b], F8_EPI_WARPS);
    }
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tmap(&tmap_a);
    ptx::prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_base_slot, 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    if (ptx::elect_one()) {
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int m_blk = t % tiles_m, n_blk = t / tiles_m;  // consecutive CTAs share the B tile
        for (int kb = 0; kb < k_blocks; kb++, it++) {
          const int s = it % F8_STAGES;
          const uint32_t ph = (it / F8_STAGES) & 1;
          if (!ptx::mbar_wait(&empty_bar[s], ph ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + s * F8_STAGE_BYTES;
          ptx::mbar_expect_tx(&full_bar[s], F8_STAGE_BYTES);
          ptx::tma_load_2d(sa, &tmap_a, &full_bar[s], kb * F8_BLOCK_K, m_blk * F8_BLOCK_M);
          ptx::tma_load_2d(sa + F8_A_BYTES, &tmap_b, &full_bar[s], kb * F8_BLOCK_K, n_blk * F8_BLOCK_N);
        }
      }
      if (!ok) {
        const uint64_t t0 = ptx::globaltimer();
        for (int s = 0; s < F8_STAGES; s++) {
          const int last = it - 1 - ((it - 1 - s) % F8_STAGES + F8_STAGES) % F8_STAGES;
          if (it == 0 || last < 0) continue;
          const uint32_t ph = (last / F8_STAGES) & 1;
          while (!ptx::mbar_try_wait(&full_bar[s], ph) && ptx::globaltimer() - t0 < NTB_WAIT_LIMIT_NS) {}
        }
      }
    }
  } else if (warp == 1) {
    if (ptx::elect_one()) {
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        for (int kb = 0; kb < k_blocks; kb++, it++) {
          const int s = it % F8_STAGES;
          const uint32_t ph = (it / F8_STAGES) & 1;
          const int pb = it & 1;
          const uint32_t pph = (it >> 1) & 1;
          if (!ptx::mbar_wait(&part_empty[pb], pph ^ 1, abort_flag)) { ok = false; break; }
          if (!ptx::mbar_wait(&full_bar[s], ph, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t sa = ptx::smem_u32(smem + s * F8_STAGE_BYTES);
          const uint32_t sb = sa + F8_A_BYTES;
          const uint32_t tmem_d = tmem_base + pb * F8_BLOCK_N;
#pragma unroll
          for (int k = 0; k < F8_BLOCK_K / F8_UMMA_K; k++)
            umma_f8(tmem_d, ptx::make_smem_desc(sa + k * F8_UMMA_K, 16, 1024), ptx::make_smem_desc(sb + k * F8_UMMA_K, 16, 1024), idesc, k != 0 ? 1u : 0u);
          ptx::umma_commit(&empty_bar[s]);
          ptx::umma_commit(&part_full[pb]);
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- promotion + write-out
    const int ew = warp - 2;
    const int q = warp & 3;          // TMEM lane quarter this warp may read
    const int cgrp = ew >> 2;        // which 64 columns of the 256-wide tile
    float* my_sb = sb_smem + ew * F8_WCOLS;
    int it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      const int m_blk = t % tiles_m, n_blk = t / tiles_m;
      const int row = m_blk * F8_BLOCK_M + q * 32 + lane;
      const int col0 = n_blk * F8_BLOCK_N + cgrp * F8_WCOLS;
      const bool row_ok = row < M;
      float acc[F8_WCOLS];
#pragma unroll
      for (int i = 0; i < F8_WCOLS; i++) acc[i] = 0.f;
      const float* sa_row = sc.sa + static_cast<int64_t>(row_ok ? row : 0) * sc.kb_total;
      float sa_next = row_ok ? __ldg(sa_row) : 0.f;
      for (int kb = 0; kb < k_blocks; kb++, it++) {
        const int pb = it & 1;
        const uint32_t pph = (it >> 1) & 1;
        const float sa_cur = sa_next;
        if (kb + 1 < k_blocks) sa_next = row_ok ? __ldg(sa_row + kb + 1) : 0.f;
        float sb_blk = 0.f;
        if (SB_ROW) {
          // stage this warp's per-row B scales for the k-block in shared memory
          __syncwarp();
#pragma unroll
          for (int i = 0; i < F8_WCOLS / 32; i++) {
            const int c = col0 + i * 32 + lane;
            my_sb[i * 32 + lane] = c < N ? __ldg(sc.sb + static_cast<int64_t>(c) * sc.kb_total + kb) : 0.f;
          }
          __syncwarp();
        } else {
          sb_blk = col0 < N ? __ldg(sc.sb + static_cast<int64_t>(col0 >> 7) * sc.kb_total + kb) : 0.f;
        }
        if (!ptx::mbar_wait(&part_full[pb], pph, abort_flag)) { ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + pb * F8_BLOCK_N + cgrp * F8_WCOLS;
        const float s_ab = sa_cur * sb_blk;
#pragma unroll
        for (int c = 0; c < F8_WCOLS / 32; c++) {
          uint32_t r[32];
          ptx::tmem_ld_32x32(taddr + c * 32, r);
          ptx::tmem_ld_wait();
          if (c == F8_WCOLS / 32 - 1) {
            // the whole partial product has been read: give the TMEM buffer back to the MMA warp before the last arithmetic
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&part_empty[pb]);
          }
          float* a0 = acc + c * 32;
          if (SB_ROW) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              const float4 sv = *reinterpret_cast<const float4*>(my_sb + c * 32 + j);
              a0[j + 0] = fmaf(__uint_as_float(r[j + 0]) * sv.x, sa_cur, a0[j + 0]);
              a0[j + 1] = fmaf(__uint_as_float(r[j + 1]) * sv.y, sa_cur, a0[j + 1]);
              a0[j + 2] = fmaf(__uint_as_float(r[j + 2]) * sv.z, sa_cur, a0[j + 2]);
              a0[j + 3] = fmaf(__uint_as_float(r[j + 3]) * sv.w, sa_cur, a0[j + 3]);
            }
          } else {
            // one weight scale per 128 columns: a promotion warp never straddles two blocks (col0 is a multiple of its width)
#pragma unroll
            for (int j = 0; j < 32; j++) a0[j] = fmaf(__uint_as_float(r[j]), s_ab, a0[j]);
          }
        }
      }
      if (!ok) break;
      if (row_ok) {
        if (OUT == F8_OUT_BF16) {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(d) + static_cast<int64_t>(row) * ldd + col0;
#pragma unroll
          for (int c = 0; c < F8_WCOLS; c += 8) {
            if (col0 + c < N) {
              uint4 pk;
              __nv_bfloat162 h0 = __floats2bfloat162_rn(acc[c], acc[c + 1]), h1 = __floats2bfloat162_rn(acc[c + 2], acc[c + 3]);
              __nv_bfloat162 h2 = __floats2bfloat162_rn(acc[c + 4], acc[c + 5]), h3 = __floats2bfloat162_rn(acc[c + 6], acc[c + 7]);
              pk.x = *reinterpret_cast<uint32_t*>(&h0); pk.y = *reinterpret_cast<uint32_t*>(&h1);
              pk.z = *reinterpret_cast<uint32_t*>(&h2); pk.w = *reinterpret_cast<uint32_t*>(&h3);
              *reinterpret_cast<uint4*>(dst + c) = pk;
            }
          }
        } else {
          float* dst = reinterpret_cast<float*>(d) + static_cast<int64_t>(row) * ldd + col0;
#pragma unroll
          for (int c = 0; c < F8_WCOLS; c += 4) {
            if (col0 + c < N) {
              float4 v = *reinterpret_cast<float4*>(dst + c);
              v.x += acc[c]; v.y += acc[c + 1]; v.z += acc[c + 2]; v.w += acc[c + 3];
              *reinterpret_cast<float4*>(dst + c) = v;
            }
          }
        }
      }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_flag && status) atomicExch(status, NTB_ERR_TIMEOUT);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn f8_get_encode() {
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

// fp8 K-major operand [rows, k] with pitch ld bytes: 2-D map {k, rows}, box {128, box_rows}; out-of-range elements read as zero.
bool f8_make_map(CUtensorMap* m, const void* ptr, int64_t rows, int64_t k, int64_t ld, int box_rows) {
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld};
  cuuint32_t box[2] = {128, (cuuint32_t)box_rows};
  cuuint32_t es[2] = {1, 1};
  return f8_get_encode()(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <bool SB_ROW, int OUT, int EW>
int f8_launch(const CUtensorMap& ta, const CUtensorMap& tb, void* d, int64_t ldd, int M, int N, int K, const F8Scales& sc, uint32_t idesc, int* status, int num_sms,
              cudaStream_t stream) {
  auto kern = gemm_fp8_kernel<SB_ROW, OUT, EW>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, F8_SMEM_BYTES) != cudaSuccess) return NTB_ERR_LAUNCH;
    configured = true;
  }
  const long long tiles = static_cast<long long>((M + F8_BLOCK_M - 1) / F8_BLOCK_M) * ((N + F8_BLOCK_N - 1) / F8_BLOCK_N);
  const int grid = tiles < num_sms ? static_cast<int>(tiles) : num_sms;
  kern<<<grid, 32 * (2 + EW), F8_SMEM_BYTES, stream>>>(ta, tb, d, ldd, M, N, K, sc, idesc, status);
  return ntb_check_launch();
}

}  // namespace

// a: fp8 [M, K] (pitch lda bytes), sa: fp32 [M, ceil(K / 128)].  b: fp8 [N, K] (pitch ldb), sb: fp32 [ceil(N / 128), ceil(K / 128)] when
// sb_per_row == 0, [N, ceil(K / 128)] when 1.  a_e5m2 / b_e5m2 select the payload format (0 = e4m3).  d: bf16 [M, N] (out_mode 0, stored)
// or fp32 [M, N] (out_mode 2, accumulated into); ldd in elements.  K must be a multiple of 16 (TMA pitch); N a multiple of 8.
NTB_EXPORT int ntb_gemm_fp8_blockscaled(const void* a, const float* sa, const void* b, const float* sb, void* d, int M, int N, int K, int64_t lda, int64_t ldb,
                                        int64_t ldd, int a_e5m2, int b_e5m2, int sb_per_row, int out_mode, int epi_warps, int* status, int num_sms,
                                        cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || !f8_get_encode() || !sa || !sb) return NTB_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(d)) & 15) return NTB_ERR_ARG;
  if (lda % 16 || ldb % 16 || N % 8 || (out_mode == F8_OUT_BF16 ? ldd % 8 : ldd % 4) || (out_mode != F8_OUT_BF16 && out_mode != F8_OUT_F32_ACCUM)) return NTB_ERR_ARG;
  CUtensorMap ta, tb;
  if (!f8_make_map(&ta, a, M, K, lda, F8_BLOCK_M) || !f8_make_map(&tb, b, N, K, ldb, F8_BLOCK_N)) return NTB_ERR_ARG;
  F8Scales sc;
  sc.sa = sa;
  sc.sb = sb;
  sc.kb_total = (K + F8_BLOCK_K - 1) / F8_BLOCK_K;
  const uint32_t idesc = make_idesc_fp8(F8_BLOCK_M, F8_BLOCK_N, a_e5m2 ? 1 : 0, b_e5m2 ? 1 : 0);
  if (num_sms <= 0) num_sms = 148;
  // epi_warps: 8 (128 columns per promotion warp) or 16 (64 columns per warp); 0 picks the default
#define NTB_F8_CASE(SBR, OM, EW) \
  if ((sb_per_row != 0) == SBR && out_mode == OM && epi_warps == EW) return f8_launch<SBR, OM, EW>(ta, tb, d, ldd, M, N, K, sc, idesc, status, num_sms, stream);
  if (epi_warps == 0) epi_warps = 8;
  NTB_F8_CASE(false, F8_OUT_BF16, 8) NTB_F8_CASE(false, F8_OUT_F32_ACCUM, 8) NTB_F8_CASE(true, F8_OUT_BF16, 8) NTB_F8_CASE(true, F8_OUT_F32_ACCUM, 8)
  NTB_F8_CASE(false, F8_OUT_BF16, 16) NTB_F8_CASE(false, F8_OUT_F32_ACCUM, 16) NTB_F8_CASE(true, F8_OUT_BF16, 16) NTB_F8_CASE(true, F8_OUT_F32_ACCUM, 16)
#undef NTB_F8_CASE
  return NTB_ERR_ARG;
}
