// RMSNorm / LayerNorm forward and backward with optional fused residual add (sm_100a).
//
// Forward: one CTA per row; the row is staged once in shared memory (fp32) so DRAM sees exactly one read of x
// (and of the residual) and one write of y (and of the new residual).  Statistics are fp32.
// Backward: a persistent grid; each CTA walks rows with a grid stride, keeps per-column partial sums of dW (and dB)
// in shared memory, and writes them to a [gridDim.x, cols] fp32 scratch that a second small kernel reduces.
#include "common.cuh"

namespace {

constexpr int NORM_THREADS = 256;

template <typename T, bool RMS>
__global__ void __launch_bounds__(NORM_THREADS) norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ residual, const T* __restrict__ w,
                                                               const T* __restrict__ b, T* __restrict__ y, T* __restrict__ pre_out,
                                                               float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows, int cols, float eps) {
  extern __shared__ float srow[];  // cols floats
  __shared__ float scratch[32];
  const int row = blockIdx.x;
  if (row >= rows) return;
  const T* xr = x + (size_t)row * cols;
  const T* rr = residual ? residual + (size_t)row * cols : nullptr;
  float sum = 0.f, sumsq = 0.f;
  for (int c = threadIdx.x * 8; c < cols; c += NORM_THREADS * 8) {
    Vec8<T> v;
    float f[8];
    v.load(xr + c);
    v.to_float(f);
    if (rr) {
      Vec8<T> r;
      float g[8];
      r.load(rr + c);
      r.to_float(g);
#pragma unroll
      for (int i = 0; i < 8; i++) f[i] += g[i];
      // the residual stream is kept in the activation dtype: round once, and normalise the rounded value so that
      // backward (which only sees the stored tensor) is consistent with forward
      Vec8<T> o;
      o.from_float(f);
      o.store(pre_out + (size_t)row * cols + c);
      o.to_float(f);
    }
#pragma unroll
    for (int i = 0; i < 8; i++) { srow[c + i] = f[i]; sum += f[i]; sumsq += f[i] * f[i]; }
  }
  float mean = 0.f, var;
  if (RMS) {
    var = block_sum(sumsq, scratch) / cols;
  } else {
    mean = block_sum(sum, scratch) / cols;
    // second pass over the staged row for a numerically safe variance
    float d2 = 0.f;
    for (int c = threadIdx.x * 8; c < cols; c += NORM_THREADS * 8) {
#pragma unroll
      for (int i = 0; i < 8; i++) { float d = srow[c + i] - mean; d2 += d * d; }
    }
    var = block_sum(d2, scratch) / cols;
  }
  const float rstd = rsqrtf(var + eps);
  if (threadIdx.x == 0) {
    rstd_out[row] = rstd;
    if (!RMS) mean_out[row] = mean;
  }
  T* yr = y + (size_t)row * cols;
  for (int c = threadIdx.x * 8; c < cols; c += NORM_THREADS * 8) {
    Vec8<T> wv, o;
    float wf[8], f[8];
    wv.load(w + c);
    wv.to_float(wf);
#pragma unroll
    for (int i = 0; i < 8; i++) f[i] = (srow[c + i] - mean) * rstd * wf[i];
    if (!RMS && b) {
      Vec8<T> bv;
      float bf[8];
      bv.load(b + c);
      bv.to_float(bf);
#pragma unroll
      for (int i = 0; i < 8; i++) f[i] += bf[i];
    }
    o.from_float(f);
    o.store(yr + c);
  }
}

// Backward.  Thread t owns columns {(it*NORM_THREADS + t)*8 .. +7 : it < ITERS}: the row slice, its dW (and dB) partial
// sums all live in registers, so a row costs one pass over dy / x (/ dres) and one block reduction.
template <typename T, bool RMS, int ITERS>
__global__ void __launch_bounds__(NORM_THREADS) norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ pre, const T* __restrict__ w,
                                                               const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                                                               const T* __restrict__ dres, T* __restrict__ dx, float* __restrict__ dw_partial,
                                                               float* __restrict__ db_partial, int rows, int cols) {
  __shared__ float scratch[2][32];
  float fw[ITERS][8], dw_acc[ITERS][8], db_acc[RMS ? 1 : ITERS][8];
#pragma unroll
  for (int it = 0; it < ITERS; it++) {
    const int c = (it * NORM_THREADS + threadIdx.x) * 8;
    if (c < cols) {
      Vec8<T> wv;
      wv.load(w + c);
      wv.to_float(fw[it]);
    }
#pragma unroll
    for (int i = 0; i < 8; i++) {
      dw_acc[it][i] = 0.f;
      if (!RMS) db_acc[it][i] = 0.f;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // Software pipeline over rows: the loads of row r + gridDim.x are issued before the block reduction of row r, so two
  // rows are in flight per CTA and the reduction latency is hidden behind memory latency.
  Vec8<T> n_dy[ITERS], n_x[ITERS], n_dr[ITERS];
  int row = blockIdx.x;
  if (row < rows) {
#pragma unroll
    for (int it = 0; it < ITERS; it++) {
      const int c = (it * NORM_THREADS + threadIdx.x) * 8;
      if (c < cols) {
        n_dy[it].load(dy + (size_t)row * cols + c);
        n_x[it].load(pre + (size_t)row * cols + c);
        if (dres) n_dr[it].load(dres + (size_t)row * cols + c);
      }
    }
  }
  for (; row < rows; row += gridDim.x) {
    const float rstd = rstd_in[row];
    const float mean = RMS ? 0.f : mean_in[row];
    float wdy[ITERS][8], xhat[ITERS][8];
    Vec8<T> c_dr[ITERS];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int it = 0; it < ITERS; it++) {
      const int c = (it * NORM_THREADS + threadIdx.x) * 8;
      if (c < cols) {
        float fdy[8], fx[8];
        n_dy[it].to_float(fdy);
        n_x[it].to_float(fx);
        c_dr[it] = n_dr[it];
#pragma unroll
        for (int i = 0; i < 8; i++) {
          xhat[it][i] = (fx[i] - mean) * rstd;
          wdy[it][i] = fdy[i] * fw[it][i];
          s1 += wdy[it][i] * xhat[it][i];
          s2 += wdy[it][i];
          dw_acc[it][i] += fdy[i] * xhat[it][i];
          if (!RMS) db_acc[it][i] += fdy[i];
        }
      }
    }
    const int nrow = row + gridDim.x;
    if (nrow < rows) {
#pragma unroll
      for (int it = 0; it < ITERS; it++) {
        const int c = (it * NORM_THREADS + threadIdx.x) * 8;
        if (c < cols) {
          n_dy[it].load(dy + (size_t)nrow * cols + c);
          n_x[it].load(pre + (size_t)nrow * cols + c);
          if (dres) n_dr[it].load(dres + (size_t)nrow * cols + c);
        }
      }
    }
    // one block reduction for both sums
    s1 = warp_sum(s1);
    if (!RMS) s2 = warp_sum(s2);
    float* sc = scratch[0];
    __syncthreads();
    if (lane == 0) { sc[warp] = s1; scratch[1][warp] = s2; }
    __syncthreads();
    float r1 = (lane < NORM_THREADS / 32) ? sc[lane] : 0.f;
    float r2 = (!RMS && lane < NORM_THREADS / 32) ? scratch[1][lane] : 0.f;
    const float c1 = warp_sum(r1) / cols;
    const float c2 = RMS ? 0.f : warp_sum(r2) / cols;
    T* dxr = dx + (size_t)row * cols;
#pragma unroll
    for (int it = 0; it < ITERS; it++) {
      const int c = (it * NORM_THREADS + threadIdx.x) * 8;
      if (c < cols) {
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; i++) f[i] = (wdy[it][i] - xhat[it][i] * c1 - c2) * rstd;
        if (dres) {
          float g[8];
          c_dr[it].to_float(g);
#pragma unroll
          for (int i = 0; i < 8; i++) f[i] += g[i];
        }
        Vec8<T> o;
        o.from_float(f);
        o.store(dxr + c);
      }
    }
  }
#pragma unroll
  for (int it = 0; it < ITERS; it++) {
    const int c = (it * NORM_THREADS + threadIdx.x) * 8;
    if (c < cols) {
      float* dst = dw_partial + (size_t)blockIdx.x * cols + c;
      *reinterpret_cast<float4*>(dst) = make_float4(dw_acc[it][0], dw_acc[it][1], dw_acc[it][2], dw_acc[it][3]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(dw_acc[it][4], dw_acc[it][5], dw_acc[it][6], dw_acc[it][7]);
      if (!RMS) {
        float* d2 = db_partial + (size_t)blockIdx.x * cols + c;
        *reinterpret_cast<float4*>(d2) = make_float4(db_acc[it][0], db_acc[it][1], db_acc[it][2], db_acc[it][3]);
        *reinterpret_cast<float4*>(d2 + 4) = make_float4(db_acc[it][4], db_acc[it][5], db_acc[it][6], db_acc[it][7]);
      }
    }
  }
}

// out[c] = sum_p partial[p, c].  Block = 32 columns x 8 part-lanes; coalesced 128-byte rows.
__global__ void reduce_partials_kernel(const float* __restrict__ partial, float* __restrict__ out, int nparts, int cols) {
  __shared__ float sm[8][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  float s = 0.f;
  if (c < cols)
    for (int p = threadIdx.y; p < nparts; p += 8) s += partial[(size_t)p * cols + c];
  sm[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && c < cols) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; k++) t += sm[k][threadIdx.x];
    out[c] = t;
  }
}

}  // namespace

// Number of CTAs the backward kernels use (== rows of the partial scratch the caller must provide).
NTB_EXPORT int ntb_norm_bwd_num_partials(int rows) {
  int n = 148 * 4;
  return rows < n ? rows : n;
}

NTB_EXPORT int ntb_norm_fwd(int is_rms, int dtype, const void* x, const void* residual, const void* w, const void* b, void* y, void* pre_out,
                            float* mean_out, float* rstd_out, int rows, int cols, float eps, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0 || cols % 8 != 0 || cols > 32768) return NTB_ERR_ARG;
  if (residual && !pre_out) return NTB_ERR_ARG;
  const size_t smem = (size_t)cols * sizeof(float);
  NTB_DISPATCH_DTYPE(dtype, {
    if (is_rms) {
      if (smem > 32 * 1024) cudaFuncSetAttribute(norm_fwd_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      norm_fwd_kernel<T, true><<<rows, NORM_THREADS, smem, stream>>>((const T*)x, (const T*)residual, (const T*)w, (const T*)b, (T*)y, (T*)pre_out, mean_out, rstd_out, rows, cols, eps);
    } else {
      if (smem > 32 * 1024) cudaFuncSetAttribute(norm_fwd_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      norm_fwd_kernel<T, false><<<rows, NORM_THREADS, smem, stream>>>((const T*)x, (const T*)residual, (const T*)w, (const T*)b, (T*)y, (T*)pre_out, mean_out, rstd_out, rows, cols, eps);
    }
  });
  return ntb_check_launch();
}

// dw_partial / db_partial: fp32 [ntb_norm_bwd_num_partials(rows), cols]; dw_out / db_out: fp32 [cols].
NTB_EXPORT int ntb_norm_bwd(int is_rms, int dtype, const void* dy, const void* pre, const void* w, const float* mean, const float* rstd,
                            const void* dres, void* dx, float* dw_partial, float* db_partial, float* dw_out, float* db_out, int rows, int cols,
                            cudaStream_t stream) {
  if (rows <= 0 || cols <= 0 || cols % 8 != 0 || cols > NORM_THREADS * 8 * 8) return NTB_ERR_ARG;
  const int nparts = ntb_norm_bwd_num_partials(rows);
  const int iters = (cols + NORM_THREADS * 8 - 1) / (NORM_THREADS * 8);
#define NTB_NORM_BWD(IT)                                                                                                                             \
  {                                                                                                                                                  \
    if (is_rms)                                                                                                                                      \
      norm_bwd_kernel<T, true, IT><<<nparts, NORM_THREADS, 0, stream>>>((const T*)dy, (const T*)pre, (const T*)w, mean, rstd, (const T*)dres, (T*)dx, \
                                                                         dw_partial, db_partial, rows, cols);                                       \
    else                                                                                                                                             \
      norm_bwd_kernel<T, false, IT><<<nparts, NORM_THREADS, 0, stream>>>((const T*)dy, (const T*)pre, (const T*)w, mean, rstd, (const T*)dres,       \
                                                                          (T*)dx, dw_partial, db_partial, rows, cols);                               \
  }
  NTB_DISPATCH_DTYPE(dtype, {
    if (iters <= 1) NTB_NORM_BWD(1)
    else if (iters <= 2) NTB_NORM_BWD(2)
    else if (iters <= 4) NTB_NORM_BWD(4)
    else NTB_NORM_BWD(8)
  });
#undef NTB_NORM_BWD
  int rc = ntb_check_launch();
  if (rc) return rc;
  dim3 rb(32, 8);
  reduce_partials_kernel<<<(cols + 31) / 32, rb, 0, stream>>>(dw_partial, dw_out, nparts, cols);
  if (!is_rms && db_out) reduce_partials_kernel<<<(cols + 31) / 32, rb, 0, stream>>>(db_partial, db_out, nparts, cols);
  return ntb_check_launch();
}

// ------------------------------------------------------------------------------------------------------------------
// RMSNorm backward for callers that must not allocate (declared in ntb_noalloc.h).
//
// The regular entry point above needs a caller-provided fp32 scratch of [partials, cols] for the per-CTA partial sums of
// dW.  Some callers cannot provide one: library hooks invoked from inside another framework's allocator callbacks, and
// runtimes that pre-plan every byte of device memory and forbid cudaMalloc (and torch's caching allocator) after start-up.  For them this variant keeps the
// scratch in a fixed array that is part of the loaded library image: every GPU on which this module gets loaded holds
// NTB_NOALLOC_PARTIALS * NTB_NOALLOC_MAX_COLS * 4 bytes (4.6 MiB) from that moment until the process exits.  The CUDA
// runtime loads modules lazily, so "that moment" is the first use of this library's kernels or symbols on the device.
//
// The array's name is only a host-side handle; the device address is looked up with cudaGetSymbolAddress the first time
// the entry point is called on each device (with that device current).  That first call should therefore come at
// start-up: before memory is frozen (it may be what loads the module and reserves the array) and before any stream
// capture.  The per-device address table below is written without a lock; racing first calls store the same value.  All calls share the one array: two calls whose kernels overlap on the GPU (different streams
// without ordering) would mix their partial sums.  Nothing in the array has to start at zero: every launch rewrites
// the rows it reads back.
constexpr int NTB_NOALLOC_PARTIALS = 148;
constexpr int NTB_NOALLOC_MAX_COLS = 8192;
static __device__ __align__(256) float g_noalloc_dw_partials[NTB_NOALLOC_PARTIALS * NTB_NOALLOC_MAX_COLS];
static float* g_noalloc_dw_ptr[64] = {};

NTB_EXPORT int ntb_rmsnorm_bwd_noalloc_max_cols() { return NTB_NOALLOC_MAX_COLS; }

NTB_EXPORT int ntb_rmsnorm_bwd_noalloc(int dtype, const void* dy, const void* pre, const void* w, const float* rstd, const void* dres, void* dx, float* dw_out,
                                       int rows, int cols, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0 || cols % 8 != 0) return NTB_ERR_ARG;
  if (cols > NTB_NOALLOC_MAX_COLS) return NTB_ERR_ARG;  // larger rows do not fit the built-in scratch: use ntb_norm_bwd
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return NTB_ERR_LAUNCH;
  if (g_noalloc_dw_ptr[dev] == nullptr) {
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_dw_partials) != cudaSuccess || p == nullptr) return NTB_ERR_LAUNCH;
    g_noalloc_dw_ptr[dev] = p;
  }
  float* partial = g_noalloc_dw_ptr[dev];
  const int nparts = rows < NTB_NOALLOC_PARTIALS ? rows : NTB_NOALLOC_PARTIALS;
  const int iters = (cols + NORM_THREADS * 8 - 1) / (NORM_THREADS * 8);
#define NTB_NORM_BWD_NA(IT) \
  norm_bwd_kernel<T, true, IT><<<nparts, NORM_THREADS, 0, stream>>>((const T*)dy, (const T*)pre, (const T*)w, nullptr, rstd, (const T*)dres, (T*)dx, partial, nullptr, rows, cols);
  NTB_DISPATCH_DTYPE(dtype, {
    if (iters <= 1) { NTB_NORM_BWD_NA(1) }
    else if (iters <= 2) { NTB_NORM_BWD_NA(2) }
    else { NTB_NORM_BWD_NA(4) }
  });
#undef NTB_NORM_BWD_NA
  int rc = ntb_check_launch();
  if (rc) return rc;
  dim3 rb(32, 8);
  reduce_partials_kernel<<<(cols + 31) / 32, rb, 0, stream>>>(partial, dw_out, nparts, cols);
  return ntb_check_launch();
}
