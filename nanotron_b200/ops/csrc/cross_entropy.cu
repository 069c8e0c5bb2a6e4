// Vocabulary-parallel cross entropy pieces (sm_100a).
//
// ce_partials: per row of the local logits shard, an online-softmax pass producing (max, sum exp(l - max), target
// logit if the target falls in this shard else 0).  Ranks combine these three numbers; logits are read once.
// ce_backward: d logits = coef * exp(l - logZ) - g * onehot(target), written in place over the logits (the loss is
// their only consumer), so no gradient tensor of vocabulary size is allocated.
#include "common.cuh"

namespace {

constexpr int CE_THREADS = 512;

template <typename T>
__global__ void __launch_bounds__(CE_THREADS) ce_partials_kernel(const T* __restrict__ logits, const int64_t* __restrict__ target, float* __restrict__ out_max,
                                                                  float* __restrict__ out_sum, float* __restrict__ out_tgt, int vocab, int64_t vocab_start) {
  __shared__ float scratch[32];
  const int64_t row = blockIdx.x;
  const T* l = logits + row * vocab;
  float m = -INFINITY, s = 0.f;
  const int vec_end = (vocab / 8) * 8;
  for (int c = threadIdx.x * 8; c < vec_end; c += CE_THREADS * 8) {
    Vec8<T> v;
    float f[8];
    v.load(l + c);
    v.to_float(f);
    float lm = f[0];
#pragma unroll
    for (int i = 1; i < 8; i++) lm = fmaxf(lm, f[i]);
    const float nm = fmaxf(m, lm);
    float add = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) add += __expf(f[i] - nm);
    s = s * __expf(m - nm) + add;
    m = nm;
  }
  for (int c = vec_end + threadIdx.x; c < vocab; c += CE_THREADS) {
    const float f = to_f<T>(l[c]);
    const float nm = fmaxf(m, f);
    s = s * __expf(m - nm) + __expf(f - nm);
    m = nm;
  }
  const float gm = block_max(m, scratch);
  const float contrib = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  const float gs = block_sum(contrib, scratch);
  if (threadIdx.x == 0) {
    out_max[row] = gm;
    out_sum[row] = gs;
    const int64_t t = target[row] - vocab_start;
    out_tgt[row] = (t >= 0 && t < vocab) ? to_f<T>(l[t]) : 0.f;
  }
}

// grad may alias logits
template <typename T>
__global__ void __launch_bounds__(CE_THREADS) ce_backward_kernel(const T* logits, const int64_t* __restrict__ target, const float* __restrict__ logz,
                                                                  const float* __restrict__ grad_loss, const float* __restrict__ grad_z, T* grad, int vocab,
                                                                  int64_t vocab_start) {
  const int64_t row = blockIdx.x;
  const T* l = logits + row * vocab;
  T* g = grad + row * vocab;
  const float lz = logz[row];
  const float gl = grad_loss[row];
  const float coef = gl + (grad_z ? grad_z[row] : 0.f);
  const int64_t t = target[row] - vocab_start;
  const int vec_end = (vocab / 8) * 8;
  for (int c = threadIdx.x * 8; c < vec_end; c += CE_THREADS * 8) {
    Vec8<T> v;
    float f[8];
    v.load(l + c);
    v.to_float(f);
#pragma unroll
    for (int i = 0; i < 8; i++) {
      f[i] = coef * __expf(f[i] - lz);
      if (c + i == t) f[i] -= gl;
    }
    v.from_float(f);
    v.store(g + c);
  }
  for (int c = vec_end + threadIdx.x; c < vocab; c += CE_THREADS) {
    float f = coef * __expf(to_f<T>(l[c]) - lz);
    if (c == t) f -= gl;
    g[c] = from_f<T>(f);
  }
}

constexpr int CE_MAX_RANKS = 8;
struct CePeers {
  const float* p[CE_MAX_RANKS];
};

// Tensor-parallel reduction of the per-rank (max, sum exp, target logit) triples by peer loads: every rank reads the [3, rows]
// partial arrays of all ranks (after a cross-rank barrier made them visible) and finishes logZ and the loss locally, in the
// same fixed rank order everywhere, so all ranks get bit-identical results without a collective.
__global__ void ce_combine_peers_kernel(CePeers parts, int world, int64_t rows, int64_t pitch, float* __restrict__ logz, float* __restrict__ loss) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= rows) return;
  float m[CE_MAX_RANKS], s[CE_MAX_RANKS], t = 0.f, gmax = -INFINITY;
#pragma unroll
  for (int r = 0; r < CE_MAX_RANKS; r++) {
    if (r < world) {
      float tv;
      asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(m[r]) : "l"(parts.p[r] + i) : "memory");
      asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(s[r]) : "l"(parts.p[r] + pitch + i) : "memory");
      asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(tv) : "l"(parts.p[r] + 2 * pitch + i) : "memory");
      t += tv;
      gmax = fmaxf(gmax, m[r]);
    }
  }
  float sum = 0.f;
#pragma unroll
  for (int r = 0; r < CE_MAX_RANKS; r++)
    if (r < world) sum += s[r] * __expf(m[r] - gmax);
  const float lz = gmax + __logf(sum);
  logz[i] = lz;
  loss[i] = lz - t;
}

}  // namespace

// part_ptrs[r]: rank r's partial array, laid out [3][pitch] fp32 (max, sum exp, target logit), `rows` valid entries per plane.
NTB_EXPORT int ntb_ce_combine_peers(const uint64_t* part_ptrs, int world, int64_t rows, int64_t pitch, float* logz, float* loss, cudaStream_t stream) {
  if (world < 1 || world > CE_MAX_RANKS || rows <= 0 || pitch < rows) return NTB_ERR_ARG;
  CePeers pp;
  for (int r = 0; r < CE_MAX_RANKS; r++) pp.p[r] = r < world ? reinterpret_cast<const float*>(part_ptrs[r]) : nullptr;
  ce_combine_peers_kernel<<<static_cast<unsigned>((rows + 255) / 256), 256, 0, stream>>>(pp, world, rows, pitch, logz, loss);
  return ntb_check_launch();
}

NTB_EXPORT int ntb_ce_partials(int dtype, const void* logits, const int64_t* target, float* out_max, float* out_sum, float* out_tgt, int64_t rows,
                               int vocab, int64_t vocab_start, cudaStream_t stream) {
  if (rows <= 0 || vocab <= 0) return NTB_ERR_ARG;
  if (vocab % 8 != 0 || (reinterpret_cast<uintptr_t>(logits) & 15)) return NTB_ERR_ARG;  // rows must stay 16-byte aligned
  NTB_DISPATCH_DTYPE(dtype, { ce_partials_kernel<T><<<(unsigned)rows, CE_THREADS, 0, stream>>>((const T*)logits, target, out_max, out_sum, out_tgt, vocab, vocab_start); });
  return ntb_check_launch();
}

NTB_EXPORT int ntb_ce_backward(int dtype, const void* logits, const int64_t* target, const float* logz, const float* grad_loss, const float* grad_z,
                               void* grad, int64_t rows, int vocab, int64_t vocab_start, cudaStream_t stream) {
  if (rows <= 0 || vocab <= 0) return NTB_ERR_ARG;
  if (vocab % 8 != 0 || ((reinterpret_cast<uintptr_t>(logits) | reinterpret_cast<uintptr_t>(grad)) & 15)) return NTB_ERR_ARG;
  NTB_DISPATCH_DTYPE(dtype, { ce_backward_kernel<T><<<(unsigned)rows, CE_THREADS, 0, stream>>>((const T*)logits, target, logz, grad_loss, grad_z, (T*)grad, vocab, vocab_start); });
  return ntb_check_launch();
}
