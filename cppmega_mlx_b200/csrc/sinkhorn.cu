// Sinkhorn normalisation of small square matrices (the mHC branch mixer's transport matrix), forward and backward in one
// launch each instead of ~6 element-wise launches per iteration.
//
//   t0 = softmax(raw) over the row index (every column sums to 1)
//   repeat `iters` times:  t ← t / max(rowsum(t), eps);  t ← t / max(colsum(t), eps)
//
// One thread owns one n×n matrix (n ≤ 8) in registers; the backward re-runs the forward keeping every intermediate in
// thread-local memory (at most (2·16 + 1)·64 floats) and walks it in reverse.  The matrices are few (one per batch entry), so
// the point is the launch count, not bandwidth.  Math: cppmega_mlx/nn/mhc.py:62 (sinkhorn_normalize).
#include <cuda_runtime.h>

namespace cmb {

constexpr int SK_MAX_ITERS = 16;

template <int N>
__device__ __forceinline__ void sk_softmax_cols(const float* x, float* y) {
#pragma unroll
  for (int j = 0; j < N; ++j) {
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < N; ++i) m = fmaxf(m, x[i * N + j]);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < N; ++i) {
      const float e = __expf(x[i * N + j] - m);
      y[i * N + j] = e;
      s += e;
    }
    const float inv = 1.f / s;
#pragma unroll
    for (int i = 0; i < N; ++i) y[i * N + j] *= inv;
  }
}

// y = x / max(sum over the normalised axis, eps); ROWS: the sum runs over j for each i.
template <int N, bool ROWS>
__device__ __forceinline__ void sk_norm(const float* x, float* y, float eps) {
#pragma unroll
  for (int a = 0; a < N; ++a) {
    float s = 0.f;
#pragma unroll
    for (int b = 0; b < N; ++b) s += ROWS ? x[a * N + b] : x[b * N + a];
    const float inv = 1.f / fmaxf(s, eps);
#pragma unroll
    for (int b = 0; b < N; ++b) {
      const int k = ROWS ? a * N + b : b * N + a;
      y[k] = x[k] * inv;
    }
  }
}

// Gradient of sk_norm: with s > eps, dx_k = (g_k − Σ_b g_b·y_b) / s over the normalised axis; with the clamp active, g / eps.
template <int N, bool ROWS>
__device__ __forceinline__ void sk_norm_bwd(const float* x, const float* y, float* g, float eps) {
#pragma unroll
  for (int a = 0; a < N; ++a) {
    float s = 0.f, dot = 0.f;
#pragma unroll
    for (int b = 0; b < N; ++b) {
      const int k = ROWS ? a * N + b : b * N + a;
      s += x[k];
      dot += g[k] * y[k];
    }
    const bool clamped = s <= eps;
    const float inv = 1.f / fmaxf(s, eps);
#pragma unroll
    for (int b = 0; b < N; ++b) {
      const int k = ROWS ? a * N + b : b * N + a;
      g[k] = clamped ? g[k] * inv : (g[k] - dot) * inv;
    }
  }
}

template <int N>
__global__ void __launch_bounds__(128) sinkhorn_fwd_kernel(const float* __restrict__ raw, float* __restrict__ out, long long count, int iters,
                                                           float eps) {
  const long long m = blockIdx.x * 128ll + threadIdx.x;
  if (m >= count) return;
  float a[N * N], b[N * N];
#pragma unroll
  for (int k = 0; k < N * N; ++k) a[k] = raw[m * N * N + k];
  sk_softmax_cols<N>(a, b);
  for (int it = 0; it < iters; ++it) {
    sk_norm<N, true>(b, a, eps);
    sk_norm<N, false>(a, b, eps);
  }
#pragma unroll
  for (int k = 0; k < N * N; ++k) out[m * N * N + k] = b[k];
}

template <int N>
__global__ void __launch_bounds__(128) sinkhorn_bwd_kernel(const float* __restrict__ raw, const float* __restrict__ gout, float* __restrict__ graw,
                                                           long long count, int iters, float eps) {
  const long long m = blockIdx.x * 128ll + threadIdx.x;
  if (m >= count) return;
  float hist[2 * SK_MAX_ITERS + 1][N * N];      // hist[0] = softmax, hist[2t+1] = after the row step, hist[2t+2] = after the column step
  float x[N * N], g[N * N];
#pragma unroll
  for (int k = 0; k < N * N; ++k) x[k] = raw[m * N * N + k];
  sk_softmax_cols<N>(x, hist[0]);
  for (int it = 0; it < iters; ++it) {
    sk_norm<N, true>(hist[2 * it], hist[2 * it + 1], eps);
    sk_norm<N, false>(hist[2 * it + 1], hist[2 * it + 2], eps);
  }
#pragma unroll
  for (int k = 0; k < N * N; ++k) g[k] = gout[m * N * N + k];
  for (int it = iters - 1; it >= 0; --it) {
    sk_norm_bwd<N, false>(hist[2 * it + 1], hist[2 * it + 2], g, eps);
    sk_norm_bwd<N, true>(hist[2 * it], hist[2 * it + 1], g, eps);
  }
  // softmax over the row index of each column: dx = y ∘ (g − Σ_i g_i·y_i)
#pragma unroll
  for (int j = 0; j < N; ++j) {
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < N; ++i) dot += g[i * N + j] * hist[0][i * N + j];
#pragma unroll
    for (int i = 0; i < N; ++i) graw[m * N * N + i * N + j] = hist[0][i * N + j] * (g[i * N + j] - dot);
  }
}

}  // namespace cmb

// raw, out: fp32 [count, n, n] contiguous; 2 <= n <= 8; 0 <= iters <= 16.
extern "C" int cmb_sinkhorn_fwd(const float* raw, float* out, long long count, int n, int iters, float eps, void* stream) {
  if (n < 2 || n > 8 || iters < 0 || iters > cmb::SK_MAX_ITERS || eps <= 0.f) return 1;
  if (count <= 0) return 0;
  const unsigned grid = static_cast<unsigned>((count + 127) / 128);
  auto st = static_cast<cudaStream_t>(stream);
  switch (n) {
#define CMB_SK_CASE(N_) case N_: cmb::sinkhorn_fwd_kernel<N_><<<grid, 128, 0, st>>>(raw, out, count, iters, eps); break;
    CMB_SK_CASE(2) CMB_SK_CASE(3) CMB_SK_CASE(4) CMB_SK_CASE(5) CMB_SK_CASE(6) CMB_SK_CASE(7) CMB_SK_CASE(8)
#undef CMB_SK_CASE
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

extern "C" int cmb_sinkhorn_bwd(const float* raw, const float* gout, float* graw, long long count, int n, int iters, float eps, void* stream) {
  if (n < 2 || n > 8 || iters < 0 || iters > cmb::SK_MAX_ITERS || eps <= 0.f) return 1;
  if (count <= 0) return 0;
  const unsigned grid = static_cast<unsigned>((count + 127) / 128);
  auto st = static_cast<cudaStream_t>(stream);
  switch (n) {
#define CMB_SK_CASE(N_) case N_: cmb::sinkhorn_bwd_kernel<N_><<<grid, 128, 0, st>>>(raw, gout, graw, count, iters, eps); break;
    CMB_SK_CASE(2) CMB_SK_CASE(3) CMB_SK_CASE(4) CMB_SK_CASE(5) CMB_SK_CASE(6) CMB_SK_CASE(7) CMB_SK_CASE(8)
#undef CMB_SK_CASE
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
