// y[M,N] = x[M,K] · W[N,K]ᵀ for a handful of rows (M ≤ 8): the decode-step shape, where the weight matrix is read once and
// nothing else matters.  A 128-row tensor-core tile would leave N/256 CTAs streaming the whole matrix; here every warp owns
// a few output columns, streams their weight rows with 16-byte loads spread over all SMs and keeps the M partial sums in
// registers.  The role of the reference's decode GEMV (cppmega_mlx/nn/_tilelang/fp8_vecmat_path_c.py, dot4 macro :559),
// for bf16 weights.  x is staged in shared memory once per CTA (M·K·2 bytes ≤ 8·16384·2 = 256 KB would not fit, so K is
// walked in slabs of SLAB columns).
#include "sm100.cuh"

namespace cmb {

constexpr int SK_THREADS = 256;
constexpr int SK_UNROLL = 4;     // 16-byte weight loads in flight per lane and column
constexpr int SK_SLAB = 2048;    // K columns of x staged at a time (M ≤ 8 → ≤ 32 KB)

template <int M, int SK_COLS>
__global__ void __launch_bounds__(SK_THREADS) skinny_gemm_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                                                                 const __nv_bfloat16* __restrict__ w, long long ldw,
                                                                 __nv_bfloat16* __restrict__ y, long long ldy,
                                                                 const __nv_bfloat16* __restrict__ bias, int N, int K) {
  __shared__ __align__(16) __nv_bfloat16 xs[M * SK_SLAB];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps = SK_THREADS / 32;
  const int n0 = (blockIdx.x * warps + warp) * SK_COLS;
  float acc[SK_COLS][M];
#pragma unroll
  for (int c = 0; c < SK_COLS; ++c)
#pragma unroll
    for (int m = 0; m < M; ++m) acc[c][m] = 0.f;

  // The first weight vectors do not depend on x: they are requested before x is staged, so the stream from HBM starts with
  // the kernel instead of after the first barrier.
  uint4 wv[SK_UNROLL][SK_COLS];
  auto load_w = [&](int k0, int kw, int k) {
#pragma unroll
    for (int u = 0; u < SK_UNROLL; ++u)
#pragma unroll
      for (int c = 0; c < SK_COLS; ++c)
        wv[u][c] = (n0 + c < N && k + u * 256 < kw) ? __ldcs(reinterpret_cast<const uint4*>(w + (n0 + c) * ldw + k0 + k + u * 256))
                                                    : make_uint4(0, 0, 0, 0);
  };
  load_w(0, min(SK_SLAB, K), lane * 8);
  for (int k0 = 0; k0 < K; k0 += SK_SLAB) {
    const int kw = min(SK_SLAB, K - k0);            // multiple of 8
    __syncthreads();
    for (int i = threadIdx.x; i < M * (kw / 8); i += SK_THREADS) {
      const int m = i / (kw / 8), c8 = i % (kw / 8);
      *reinterpret_cast<uint4*>(xs + m * SK_SLAB + c8 * 8) = *reinterpret_cast<const uint4*>(x + m * ldx + k0 + c8 * 8);
    }
    __syncthreads();
    for (int k = lane * 8; k < kw; k += 256 * SK_UNROLL) {
      if (k0 > 0 || k > lane * 8) load_w(k0, kw, k);   // the very first batch is already in flight
#pragma unroll
      for (int u = 0; u < SK_UNROLL; ++u) {
        if (k + u * 256 >= kw) break;
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const uint4 xv = *reinterpret_cast<const uint4*>(xs + m * SK_SLAB + k + u * 256);
          const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
          for (int c = 0; c < SK_COLS; ++c) {
            const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv[u][c]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 a = __bfloat1622float2(xp[j]), b = __bfloat1622float2(wp[j]);
              acc[c][m] = fmaf(a.x, b.x, fmaf(a.y, b.y, acc[c][m]));
            }
          }
        }
      }
    }
  }
  if (n0 >= N) return;
#pragma unroll
  for (int c = 0; c < SK_COLS; ++c)
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const float v = warp_sum(acc[c][m]);
      if (lane == 0 && n0 + c < N)
        y[m * ldy + n0 + c] = __float2bfloat16(v + (bias != nullptr ? __bfloat162float(bias[n0 + c]) : 0.f));
    }
}

}  // namespace cmb

// x [M,K] (row pitch ldx), W [N,K] (row pitch ldw), y [M,N] (row pitch ldy), all bf16; bias [N] or null. 1 ≤ M ≤ 8,
// K % 8 == 0, pitches % 8 == 0, 16-byte aligned bases. Returns 1 for an unsupported shape.
extern "C" int cmb_skinny_gemm(const void* x, long long ldx, const void* w, long long ldw, void* y, long long ldy,
                               const void* bias, int M, int N, int K, void* stream) {
  if (M < 1 || M > 8 || K % 8 || ldx % 8 || ldw % 8 || N <= 0) return 1;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) return 1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto W = static_cast<const __nv_bfloat16*>(w);
  auto Y = static_cast<__nv_bfloat16*>(y);
  auto Bv = static_cast<const __nv_bfloat16*>(bias);
  const int warps = cmb::SK_THREADS / 32;
  // two columns per warp halve the x reads from shared memory, but a narrow output needs the CTAs more than that
  const bool two = (N + 2 * warps - 1) / (2 * warps) >= 2 * 148;
  const unsigned grid = static_cast<unsigned>((N + (two ? 2 : 1) * warps - 1) / ((two ? 2 : 1) * warps));
#define CMB_SK_CASE(MM)                                                                                               \
  case MM:                                                                                                            \
    if (two) cmb::skinny_gemm_kernel<MM, 2><<<grid, cmb::SK_THREADS, 0, st>>>(X, ldx, W, ldw, Y, ldy, Bv, N, K);        \
    else cmb::skinny_gemm_kernel<MM, 1><<<grid, cmb::SK_THREADS, 0, st>>>(X, ldx, W, ldw, Y, ldy, Bv, N, K);            \
    break;
  switch (M) {
    CMB_SK_CASE(1) CMB_SK_CASE(2) CMB_SK_CASE(3) CMB_SK_CASE(4) CMB_SK_CASE(5) CMB_SK_CASE(6) CMB_SK_CASE(7)
    default:
      if (two) cmb::skinny_gemm_kernel<8, 2><<<grid, cmb::SK_THREADS, 0, st>>>(X, ldx, W, ldw, Y, ldy, Bv, N, K);
      else cmb::skinny_gemm_kernel<8, 1><<<grid, cmb::SK_THREADS, 0, st>>>(X, ldx, W, ldw, Y, ldy, Bv, N, K);
      break;
  }
#undef CMB_SK_CASE
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
