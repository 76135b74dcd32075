// y[M,N] = x[M,K]·W[N,K]ᵀ (+bias) for 2 ≤ M ≤ 32 activation rows: the decode-step linear for small batches (sm_100a).
//
// The work is a weight stream (every weight byte is used once), so the kernel is organised around keeping 16-byte weight
// loads in flight on every SM rather than around a large MMA tile: a warp owns 8·NT output columns, and KS warps of a
// CTA share one column group and split its contraction into contiguous ranges (folded through shared memory at the
// end); KS is chosen at launch so that even the narrow projections put about a dozen warps on every SM.  Each lane
// loads 8 consecutive bf16 of one weight row and of two activation rows per chunk; those 8 values feed two
// `mma.sync.m16n8k16` instructions — the contraction index inside a chunk is permuted (the same way for both operands, which
// leaves the sum unchanged) so that one 16-byte load is exactly one lane's fragment pair.  Accumulation is fp32.
// A tcgen05 tile (M = 128, or 64 columns of a swapped product) would leave most of the tensor work idle and, more
// importantly, yields far too few CTAs to pull HBM bandwidth at these sizes; the warp-level MMA is only the adder here.
//
// Reference: the decode GEMV role of `mx.quantized_matmul` / plain `nn.Linear` on one-token steps
// (cppmega_mlx/inference/generation.py:142-227); no counterpart kernel exists there.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace cmb {

constexpr int SM_WARPS = 8;
constexpr int SM_THREADS = SM_WARPS * 32;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// MT: 16-row activation tiles (1 → M ≤ 16, 2 → M ≤ 32).  NT: 8-column weight tiles per warp.  KS: warps that share one
// column group and split its contraction (a CTA holds 8 / KS column groups).
template <int MT, int NT, int KS>
__global__ void __launch_bounds__(SM_THREADS, 2) skinny_mma_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                                                                const __nv_bfloat16* __restrict__ w, long long ldw,
                                                                __nv_bfloat16* __restrict__ y, long long ldy,
                                                                const __nv_bfloat16* __restrict__ bias, int M, int N, int K) {
  constexpr int GROUPS = SM_WARPS / KS;
  __shared__ float red[KS > 1 ? SM_WARPS : 1][MT][NT][32][4];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int kslice = warp % KS, group = warp / KS;
  const int n0 = (blockIdx.x * GROUPS + group) * 8 * NT;
  float acc[MT][NT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[mt][nt][i] = 0.f;
  // per-lane row pointers; rows / columns past the edge are clamped for the address and zeroed by the predicate
  const __nv_bfloat16* wrow[NT];
  bool wok[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int n = n0 + nt * 8 + g;
    wok[nt] = n < N;
    wrow[nt] = w + static_cast<long long>(wok[nt] ? n : 0) * ldw + t * 8;
  }
  const __nv_bfloat16* xrow[MT][2];
  bool xok[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int m = mt * 16 + hf * 8 + g;
      xok[mt][hf] = m < M;
      xrow[mt][hf] = x + static_cast<long long>(xok[mt][hf] ? m : 0) * ldx + t * 8;
    }
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  // contiguous contraction range per slice, so that a lane's consecutive 16-byte loads walk along one weight row
  const int chunks = (K + 31) / 32, per = (chunks + KS - 1) / KS;
  const int k_begin = kslice * per * 32, k_end = min(K, k_begin + per * 32);
#pragma unroll(MT == 2 ? 2 : 4)
  for (int k0 = k_begin; k0 < k_end; k0 += 32) {
    const bool kok = k0 + t * 8 < K;      // K is a multiple of 8, so a lane's 8 values are all inside or all outside
    uint4 wb[NT], xa[MT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) wb[nt] = (kok && wok[nt]) ? ldg_stream(wrow[nt] + k0) : zero;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) xa[mt][hf] = (kok && xok[mt][hf]) ? *reinterpret_cast<const uint4*>(xrow[mt][hf] + k0) : zero;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        mma_bf16_16816(acc[mt][nt], xa[mt][0].x, xa[mt][1].x, xa[mt][0].y, xa[mt][1].y, wb[nt].x, wb[nt].y);
        mma_bf16_16816(acc[mt][nt], xa[mt][0].z, xa[mt][1].z, xa[mt][0].w, xa[mt][1].w, wb[nt].z, wb[nt].w);
      }
  }
  if (KS > 1) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) red[warp][mt][nt][lane][i] = acc[mt][nt][i];
    __syncthreads();
    if (kslice != 0) return;
    // the first warp of each column group folds the other contraction slices into its own accumulators
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float s = acc[mt][nt][i];
#pragma unroll
          for (int ks = 1; ks < KS; ++ks) s += red[warp + ks][mt][nt][lane][i];
          acc[mt][nt][i] = s;
        }
  }
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int m = mt * 16 + hf * 8 + g;
        const int n = n0 + nt * 8 + t * 2;
        if (m >= M || n >= N) continue;
        float c0 = acc[mt][nt][2 * hf], c1 = acc[mt][nt][2 * hf + 1];
        __nv_bfloat16* dst = y + static_cast<long long>(m) * ldy + n;
        if (n + 1 < N) {
          if (bias != nullptr) { c0 += __bfloat162float(bias[n]); c1 += __bfloat162float(bias[n + 1]); }
          if ((reinterpret_cast<uintptr_t>(dst) & 3) == 0) {
            *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(c0, c1);
          } else {
            dst[0] = __float2bfloat16(c0);
            dst[1] = __float2bfloat16(c1);
          }
        } else {
          if (bias != nullptr) c0 += __bfloat162float(bias[n]);
          dst[0] = __float2bfloat16(c0);
        }
      }
}

template <int MT, int NT>
static void launch_skinny_mma(int ks, unsigned tiles, cudaStream_t st, const __nv_bfloat16* X, long long ldx, const __nv_bfloat16* W,
                              long long ldw, __nv_bfloat16* Y, long long ldy, const __nv_bfloat16* Bv, int M, int N, int K) {
  const unsigned groups = SM_WARPS / ks;
  const unsigned grid = (tiles + groups - 1) / groups;
  switch (ks) {
    case 1: skinny_mma_kernel<MT, NT, 1><<<grid, SM_THREADS, 0, st>>>(X, ldx, W, ldw, Y, ldy, Bv, M, N, K); break;
    case 2: skinny_mma_kernel<MT, NT, 2><<<grid, SM_THREADS, 0, st>>>(X, ldx, W, ldw, Y, ldy, Bv, M, N, K); break;
    case 4: skinny_mma_kernel<MT, NT, 4><<<grid, SM_THREADS, 0, st>>>(X, ldx, W, ldw, Y, ldy, Bv, M, N, K); break;
    default: skinny_mma_kernel<MT, NT, 8><<<grid, SM_THREADS, 0, st>>>(X, ldx, W, ldw, Y, ldy, Bv, M, N, K); break;
  }
}

}  // namespace cmb

// x [M,K] bf16 (pitch ldx), w [N,K] bf16 (pitch ldw), y [M,N] bf16 (pitch ldy), optional bf16 bias [N].  1 ≤ M ≤ 32,
// K and both pitches multiples of 8, x and w 16-byte aligned; returns 1 otherwise.
extern "C" int cmb_skinny_mma(const void* x, long long ldx, const void* w, long long ldw, void* y, long long ldy, const void* bias,
                              int M, int N, int K, void* stream) {
  if (M < 1 || M > 32 || K <= 0 || K % 8 || ldx % 8 || ldw % 8 || N <= 0) return 1;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) return 1;
  auto st = static_cast<cudaStream_t>(stream);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto W = static_cast<const __nv_bfloat16*>(w);
  auto Y = static_cast<__nv_bfloat16*>(y);
  auto Bv = static_cast<const __nv_bfloat16*>(bias);
  // Columns per warp: more columns amortise the activation loads (which matter most with two row tiles), fewer give narrow
  // matrices enough warps.  Contraction split: the smallest power of two that puts about twelve warps on every SM.
  const int nt = (M > 16 && N >= 8192) ? 4 : (N >= 4096 || M > 16 ? 2 : 1);
  const unsigned tiles = static_cast<unsigned>((N + 8 * nt - 1) / (8 * nt));
  int ks = 1;
  while (ks < 8 && tiles * ks < 148u * 12u && K / (ks * 2) >= 256) ks *= 2;
  if (M <= 16) {
    if (nt == 4) cmb::launch_skinny_mma<1, 4>(ks, tiles, st, X, ldx, W, ldw, Y, ldy, Bv, M, N, K);
    else if (nt == 2) cmb::launch_skinny_mma<1, 2>(ks, tiles, st, X, ldx, W, ldw, Y, ldy, Bv, M, N, K);
    else cmb::launch_skinny_mma<1, 1>(ks, tiles, st, X, ldx, W, ldw, Y, ldy, Bv, M, N, K);
  } else {
    if (nt == 4) cmb::launch_skinny_mma<2, 4>(ks, tiles, st, X, ldx, W, ldw, Y, ldy, Bv, M, N, K);
    else cmb::launch_skinny_mma<2, 2>(ks, tiles, st, X, ldx, W, ldw, Y, ldy, Bv, M, N, K);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
