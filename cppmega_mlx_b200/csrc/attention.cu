// Small kernels around the attention GEMMs (ops/attention.py): key bitmask from a top-k index list,
// log-sum-exp combine of per-tile softmax statistics, and the backward's row term δ = Σ_d dO·O.
// The index/mask semantics follow the sparse-MLA oracle (cppmega_mlx/nn/sparse_mla.py:125-210:
// `-1` marks an unused slot, a query with no valid slot produces zeros).
#include "sm100.cuh"

namespace cmb {

// mask[b, t, w] bit j set ⇔ key 32w+j is listed for query t (and 32w+j ≤ t + q_off). One warp per (b,t) row.
__global__ void attn_build_mask_kernel(const int* __restrict__ idx, unsigned* __restrict__ mask, long long rows, int S,
                                       int Skv, int topk, int W, int q_off) {
  extern __shared__ unsigned sm[];
  const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = blockIdx.x * static_cast<long long>(blockDim.x >> 5) + wib;
  unsigned* mine = sm + wib * W;
  if (row >= rows) return;
  for (int w = lane; w < W; w += 32) mine[w] = 0u;
  __syncwarp();
  const int t = static_cast<int>(row % S);
  const int* ir = idx + row * topk;
  for (int k = lane; k < topk; k += 32) {
    const int key = ir[k];
    if (key >= 0 && key < Skv && key <= t + q_off) atomicOr(&mine[key >> 5], 1u << (key & 31));
  }
  __syncwarp();
  unsigned* out = mask + row * W;
  for (int w = lane; w < W; w += 32) out[w] = mine[w];
}

// lse[row] = log Σ over the tile halves at or below the diagonal. stats: float2 per (row, 2·num_n halves).
__global__ void attn_lse_combine_kernel(const float2* __restrict__ stats, float* __restrict__ lse, long long rows, int S,
                                        int halves, int half_cols) {
  const long long row = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (row >= rows) return;
  const int t = static_cast<int>(row % S);
  const int last = min(halves - 1, t / half_cols);
  // a half is written only when its tile was computed: tiles with n0 < m0 + 128, i.e. up to the tile holding column
  // (t | 127); the per-row causal limit already zeroed later halves, so stopping at t's own half is exact.
  float m = -INFINITY, l = 0.f;
  const float2* sr = stats + row * halves;
  for (int i = 0; i <= last; ++i) {
    const float2 v = sr[i];
    if (v.y > 0.f) {
      const float nm = fmaxf(m, v.x);
      l = l * __expf(m - nm) + v.y * __expf(v.x - nm);
      m = nm;
    }
  }
  lse[row] = l > 0.f ? m + __logf(l) : INFINITY;  // +inf ⇒ exp(s − lse) = 0 for rows that see no key
}

// delta[b,h,t] = Σ_d dO[b,t,h,d]·O[b,t,h,d]; one warp per (b,t,h). Output laid out [B,H,S].
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ dO, const __nv_bfloat16* __restrict__ O,
                                  float* __restrict__ delta, int Bn, int S, int H, int Dv) {
  const long long wid = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= static_cast<long long>(Bn) * S * H) return;
  const int h = static_cast<int>(wid % H);
  const long long bt = wid / H;
  const int t = static_cast<int>(bt % S);
  const int b = static_cast<int>(bt / S);
  const long long base = wid * Dv;
  float acc = 0.f;
  for (int d = 2 * lane; d < Dv; d += 64) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dO + base + d));
    const float2 o = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(O + base + d));
    acc += a.x * o.x + a.y * o.y;
  }
  acc = warp_sum(acc);
  if (lane == 0) delta[(static_cast<long long>(b) * H + h) * S + t] = acc;
}

}  // namespace cmb

extern "C" int cmb_attn_build_mask(const int* idx, unsigned* mask, long long rows, int S, int Skv, int topk, int q_off,
                                   void* stream) {
  const int W = (Skv + 31) / 32;
  if (W > 1024) return 1;
  const int wpb = 4;
  cmb::attn_build_mask_kernel<<<static_cast<unsigned>((rows + wpb - 1) / wpb), wpb * 32, wpb * W * sizeof(unsigned),
                                static_cast<cudaStream_t>(stream)>>>(idx, mask, rows, S, Skv, topk, W, q_off);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
extern "C" int cmb_attn_lse_combine(const float* stats, float* lse, long long rows, int S, int halves, int half_cols,
                                    void* stream) {
  cmb::attn_lse_combine_kernel<<<static_cast<unsigned>((rows + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const float2*>(stats), lse, rows, S, halves, half_cols);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
extern "C" int cmb_attn_delta(const void* dO, const void* O, float* delta, int Bn, int S, int H, int Dv, void* stream) {
  if (Dv % 2) return 1;
  const long long warps = static_cast<long long>(Bn) * S * H;
  cmb::attn_delta_kernel<<<static_cast<unsigned>((warps * 32 + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(dO), static_cast<const __nv_bfloat16*>(O), delta, Bn, S, H, Dv);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
