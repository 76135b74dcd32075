// DSA indexer KL loss, row stage (sm_100a): teacher softmax over heads, student softmax, KL and its gradient in one launch.
//
// The attention logits of a block of query rows come from the tcgen05 GEMM as fp32 [rows·H, Sk] (row = q·H + h, unscaled).
// One CTA per query row then makes two passes over that row's H logit rows and its index-score row:
//   pass 1  one warp per head (the index scores count as head H): online max / sum of exp over the live keys;
//   pass 2  one thread per key: p_k = mean_h exp(l_hk − m_h)/s_h, q_k = exp(x_k − m_x)/s_x,
//           KL += p_k (log p_k − log q_k), and d(KL)/dx_k = q_k − p_k is written straight into the gradient row.
// Live keys: k ≤ absolute query position, and (when a bit row is given) bit k of the row's top-k membership mask.
// A row without live keys reports valid = 0, KL = 0 and a zero gradient row.
//
// Reference: cppmega_mlx/nn/_tilelang/dsa_splitk_indexer_loss.py:327-690 (stage 1: per-head online-softmax statistics)
// and :781-1170 (stage 2: recompute, head mean, KL reduction); this kernel is both stages for one query row, and also
// produces the gradient that the reference leaves to autodiff of its wrapper (:1327-1570).
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

namespace cmb {

constexpr int DL_THREADS = 256;
constexpr int DL_MAX_HEADS = 128;

struct DsaLossParams {
  const float* logits;     // [rows·H, ldl]
  const float* x;          // [rows, ldx] index scores
  float* grad;             // [rows, ldx]
  const uint32_t* bits;    // [rows, ldbits] or null
  float* kl;               // [rows]
  float* valid;            // [rows]
  long long ldl, ldx, ldbits;
  int rows, H, Sk, q0;     // q0 = absolute position of local row 0
  float scale;
};

__device__ __forceinline__ void online_merge(float& m, float& s, float m2, float s2) {
  const float M = fmaxf(m, m2);
  const float a = (m == -CUDART_INF_F) ? 0.f : s * __expf(m - M);
  const float b = (m2 == -CUDART_INF_F) ? 0.f : s2 * __expf(m2 - M);
  m = M;
  s = a + b;
}

__global__ void __launch_bounds__(DL_THREADS) dsa_kl_rows_kernel(const DsaLossParams p) {
  __shared__ float s_m[DL_MAX_HEADS + 1], s_inv[DL_MAX_HEADS + 1];
  __shared__ float s_red[DL_THREADS / 32];
  const int row = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int H = p.H;
  const long long kmax_ll = static_cast<long long>(p.q0) + row + 1;
  const int kmax = kmax_ll < 0 ? 0 : (kmax_ll < p.Sk ? static_cast<int>(kmax_ll) : p.Sk);
  const uint32_t* brow = p.bits != nullptr ? p.bits + static_cast<long long>(row) * p.ldbits : nullptr;
  const float* xrow = p.x + static_cast<long long>(row) * p.ldx;
  const float* lrow = p.logits + static_cast<long long>(row) * H * p.ldl;

  // pass 1: softmax statistics, one warp per head
  for (int hh = warp; hh <= H; hh += DL_THREADS / 32) {
    const float* src = hh < H ? lrow + static_cast<long long>(hh) * p.ldl : xrow;
    const float sc = hh < H ? p.scale : 1.f;
    float m = -CUDART_INF_F, s = 0.f;
    for (int k0 = 0; k0 < kmax; k0 += 32) {
      const int k = k0 + lane;
      const uint32_t word = brow != nullptr ? brow[k0 >> 5] : 0xffffffffu;
      if (k < kmax && ((word >> lane) & 1u)) {
        const float v = src[k] * sc;
        if (v > m) {
          s = s * __expf(m - v) + 1.f;     // exp(−inf) = 0 covers the first live element
          m = v;
        } else {
          s += __expf(v - m);
        }
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, off);
      const float s2 = __shfl_xor_sync(0xffffffffu, s, off);
      online_merge(m, s, m2, s2);
    }
    if (lane == 0) {
      s_m[hh] = m;
      s_inv[hh] = s > 0.f ? 1.f / s : 0.f;
    }
  }
  __syncthreads();

  const bool row_valid = s_inv[H] > 0.f;
  const float m_x = s_m[H], inv_x = s_inv[H];
  const float log_sx = row_valid ? -__logf(inv_x) : 0.f;
  const float inv_h = 1.f / static_cast<float>(H);
  float* grow = p.grad + static_cast<long long>(row) * p.ldx;
  float kl = 0.f;
  // pass 2: head mean, KL and gradient, one thread per key
  for (int k = tid; k < p.Sk; k += DL_THREADS) {
    float g = 0.f;
    bool live = row_valid && k < kmax;
    if (live && brow != nullptr) live = (brow[k >> 5] >> (k & 31)) & 1u;
    if (live) {
      float pk = 0.f;
      for (int h = 0; h < H; ++h) pk += __expf(lrow[static_cast<long long>(h) * p.ldl + k] * p.scale - s_m[h]) * s_inv[h];
      pk *= inv_h;
      const float xs = xrow[k] - m_x;
      const float qk = __expf(xs) * inv_x;
      if (pk > 0.f) kl += pk * (__logf(pk) - (xs - log_sx));
      g = qk - pk;
    }
    grow[k] = g;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) kl += __shfl_xor_sync(0xffffffffu, kl, off);
  if (lane == 0) s_red[warp] = kl;
  __syncthreads();
  if (tid == 0) {
    float t = 0.f;
    for (int w = 0; w < DL_THREADS / 32; ++w) t += s_red[w];
    p.kl[row] = row_valid ? t : 0.f;
    p.valid[row] = row_valid ? 1.f : 0.f;
  }
}

}  // namespace cmb

// `ip` = {rows, H, Sk, q0}; `lp` = {ldl, ldx, ldbits}.  Returns 1 for a geometry the kernel does not take.
extern "C" int cmb_dsa_kl_rows(const void* logits, const void* x, void* grad, const void* bits, void* kl, void* valid,
                               const int* ip, const long long* lp, float scale, void* stream) {
  cmb::DsaLossParams p{};
  p.logits = static_cast<const float*>(logits);
  p.x = static_cast<const float*>(x);
  p.grad = static_cast<float*>(grad);
  p.bits = static_cast<const uint32_t*>(bits);
  p.kl = static_cast<float*>(kl);
  p.valid = static_cast<float*>(valid);
  p.rows = ip[0]; p.H = ip[1]; p.Sk = ip[2]; p.q0 = ip[3];
  p.ldl = lp[0]; p.ldx = lp[1]; p.ldbits = lp[2];
  p.scale = scale;
  if (p.rows <= 0 || p.H < 1 || p.H > cmb::DL_MAX_HEADS || p.Sk <= 0 || p.ldl < p.Sk || p.ldx < p.Sk) return 1;
  if (p.bits != nullptr && p.ldbits * 32 < p.Sk) return 1;
  cmb::dsa_kl_rows_kernel<<<static_cast<unsigned>(p.rows), cmb::DL_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
