// Cut cross-entropy row kernel: turns a chunk of bf16 logits [rows, V] into per-row losses and, in
// place, into the gradient of the mean loss with respect to those logits.
//
//   lse_r   = log Σ_j exp(l_rj)                (online max/sum in fp32, one pass)
//   loss_r  = valid_r · (lse_r − l_r,t_r)
//   l_rj   ← scale · valid_r · (exp(l_rj − lse_r) − [j = t_r])        (second pass, L2-resident row)
//
// One CTA per row, 16-byte accesses. Used between the logits GEMM and the two gradient GEMMs of
// ops/cce.py so the full [tokens, vocab] matrix is never held. Math parity with the reference's manual
// forward+backward: cppmega_mlx/training/cut_cross_entropy.py:147-201.
#include "sm100.cuh"

namespace cmb {

template <int THREADS>
__global__ void __launch_bounds__(THREADS) cce_rows_kernel(__nv_bfloat16* __restrict__ logits,
                                                            const int* __restrict__ targets,
                                                            const uint8_t* __restrict__ valid,
                                                            float* __restrict__ loss_rows, int64_t rows, int V,
                                                            const float* __restrict__ scale_ptr, int write_grad, int* status) {
  __shared__ float red_m[THREADS / 32];
  __shared__ float red_s[THREADS / 32];
  __shared__ float bcast[2];
  const int nvec = V >> 3;
  const float scale = scale_ptr != nullptr ? *scale_ptr : 1.f;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    __nv_bfloat16* lr = logits + row * V;
    float m = -INFINITY, s = 0.f;
    for (int v = threadIdx.x; v < nvec; v += THREADS) {
      const uint4 q = *reinterpret_cast<const uint4*>(lr + 8 * v);
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&q);
      float f[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 t = __bfloat1622float2(b[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
      }
      float lm = f[0];
#pragma unroll
      for (int i = 1; i < 8; ++i) lm = fmaxf(lm, f[i]);
      const float nm = fmaxf(m, lm);
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc += __expf(f[i] - nm);
      s = s * __expf(m - nm) + acc;
      m = nm;
    }
    // warp then block combine of (m, s)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o);
      const float os = __shfl_xor_sync(0xffffffffu, s, o);
      const float nm = fmaxf(m, om);
      s = (nm == -INFINITY) ? 0.f : s * __expf(m - nm) + os * __expf(om - nm);
      m = nm;
    }
    if ((threadIdx.x & 31) == 0) {
      red_m[threadIdx.x >> 5] = m;
      red_s[threadIdx.x >> 5] = s;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float M = red_m[0], S = red_s[0];
      for (int w = 1; w < THREADS / 32; ++w) {
        const float nm = fmaxf(M, red_m[w]);
        S = (nm == -INFINITY) ? 0.f : S * __expf(M - nm) + red_s[w] * __expf(red_m[w] - nm);
        M = nm;
      }
      const float lse = M + __logf(S);
      int t = targets[row];
      bool in_range = t >= 0 && t < V;
      if (!in_range && valid[row]) {
        // a target outside the vocabulary: the row contributes nothing, nothing is read at that index, and the first such row
        // is reported through the status block (code, row, target, vocabulary size)
        if (status != nullptr && atomicCAS(status, 0, ST_BAD_ARGUMENT) == 0) {
          status[1] = static_cast<int>(row);
          status[2] = t;
          status[3] = V;
        }
      }
      if (!in_range) t = 0;
      const float tl = __bfloat162float(lr[t]);
      const float ok = (valid[row] && in_range) ? 1.f : 0.f;
      loss_rows[row] = ok * (lse - tl);
      bcast[0] = lse;
      bcast[1] = ok * scale;
    }
    __syncthreads();
    if (write_grad) {
      const float lse = bcast[0], g = bcast[1];
      const int t = targets[row];
      for (int v = threadIdx.x; v < nvec; v += THREADS) {
        uint4 q = *reinterpret_cast<const uint4*>(lr + 8 * v);
        __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float2 x = __bfloat1622float2(b[i]);
          const int j = 8 * v + 2 * i;
          x.x = g * (__expf(x.x - lse) - (j == t ? 1.f : 0.f));
          x.y = g * (__expf(x.y - lse) - (j + 1 == t ? 1.f : 0.f));
          b[i] = __floats2bfloat162_rn(x.x, x.y);
        }
        *reinterpret_cast<uint4*>(lr + 8 * v) = q;
      }
    }
    __syncthreads();
  }
}

}  // namespace cmb

// scale_ptr: device scalar (1 / number of valid targets), so the caller never syncs to learn the count.
// logits: bf16 [rows, V] (V % 8 == 0, rows contiguous), overwritten with dlogits when write_grad != 0.
extern "C" int cmb_cce_rows(void* logits, const int* targets, const uint8_t* valid, float* loss_rows, int64_t rows,
                            int V, const float* scale_ptr, int write_grad, int* status, void* stream) {
  if (V % 8) return 1;
  if (rows <= 0) return 0;
  const int grid = static_cast<int>(rows < 148 * 8 ? rows : 148 * 8);
  cmb::cce_rows_kernel<512><<<grid, 512, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(logits), targets, valid, loss_rows, rows, V, scale_ptr, write_grad, status);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
