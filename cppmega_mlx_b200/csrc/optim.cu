// Fused optimizer kernels: AdamW (fp32 moments), 8-bit AdamW / Lion (uint8 codes + per-256 absmax,
// symmetric int8 or 256-entry dynamic code book), Muon momentum stage.
//
// 8-bit layout: one warp owns one 256-value quantisation block (8 values per lane, one 64-bit
// code load per lane); the new absmax is a shuffle reduction; the step uses the fresh fp32 moments
// and the per-block noise floor max(prev_absmax, new_absmax)/127 before re-quantising.
// Math parity: cppmega_mlx/training/native_optim/fused_8bit.metal:8-110 (Adam symmetric),
// :112-249 (Adam dynamic, binary-search requant), :251-305 / :307-382 (Lion).
#include "optim.h"
#include <type_traits>

#include "sm100.cuh"

namespace cmb {

template <typename T>
struct Cvt;
template <>
struct Cvt<float> {
  static __device__ __forceinline__ float ld(const float* p, int64_t i) { return p[i]; }
  static __device__ __forceinline__ void st(float* p, int64_t i, float v) { p[i] = v; }
};
template <>
struct Cvt<__half> {
  static __device__ __forceinline__ float ld(const __half* p, int64_t i) { return __half2float(p[i]); }
  static __device__ __forceinline__ void st(__half* p, int64_t i, float v) { p[i] = __float2half_rn(v); }
};
template <>
struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ float ld(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, int64_t i, float v) { p[i] = __float2bfloat16(v); }
};

template <typename T>
__global__ void adamw_kernel(T* __restrict__ p, const T* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                             int64_t n, float lr, float b1, float b2, float eps, float wd, float c1, float c2,
                             float gscale) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const float gi = Cvt<T>::ld(g, i) * gscale;
    const float mi = b1 * m[i] + (1.f - b1) * gi;
    const float vi = b2 * v[i] + (1.f - b2) * gi * gi;
    m[i] = mi;
    v[i] = vi;
    const float pi = Cvt<T>::ld(p, i) * (1.f - lr * wd) - lr * c1 * mi / (sqrtf(vi) * c2 + eps);
    Cvt<T>::st(p, i, pi);
  }
}

__device__ __forceinline__ float deq_sym(uint8_t q, float absmax) {
  return static_cast<float>(static_cast<int>(q) - 128) * (1.f / 127.f) * absmax;
}
__device__ __forceinline__ uint8_t q_sym(float v, float absmax) {
  const float d = absmax > 0.f ? absmax : 1.f;
  float r = rintf(v / d * 127.f);
  r = fminf(fmaxf(r, -127.f), 127.f);
  return static_cast<uint8_t>(static_cast<int>(r) + 128);
}
__device__ __forceinline__ uint8_t q_dyn(float v, float absmax, const float* lut) {
  const float d = absmax > 0.f ? absmax : 1.f;
  const float x = fminf(fmaxf(v / d, -1.f), 1.f);
  int lo = 0, hi = 255;
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int mid = (lo + hi) >> 1;
    const bool right = lut[mid] < x;
    lo = right ? mid + 1 : lo;
    hi = right ? hi : mid;
  }
  const int prev = lo > 0 ? lo - 1 : 0;
  const bool use_prev = lo > 0 && fabsf(lut[prev] - x) < fabsf(lut[lo] - x);
  return static_cast<uint8_t>(use_prev ? prev : lo);
}

// One warp per 256-block. `lut` != nullptr selects the dynamic code book (staged in shared memory).
template <typename T, bool DYN>
__global__ void __launch_bounds__(256) adam8bit_kernel(T* __restrict__ p, const T* __restrict__ g,
                                                        uint8_t* __restrict__ mq, float* __restrict__ ma,
                                                        uint8_t* __restrict__ vq, float* __restrict__ va,
                                                        const float* __restrict__ lut, int64_t n, float lr, float b1,
                                                        float b2, float eps, float wd, float c1, float c2) {
  __shared__ float slut[256];
  if (DYN) {
    slut[threadIdx.x] = lut[threadIdx.x];
    __syncthreads();
  }
  const int lane = threadIdx.x & 31;
  const int64_t nblk = (n + 255) / 256;
  const int64_t warp0 = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t blk = warp0; blk < nblk; blk += nwarps) {
    const int64_t base = blk * 256 + lane * 8;
    const float am_prev = ma[blk], av_prev = va[blk];
    float mv[8], vv[8], gv[8];
    float am_new = 0.f, av_new = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int64_t i = base + e;
      if (i < n) {
        const uint8_t qm = mq[i], qv = vq[i];
        const float m0 = DYN ? slut[qm] * am_prev : deq_sym(qm, am_prev);
        const float v0 = fmaxf(DYN ? slut[qv] * av_prev : deq_sym(qv, av_prev), 0.f);
        gv[e] = Cvt<T>::ld(g, i);
        mv[e] = b1 * m0 + (1.f - b1) * gv[e];
        vv[e] = fmaxf(b2 * v0 + (1.f - b2) * gv[e] * gv[e], 0.f);
        am_new = fmaxf(am_new, fabsf(mv[e]));
        av_new = fmaxf(av_new, vv[e]);
      } else {
        mv[e] = vv[e] = gv[e] = 0.f;
      }
    }
    am_new = warp_max(am_new);
    av_new = warp_max(av_new);
    const float floor_v = fmaxf(av_prev, av_new) * (1.f / 127.f);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int64_t i = base + e;
      if (i < n) {
        const float pi = Cvt<T>::ld(p, i) * (1.f - lr * wd) - lr * c1 * mv[e] / (sqrtf(vv[e]) * c2 + floor_v + eps);
        Cvt<T>::st(p, i, pi);
        mq[i] = DYN ? q_dyn(mv[e], am_new, slut) : q_sym(mv[e], am_new);
        vq[i] = DYN ? q_dyn(vv[e], av_new, slut) : q_sym(vv[e], av_new);
      }
    }
    if (lane == 0) {
      ma[blk] = am_new;
      va[blk] = av_new;
    }
  }
}

template <typename T, bool DYN>
__global__ void __launch_bounds__(256) lion8bit_kernel(T* __restrict__ p, const T* __restrict__ g,
                                                        uint8_t* __restrict__ mq, float* __restrict__ ma,
                                                        const float* __restrict__ lut, int64_t n, float lr, float b1,
                                                        float b2, float wd) {
  __shared__ float slut[256];
  if (DYN) {
    slut[threadIdx.x] = lut[threadIdx.x];
    __syncthreads();
  }
  const int lane = threadIdx.x & 31;
  const int64_t nblk = (n + 255) / 256;
  const int64_t warp0 = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t blk = warp0; blk < nblk; blk += nwarps) {
    const int64_t base = blk * 256 + lane * 8;
    const float am_prev = ma[blk];
    float mv[8];
    float am_new = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int64_t i = base + e;
      mv[e] = 0.f;
      if (i < n) {
        const uint8_t q = mq[i];
        const float m0 = DYN ? slut[q] * am_prev : deq_sym(q, am_prev);
        const float gi = Cvt<T>::ld(g, i);
        const float c = b1 * m0 + (1.f - b1) * gi;
        const float sgn = c > 0.f ? 1.f : (c < 0.f ? -1.f : 0.f);
        Cvt<T>::st(p, i, Cvt<T>::ld(p, i) * (1.f - lr * wd) - lr * sgn);
        mv[e] = b2 * m0 + (1.f - b2) * gi;
        am_new = fmaxf(am_new, fabsf(mv[e]));
      }
    }
    am_new = warp_max(am_new);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int64_t i = base + e;
      if (i < n) mq[i] = DYN ? q_dyn(mv[e], am_new, slut) : q_sym(mv[e], am_new);
    }
    if (lane == 0) ma[blk] = am_new;
  }
}

// Muon stage 1: momentum with weight decay folded into the gradient, Nesterov blend written as the bf16
// Newton–Schulz input, and Σ update² (for the Frobenius normalisation) accumulated with one atomic per CTA.
template <typename T>
__global__ void __launch_bounds__(256) muon_momentum_kernel(const T* __restrict__ g, const T* __restrict__ p,
                                                             float* __restrict__ v, __nv_bfloat16* __restrict__ out,
                                                             float* __restrict__ sumsq, int64_t n, float mu, float wd,
                                                             int nesterov) {
  __shared__ float red[8];
  float acc = 0.f;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const float gi = Cvt<T>::ld(g, i) + wd * Cvt<T>::ld(p, i);
    const float vi = mu * v[i] + (1.f - mu) * gi;
    v[i] = vi;
    const float u = nesterov ? gi * (1.f - mu) + vi * mu : vi;
    acc += u * u;
    out[i] = __float2bfloat16(u);
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 8) {
    float t = red[threadIdx.x];
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffu, t, o);
    if (threadIdx.x == 0 && sumsq != nullptr) atomicAdd(sumsq, t);
  }
}

// x ← x / (sqrt(*sumsq) + eps)   (bf16, in place): the Frobenius normalisation in front of Newton–Schulz.
__global__ void scale_inv_norm_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ sumsq, int64_t n, float eps) {
  const float inv = 1.f / (sqrtf(*sumsq) + eps);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    x[i] = __float2bfloat16(__bfloat162float(x[i]) * inv);
}

// p ← p − coef · u   (u bf16, the orthogonalised update).
template <typename T>
__global__ void axpy_update_kernel(T* __restrict__ p, const __nv_bfloat16* __restrict__ u, int64_t n, float coef) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    Cvt<T>::st(p, i, Cvt<T>::ld(p, i) - coef * __bfloat162float(u[i]));
}

static inline int grid_for(int64_t n, int per_block) {
  int64_t b = (n + per_block - 1) / per_block;
  const int64_t cap = 148 * 16;
  return static_cast<int>(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace cmb

#define CMB_DISPATCH_DTYPE(dtype, CALL)     \
  switch (dtype) {                          \
    case 0: { using T = float; CALL; break; }          \
    case 1: { using T = __half; CALL; break; }         \
    case 2: { using T = __nv_bfloat16; CALL; break; }  \
    default: return 1;                      \
  }

extern "C" int cmb_adamw(void* p, const void* g, float* m, float* v, int64_t n, int dtype, float lr, float b1, float b2,
                         float eps, float wd, float c1, float c2, float grad_scale, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  CMB_DISPATCH_DTYPE(dtype, (cmb::adamw_kernel<T><<<cmb::grid_for(n, 1024), 256, 0, s>>>(
                                static_cast<T*>(p), static_cast<const T*>(g), m, v, n, lr, b1, b2, eps, wd, c1, c2, grad_scale)));
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

extern "C" int cmb_adam8bit(void* p, const void* g, uint8_t* mq, float* ma, uint8_t* vq, float* va, const float* lut,
                            int64_t n, int dtype, float lr, float b1, float b2, float eps, float wd, float c1, float c2,
                            void* stream) {
  if (n <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = cmb::grid_for((n + 255) / 256, 8);
  if (lut != nullptr) {
    CMB_DISPATCH_DTYPE(dtype, (cmb::adam8bit_kernel<T, true><<<grid, 256, 0, s>>>(
                                  static_cast<T*>(p), static_cast<const T*>(g), mq, ma, vq, va, lut, n, lr, b1, b2, eps, wd, c1, c2)));
  } else {
    CMB_DISPATCH_DTYPE(dtype, (cmb::adam8bit_kernel<T, false><<<grid, 256, 0, s>>>(
                                  static_cast<T*>(p), static_cast<const T*>(g), mq, ma, vq, va, lut, n, lr, b1, b2, eps, wd, c1, c2)));
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

extern "C" int cmb_lion8bit(void* p, const void* g, uint8_t* mq, float* ma, const float* lut, int64_t n, int dtype,
                            float lr, float b1, float b2, float wd, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = cmb::grid_for((n + 255) / 256, 8);
  if (lut != nullptr) {
    CMB_DISPATCH_DTYPE(dtype, (cmb::lion8bit_kernel<T, true><<<grid, 256, 0, s>>>(static_cast<T*>(p), static_cast<const T*>(g),
                                                                                  mq, ma, lut, n, lr, b1, b2, wd)));
  } else {
    CMB_DISPATCH_DTYPE(dtype, (cmb::lion8bit_kernel<T, false><<<grid, 256, 0, s>>>(static_cast<T*>(p), static_cast<const T*>(g),
                                                                                   mq, ma, lut, n, lr, b1, b2, wd)));
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

extern "C" int cmb_muon_momentum(const void* g, const void* p, float* v, void* out_bf16, float* sumsq, int64_t n,
                                 int dtype, float momentum, float wd, int nesterov, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  CMB_DISPATCH_DTYPE(dtype, (cmb::muon_momentum_kernel<T><<<cmb::grid_for(n, 2048), 256, 0, s>>>(
                                static_cast<const T*>(g), static_cast<const T*>(p), v, static_cast<__nv_bfloat16*>(out_bf16), sumsq,
                                n, momentum, wd, nesterov)));
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

extern "C" int cmb_scale_inv_norm(void* x, const float* sumsq, int64_t n, float eps, void* stream) {
  if (n <= 0) return 0;
  cmb::scale_inv_norm_kernel<<<cmb::grid_for(n, 2048), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(x), sumsq, n, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

extern "C" int cmb_axpy_update(void* p, const void* u, int64_t n, int dtype, float coef, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  CMB_DISPATCH_DTYPE(dtype, (cmb::axpy_update_kernel<T><<<cmb::grid_for(n, 2048), 256, 0, s>>>(
                                static_cast<T*>(p), static_cast<const __nv_bfloat16*>(u), n, coef)));
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// ---------------------------------------------------------------------------------------------- multi-tensor forms
// One launch over a table of tensors (device memory).  A block owns one 4096-element chunk of one tensor; `chunk_start[t]` is the
// first chunk of tensor t (prefix sums, n + 1 entries), found by binary search.  Every entry carries its own pointers, so the
// tensors may live anywhere (views of flat ZeRO-1 buffers, group workspaces of the batched Newton–Schulz, autograd's gradients).
namespace cmb {

constexpr int MT_CHUNK_ELEMS = 4096;

struct TensorEntry {
  void* p;            // parameter (dtype `dt`)
  const void* g;      // gradient (same dtype) or null
  float* s0;          // fp32 state 0 (Adam m / Muon momentum)
  float* s1;          // fp32 state 1 (Adam v) or null
  __nv_bfloat16* u;   // Muon: bf16 update in / out of Newton–Schulz
  float* sumsq;       // Muon: Σ u² slot of this tensor
  long long numel;
  float coef;         // Muon: learning-rate factor of this tensor
  int pad;
};

__device__ __forceinline__ int mt_find(const int* __restrict__ chunk_start, int n, int chunk) {
  int lo = 0, hi = n - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (chunk_start[mid] <= chunk) lo = mid;
    else hi = mid - 1;
  }
  return lo;
}

// 16-byte forms of the table kernels for bf16 tensors whose pointers are 16-byte aligned and whose length is a multiple of 8:
// a thread moves 8 elements per access instead of one (the scalar loops issue 2-byte loads and are bound by the number of memory
// instructions, 2-3× below the copy rate).
__device__ __forceinline__ bool mt_wide(const TensorEntry& e, bool need_g, bool need_u, bool need_s1) {
  auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  return (e.numel & 7) == 0 && al(e.p) && (!need_g || al(e.g)) && (!need_u || al(e.u)) && al(e.s0) && (!need_s1 || al(e.s1));
}
__device__ __forceinline__ void mt_ld8(const float* p, float (&x)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}
__device__ __forceinline__ void mt_st8(float* p, const float (&x)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(x[4], x[5], x[6], x[7]);
}
__device__ __forceinline__ uint4 mt_pack8(const float (&f)[8]) {
  uint4 v;
  v.x = pack_bf16x2(f[0], f[1]); v.y = pack_bf16x2(f[2], f[3]); v.z = pack_bf16x2(f[4], f[5]); v.w = pack_bf16x2(f[6], f[7]);
  return v;
}

template <typename T>
__global__ void __launch_bounds__(256) muon_momentum_multi_kernel(const TensorEntry* __restrict__ tab, const int* __restrict__ chunk_start, int n,
                                                                   float mu, float wd, int nesterov) {
  __shared__ float red[8];
  const int t = mt_find(chunk_start, n, blockIdx.x);
  const TensorEntry e = tab[t];
  const long long i0 = static_cast<long long>(blockIdx.x - chunk_start[t]) * MT_CHUNK_ELEMS;
  const long long i1 = min(e.numel, i0 + MT_CHUNK_ELEMS);
  const T* g = static_cast<const T*>(e.g);
  const T* p = static_cast<const T*>(e.p);
  float acc = 0.f;
  if (std::is_same<T, __nv_bfloat16>::value && mt_wide(e, true, true, false)) {
    for (long long i = i0 + 8 * threadIdx.x; i < i1; i += 2048) {
      float gg[8], pp[8], vv[8], uu[8];
      unpack8_bf16(*reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(g) + i), gg);
      unpack8_bf16(*reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p) + i), pp);
      mt_ld8(e.s0 + i, vv);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float gi = gg[k] + wd * pp[k];
        vv[k] = mu * vv[k] + (1.f - mu) * gi;
        uu[k] = nesterov ? gi * (1.f - mu) + vv[k] * mu : vv[k];
        acc += uu[k] * uu[k];
      }
      mt_st8(e.s0 + i, vv);
      *reinterpret_cast<uint4*>(e.u + i) = mt_pack8(uu);
    }
  } else
  for (long long i = i0 + threadIdx.x; i < i1; i += 256) {
    const float gi = Cvt<T>::ld(g, i) + wd * Cvt<T>::ld(p, i);
    const float vi = mu * e.s0[i] + (1.f - mu) * gi;
    e.s0[i] = vi;
    const float u = nesterov ? gi * (1.f - mu) + vi * mu : vi;
    acc += u * u;
    e.u[i] = __float2bfloat16(u);
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 8) {
    float r = red[threadIdx.x];
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) r += __shfl_xor_sync(0xffu, r, o);
    if (threadIdx.x == 0) atomicAdd(e.sumsq, r);
  }
}

// u ← u / (sqrt(Σu²) + eps) for every tensor of the table.
__global__ void __launch_bounds__(256) scale_inv_norm_multi_kernel(const TensorEntry* __restrict__ tab, const int* __restrict__ chunk_start, int n,
                                                                    float eps) {
  const int t = mt_find(chunk_start, n, blockIdx.x);
  const TensorEntry e = tab[t];
  const long long i0 = static_cast<long long>(blockIdx.x - chunk_start[t]) * MT_CHUNK_ELEMS;
  const long long i1 = min(e.numel, i0 + MT_CHUNK_ELEMS);
  const float inv = 1.f / (sqrtf(*e.sumsq) + eps);
  if ((e.numel & 7) == 0 && (reinterpret_cast<uintptr_t>(e.u) & 15) == 0) {
    for (long long i = i0 + 8 * threadIdx.x; i < i1; i += 2048) {
      float uu[8];
      unpack8_bf16(*reinterpret_cast<const uint4*>(e.u + i), uu);
#pragma unroll
      for (int k = 0; k < 8; ++k) uu[k] *= inv;
      *reinterpret_cast<uint4*>(e.u + i) = mt_pack8(uu);
    }
    return;
  }
  for (long long i = i0 + threadIdx.x; i < i1; i += 256) e.u[i] = __float2bfloat16(__bfloat162float(e.u[i]) * inv);
}

// p ← p − coef_t · u for every tensor of the table (u = the orthogonalised update).
template <typename T>
__global__ void __launch_bounds__(256) axpy_update_multi_kernel(const TensorEntry* __restrict__ tab, const int* __restrict__ chunk_start, int n) {
  const int t = mt_find(chunk_start, n, blockIdx.x);
  const TensorEntry e = tab[t];
  const long long i0 = static_cast<long long>(blockIdx.x - chunk_start[t]) * MT_CHUNK_ELEMS;
  const long long i1 = min(e.numel, i0 + MT_CHUNK_ELEMS);
  T* p = static_cast<T*>(e.p);
  if (std::is_same<T, __nv_bfloat16>::value && (e.numel & 7) == 0 && ((reinterpret_cast<uintptr_t>(e.p) | reinterpret_cast<uintptr_t>(e.u)) & 15) == 0) {
    __nv_bfloat16* pb = reinterpret_cast<__nv_bfloat16*>(p);
    for (long long i = i0 + 8 * threadIdx.x; i < i1; i += 2048) {
      float pp[8], uu[8];
      unpack8_bf16(*reinterpret_cast<const uint4*>(pb + i), pp);
      unpack8_bf16(*reinterpret_cast<const uint4*>(e.u + i), uu);
#pragma unroll
      for (int k = 0; k < 8; ++k) pp[k] -= e.coef * uu[k];
      *reinterpret_cast<uint4*>(pb + i) = mt_pack8(pp);
    }
    return;
  }
  for (long long i = i0 + threadIdx.x; i < i1; i += 256) Cvt<T>::st(p, i, Cvt<T>::ld(p, i) - e.coef * __bfloat162float(e.u[i]));
}

template <typename T>
__global__ void __launch_bounds__(256) adamw_multi_kernel(const TensorEntry* __restrict__ tab, const int* __restrict__ chunk_start, int n, float lr,
                                                           float b1, float b2, float eps, float wd, float c1, float c2) {
  const int t = mt_find(chunk_start, n, blockIdx.x);
  const TensorEntry e = tab[t];
  const long long i0 = static_cast<long long>(blockIdx.x - chunk_start[t]) * MT_CHUNK_ELEMS;
  const long long i1 = min(e.numel, i0 + MT_CHUNK_ELEMS);
  T* p = static_cast<T*>(e.p);
  const T* g = static_cast<const T*>(e.g);
  if (std::is_same<T, __nv_bfloat16>::value && mt_wide(e, true, false, true)) {
    __nv_bfloat16* pb = reinterpret_cast<__nv_bfloat16*>(p);
    for (long long i = i0 + 8 * threadIdx.x; i < i1; i += 2048) {
      float gg[8], pp[8], mm[8], vv[8];
      unpack8_bf16(*reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(g) + i), gg);
      unpack8_bf16(*reinterpret_cast<const uint4*>(pb + i), pp);
      mt_ld8(e.s0 + i, mm);
      mt_ld8(e.s1 + i, vv);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        mm[k] = b1 * mm[k] + (1.f - b1) * gg[k];
        vv[k] = b2 * vv[k] + (1.f - b2) * gg[k] * gg[k];
        pp[k] = pp[k] * (1.f - lr * wd) - lr * c1 * mm[k] / (sqrtf(vv[k]) * c2 + eps);
      }
      mt_st8(e.s0 + i, mm);
      mt_st8(e.s1 + i, vv);
      *reinterpret_cast<uint4*>(pb + i) = mt_pack8(pp);
    }
    return;
  }
  for (long long i = i0 + threadIdx.x; i < i1; i += 256) {
    const float gi = Cvt<T>::ld(g, i);
    const float mi = b1 * e.s0[i] + (1.f - b1) * gi;
    const float vi = b2 * e.s1[i] + (1.f - b2) * gi * gi;
    e.s0[i] = mi;
    e.s1[i] = vi;
    Cvt<T>::st(p, i, Cvt<T>::ld(p, i) * (1.f - lr * wd) - lr * c1 * mi / (sqrtf(vi) * c2 + eps));
  }
}

}  // namespace cmb

// `tab`: device array of n entries {p, g, s0, s1, u, sumsq, numel (int64), coef (fp32), pad} (64 bytes); `chunk_start`: device int32[n + 1],
// prefix sums of ceil(numel / 4096).  `op`: 0 Muon momentum (+Σu² into the entries' sumsq slots, which the caller zeroed), 1 Frobenius
// normalisation of u, 2 p −= coef·u, 3 AdamW.  f = {mu, wd, nesterov} | {eps} | {} | {lr, b1, b2, eps, wd, c1, c2}.
extern "C" int cmb_optim_multi(int op, const void* tab, const int* chunk_start, int n, int total_chunks, int dtype, const float* f, void* stream) {
  if (n <= 0 || total_chunks <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const cmb::TensorEntry* t = static_cast<const cmb::TensorEntry*>(tab);
  switch (op) {
    case 0:
      CMB_DISPATCH_DTYPE(dtype, (cmb::muon_momentum_multi_kernel<T><<<total_chunks, 256, 0, s>>>(t, chunk_start, n, f[0], f[1], static_cast<int>(f[2]))));
      break;
    case 1:
      cmb::scale_inv_norm_multi_kernel<<<total_chunks, 256, 0, s>>>(t, chunk_start, n, f[0]);
      break;
    case 2:
      CMB_DISPATCH_DTYPE(dtype, (cmb::axpy_update_multi_kernel<T><<<total_chunks, 256, 0, s>>>(t, chunk_start, n)));
      break;
    case 3:
      CMB_DISPATCH_DTYPE(dtype, (cmb::adamw_multi_kernel<T><<<total_chunks, 256, 0, s>>>(t, chunk_start, n, f[0], f[1], f[2], f[3], f[4], f[5], f[6])));
      break;
    default:
      return 1;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// ---------------------------------------------------------------------------------------------- symmetric completion
namespace cmb {
// G[i][j] = G[j][i] for j > i (n×n bf16, row pitch ld): completes a matrix whose lower triangle was computed by a GEMM that
// skipped the tiles above the diagonal.  64×64 tiles through shared memory; both sides move whole 128-byte lines as bf16 pairs
// (n and ld even; the entry point falls back to the scalar form otherwise).
__global__ void __launch_bounds__(256) mirror_lower_kernel(__nv_bfloat16* __restrict__ g, int n, long long ld) {
  __shared__ __nv_bfloat16 tile[64][66];
  const int bi = blockIdx.y, bj = blockIdx.x;        // destination tile (rows bi, cols bj), only bj >= bi
  if (bj < bi) return;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 column pairs × 8 rows per pass
#pragma unroll
  for (int r = ty; r < 64; r += 8) {                 // source tile: rows bj·64.., cols bi·64..
    const int sr = bj * 64 + r, sc = bi * 64 + 2 * tx;
    __nv_bfloat162 v = __floats2bfloat162_rn(0.f, 0.f);
    if (sr < n && sc + 1 < n) v = *reinterpret_cast<const __nv_bfloat162*>(g + sr * ld + sc);
    else if (sr < n && sc < n) v.x = g[sr * ld + sc];
    tile[r][2 * tx] = v.x;
    tile[r][2 * tx + 1] = v.y;
  }
  __syncthreads();
#pragma unroll
  for (int r = ty; r < 64; r += 8) {
    const int dr = bi * 64 + r, dc = bj * 64 + 2 * tx;
    if (dr >= n || dc >= n) continue;
    const __nv_bfloat16 a = tile[2 * tx][r], b = tile[2 * tx + 1][r];
    if (dc > dr && dc + 1 < n) {                     // the whole pair lies above the diagonal
      __nv_bfloat162 v;
      v.x = a;
      v.y = b;
      *reinterpret_cast<__nv_bfloat162*>(g + dr * ld + dc) = v;
    } else {                                         // pair straddles the diagonal or the edge
      if (dc > dr) g[dr * ld + dc] = a;
      if (dc + 1 > dr && dc + 1 < n) g[dr * ld + dc + 1] = b;
    }
  }
}

// Scalar form for odd sizes / pitches.
__global__ void mirror_lower_scalar_kernel(__nv_bfloat16* __restrict__ g, int n, long long ld) {
  __shared__ __nv_bfloat16 tile[32][33];
  const int bi = blockIdx.y, bj = blockIdx.x;
  if (bj < bi) return;
  const int tx = threadIdx.x, ty = threadIdx.y;      // 32 × 8
  for (int r = ty; r < 32; r += 8) {
    const int sr = bj * 32 + r, sc = bi * 32 + tx;
    tile[r][tx] = (sr < n && sc < n) ? g[sr * ld + sc] : __float2bfloat16(0.f);
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    const int dr = bi * 32 + r, dc = bj * 32 + tx;
    if (dr < n && dc < n && dc > dr) g[dr * ld + dc] = tile[tx][r];
  }
}
}  // namespace cmb

extern "C" int cmb_mirror_lower(void* g, int n, long long ld, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if ((n % 2) == 0 && (ld % 2) == 0 && (reinterpret_cast<uintptr_t>(g) & 3) == 0) {
    const int t = (n + 63) / 64;
    cmb::mirror_lower_kernel<<<dim3(t, t), 256, 0, st>>>(static_cast<__nv_bfloat16*>(g), n, ld);
  } else {
    const int t = (n + 31) / 32;
    cmb::mirror_lower_scalar_kernel<<<dim3(t, t), dim3(32, 8), 0, st>>>(static_cast<__nv_bfloat16*>(g), n, ld);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
