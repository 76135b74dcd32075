// Per-tensor FP8 scaling primitives: abs-max with a NaN filter, and scale + clamp + round to e4m3.
//
//   amax     : out[0] = max(out[0], max |x_i| over the non-NaN elements)        (fp32 scalar, zeroed by the caller)
//   quantize : q_i = e4m3_rn_sat(clamp(x_i · inv_scale, ±448)), inv_scale read from the device (no host round trip), or
//              derived on the device from an amax scalar as 448 / max(amax, floor)
//
// Non-negative floats order like their bit patterns, so the cross-block maximum is an integer atomicMax.
// Semantics: cppmega_mlx/nn/_tilelang/fp8_amax.py:323-432 (amax), :435-507 (quantize), :726 (pack = amax then quantize).
// The tcgen05 GEMM can produce the same scalar from its epilogue (GEMM_EPI_AMAX in gemm_bf16.cu), so a following quantiser needs
// no separate reduction pass over the product.
#include <cuda_fp8.h>

#include "sm100.cuh"

namespace cmb {

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename T>
__global__ void __launch_bounds__(256) fp8_amax_kernel(const T* __restrict__ x, long long n, float* __restrict__ out) {
  __shared__ float red[8];
  float m = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float v = fabsf(to_f32<T>(x[i]));
    if (v == v) m = fmaxf(m, v);          // NaN filter
  }
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t = fmaxf(t, red[w]);
    atomicMax(reinterpret_cast<unsigned int*>(out), __float_as_uint(t));
  }
}

// mode 0: *scalar is inv_scale; mode 1: *scalar is an amax and inv_scale = 448 / max(amax, floor)
template <typename T>
__global__ void __launch_bounds__(256) fp8_quantize_kernel(const T* __restrict__ x, uint8_t* __restrict__ q, long long n,
                                                            const float* __restrict__ scalar, int mode, float floor_) {
  const float inv = mode == 0 ? *scalar : 448.f / fmaxf(*scalar, floor_);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float v = fminf(fmaxf(to_f32<T>(x[i]) * inv, -448.f), 448.f);
    q[i] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
  }
}

}  // namespace cmb

#define CMB_FP8_DISPATCH(dtype, CALL)                      \
  switch (dtype) {                                         \
    case 0: { using T = float; CALL; break; }              \
    case 1: { using T = __half; CALL; break; }             \
    case 2: { using T = __nv_bfloat16; CALL; break; }      \
    default: return 1;                                     \
  }

static inline int fp8_grid(long long n) {
  const long long b = (n + 255) / 256;
  return static_cast<int>(b < 1 ? 1 : (b > 148LL * 8 ? 148LL * 8 : b));
}

// dtype: 0 fp32, 1 fp16, 2 bf16.  `out` is one fp32 word; the maximum is folded into it (zero it for a fresh reduction).
extern "C" int cmb_fp8_amax(const void* x, long long n, int dtype, float* out, void* stream) {
  if (n <= 0) return 0;
  CMB_FP8_DISPATCH(dtype, (cmb::fp8_amax_kernel<T><<<fp8_grid(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const T*>(x), n, out)));
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

extern "C" int cmb_fp8_quantize(const void* x, void* q, long long n, int dtype, const float* scalar, int mode, float floor_, void* stream) {
  if (n <= 0) return 0;
  if (mode != 0 && mode != 1) return 1;
  CMB_FP8_DISPATCH(dtype, (cmb::fp8_quantize_kernel<T><<<fp8_grid(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(
                               static_cast<const T*>(x), static_cast<uint8_t*>(q), n, scalar, mode, floor_)));
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
