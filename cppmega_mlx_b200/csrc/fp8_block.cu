// e4m3 weights with one fp32 scale per 128×128 block → bf16, one pass (sm_100a).
//
// The stored form is the DeepSeek-V3 checkpoint layout: `w_fp8[r, c]` (e4m3) and `scale_inv[r / 128, c / 128]` (fp32) with
// `w ≈ w_fp8 · scale_inv`.  Each thread converts 16 consecutive elements of one row (one 16-byte load, two 16-byte stores);
// a 16-element run never crosses a 128-column block, so it needs one scale.  Matrices are stacked along dim 0 (`batch`).
//
// Reference: cppmega_v4/nn/_external/_mlx_lm_fp8_dequant_vendored.py (block dequantisation) and
// cppmega_v4/_tilelang/fused_fp8_gemm.py (dequantise inside the GEMM's operand load); here the dequantised tile goes
// through HBM once and the product runs on the bf16 tcgen05 GEMM.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace cmb {

__global__ void __launch_bounds__(256) fp8_block_dequant_kernel(const uint8_t* __restrict__ w, const float* __restrict__ scale_inv,
                                                                __nv_bfloat16* __restrict__ out, long long batch, int rows, int cols,
                                                                int blocks_r, int blocks_c) {
  const int runs_per_row = cols / 16;
  const long long total = batch * rows * runs_per_row;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * 256) {
    const int run = static_cast<int>(i % runs_per_row);
    const long long rr = i / runs_per_row;
    const int r = static_cast<int>(rr % rows);
    const long long b = rr / rows;
    const float s = scale_inv[(b * blocks_r + r / 128) * blocks_c + (run * 16) / 128];
    const long long off = (b * rows + r) * static_cast<long long>(cols) + run * 16;
    const uint4 raw = *reinterpret_cast<const uint4*>(w + off);
    const uint8_t* bytes = reinterpret_cast<const uint8_t*>(&raw);
    __align__(16) __nv_bfloat16 o[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      __nv_fp8_e4m3 v;
      v.__x = bytes[j];
      o[j] = __float2bfloat16(static_cast<float>(v) * s);
    }
    uint4* dst = reinterpret_cast<uint4*>(out + off);
    dst[0] = *reinterpret_cast<const uint4*>(o);
    dst[1] = *reinterpret_cast<const uint4*>(o + 8);
  }
}

}  // namespace cmb

// cols must be a multiple of 16 and both pointers 16-byte aligned (returns 1 otherwise).
extern "C" int cmb_fp8_block_dequant(const void* w, const void* scale_inv, void* out, long long batch, int rows, int cols, void* stream) {
  if (batch <= 0 || rows <= 0 || cols <= 0 || cols % 16) return 1;
  if ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out)) & 15) return 1;
  const long long total = batch * rows * (cols / 16);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  cmb::fp8_block_dequant_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(w), static_cast<const float*>(scale_inv), static_cast<__nv_bfloat16*>(out), batch, rows, cols,
      (rows + 127) / 128, (cols + 127) / 128);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
