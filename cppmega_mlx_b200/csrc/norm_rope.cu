// Memory-bound row kernels: RMSNorm (fwd / bwd), split-half RoPE, SwiGLU (fwd / bwd).
// bf16 in / out, fp32 math, 128-bit accesses. These replace the reference's library calls
// mx.fast.rms_norm / mx.fast.rope (docs/production_kernel_routing.md:62-140); rotary layout and
// scaling tables follow cppmega_mlx/nn/attention.py:399-538 (tables are built on the host).
#include <mutex>

#include "sm100.cuh"

namespace cmb {

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(b[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 v;
  v.x = pack_bf16x2(f[0], f[1]);
  v.y = pack_bf16x2(f[2], f[3]);
  v.z = pack_bf16x2(f[4], f[5]);
  v.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = v;
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < THREADS / 32) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (l == 0) red[0] = t;
  }
  __syncthreads();
  const float out = red[0];
  __syncthreads();
  return out;
}

// One CTA per row (grid-stride over rows); cols % 8 == 0.
template <int THREADS>
__global__ void __launch_bounds__(THREADS) rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                               const __nv_bfloat16* __restrict__ w,
                                                               __nv_bfloat16* __restrict__ y, float* __restrict__ rstd,
                                                               int64_t rows, int cols, float eps) {
  __shared__ float red[32];
  const int nvec = cols >> 3;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const __nv_bfloat16* xr = x + row * cols;
    float ss = 0.f;
    for (int v = threadIdx.x; v < nvec; v += THREADS) {
      float f[8];
      load8(xr + 8 * v, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
    }
    ss = block_sum<THREADS>(ss, red);
    const float r = rsqrtf(ss / cols + eps);
    if (threadIdx.x == 0 && rstd != nullptr) rstd[row] = r;
    __nv_bfloat16* yr = y + row * cols;
    for (int v = threadIdx.x; v < nvec; v += THREADS) {
      float f[8], g[8];
      load8(xr + 8 * v, f);
      load8(w + 8 * v, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = f[i] * r * g[i];
      store8(yr + 8 * v, f);
    }
  }
}

// dx = rstd * (g*w) - x * rstd^3/cols * sum(g*w*x);  dw partials per CTA (summed on the host side).
template <int THREADS>
__global__ void __launch_bounds__(THREADS) rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ gy,
                                                               const __nv_bfloat16* __restrict__ x,
                                                               const __nv_bfloat16* __restrict__ w,
                                                               const float* __restrict__ rstd,
                                                               __nv_bfloat16* __restrict__ gx, float* __restrict__ gw_part,
                                                               int64_t rows, int cols) {
  __shared__ float red[32];
  const int nvec = cols >> 3;
  // Per-thread dw accumulators for up to 4 vectors per thread (cols <= THREADS*32); wider rows spill to a loop.
  constexpr int MAXV = 4;
  float acc[MAXV][8];
#pragma unroll
  for (int a = 0; a < MAXV; ++a)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[a][i] = 0.f;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const __nv_bfloat16* xr = x + row * cols;
    const __nv_bfloat16* gr = gy + row * cols;
    const float r = rstd[row];
    float dot = 0.f;
    for (int v = threadIdx.x; v < nvec; v += THREADS) {
      float fx[8], fg[8], fw[8];
      load8(xr + 8 * v, fx);
      load8(gr + 8 * v, fg);
      load8(w + 8 * v, fw);
#pragma unroll
      for (int i = 0; i < 8; ++i) dot += fg[i] * fw[i] * fx[i];
    }
    dot = block_sum<THREADS>(dot, red);
    const float c = dot * r * r * r / cols;
    __nv_bfloat16* gxr = gx + row * cols;
#pragma unroll
    for (int a = 0; a < MAXV; ++a) {
      const int v = threadIdx.x + a * THREADS;
      if (v < nvec) {
        float fx[8], fg[8], fw[8], o[8];
        load8(xr + 8 * v, fx);
        load8(gr + 8 * v, fg);
        load8(w + 8 * v, fw);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          o[i] = fg[i] * fw[i] * r - fx[i] * c;
          acc[a][i] += fg[i] * fx[i] * r;
        }
        store8(gxr + 8 * v, o);
      }
    }
    for (int v = threadIdx.x + MAXV * THREADS; v < nvec; v += THREADS) {  // very wide rows: atomics on the tail
      float fx[8], fg[8], fw[8], o[8];
      load8(xr + 8 * v, fx);
      load8(gr + 8 * v, fg);
      load8(w + 8 * v, fw);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        o[i] = fg[i] * fw[i] * r - fx[i] * c;
        atomicAdd(&gw_part[static_cast<size_t>(blockIdx.x) * cols + 8 * v + i], fg[i] * fx[i] * r);
      }
      store8(gxr + 8 * v, o);
    }
  }
#pragma unroll
  for (int a = 0; a < MAXV; ++a) {
    const int v = threadIdx.x + a * THREADS;
    if (v < nvec) {
#pragma unroll
      for (int i = 0; i < 8; ++i) gw_part[static_cast<size_t>(blockIdx.x) * cols + 8 * v + i] = acc[a][i];
    }
  }
}

// Warp-per-row variants for rows of up to VPL·256 columns: the whole row stays in registers (VPL 16-byte vectors per
// lane), so a row costs one pass over memory, one warp reduction and no block barrier, and every lane has VPL independent
// loads in flight.  Four warps (rows) per CTA, grid-stride over rows.
// With `delta` the row normalised is bf16(x + delta), which is also written to `sum` (the residual add that precedes the norm,
// same arithmetic as an element-wise add followed by the norm).
template <int VPL>
__global__ void __launch_bounds__(128) rmsnorm_fwd_warp_kernel(const __nv_bfloat16* __restrict__ x,
                                                                const __nv_bfloat16* __restrict__ w,
                                                                __nv_bfloat16* __restrict__ y, float* __restrict__ rstd,
                                                                int64_t rows, int cols, float eps,
                                                                const __nv_bfloat16* __restrict__ delta = nullptr,
                                                                __nv_bfloat16* __restrict__ sum = nullptr) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nvec = cols >> 3;
  for (int64_t row = blockIdx.x * 4 + warp; row < rows; row += static_cast<int64_t>(gridDim.x) * 4) {
    const __nv_bfloat16* xr = x + row * cols;
    float f[VPL][8];
    float ss = 0.f;
    if (delta != nullptr) {
      // every 16-byte load of both operands is issued before the first store to `sum`
      const __nv_bfloat16* dr = delta + row * cols;
      uint4 rx[VPL], rd[VPL];
#pragma unroll
      for (int a = 0; a < VPL; ++a) {
        const int v = lane + 32 * a;
        if (v < nvec) {
          rx[a] = *reinterpret_cast<const uint4*>(xr + 8 * v);
          rd[a] = *reinterpret_cast<const uint4*>(dr + 8 * v);
        }
      }
#pragma unroll
      for (int a = 0; a < VPL; ++a) {
        const int v = lane + 32 * a;
        if (v < nvec) {
          const __nv_bfloat162* bx = reinterpret_cast<const __nv_bfloat162*>(&rx[a]);
          const __nv_bfloat162* bd = reinterpret_cast<const __nv_bfloat162*>(&rd[a]);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 fx = __bfloat1622float2(bx[i]), fd = __bfloat1622float2(bd[i]);
            f[a][2 * i] = __bfloat162float(__float2bfloat16(fx.x + fd.x));
            f[a][2 * i + 1] = __bfloat162float(__float2bfloat16(fx.y + fd.y));
          }
          store8(sum + row * cols + 8 * v, f[a]);
#pragma unroll
          for (int i = 0; i < 8; ++i) ss += f[a][i] * f[a][i];
        }
      }
    } else {
#pragma unroll
      for (int a = 0; a < VPL; ++a) {
        const int v = lane + 32 * a;
        if (v < nvec) {
          load8(xr + 8 * v, f[a]);
#pragma unroll
          for (int i = 0; i < 8; ++i) ss += f[a][i] * f[a][i];
        }
      }
    }
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / cols + eps);
    if (lane == 0 && rstd != nullptr) rstd[row] = r;
    __nv_bfloat16* yr = y + row * cols;
#pragma unroll
    for (int a = 0; a < VPL; ++a) {
      const int v = lane + 32 * a;
      if (v < nvec) {
        float g[8];
        load8(w + 8 * v, g);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[a][i] = f[a][i] * r * g[i];
        store8(yr + 8 * v, f[a]);
      }
    }
  }
}

// Residual add fused with the RMS norm that follows it (inference: no statistics kept).  `sum = bf16(h + delta)` is written
// out as the new residual stream and the norm is taken of that rounded value, i.e. the same arithmetic as an element-wise add
// followed by the norm; one launch and one pass instead of two launches and three passes.  One CTA per row, one 16-byte
// vector per thread (cols ≤ 2048), and all three operands are loaded before anything is used: a decode step has one to a few
// dozen rows, so the launch is a single memory round trip plus one block reduction.
__global__ void __launch_bounds__(256) add_rmsnorm_block_kernel(const __nv_bfloat16* __restrict__ h,
                                                                 const __nv_bfloat16* __restrict__ delta,
                                                                 const __nv_bfloat16* __restrict__ w,
                                                                 __nv_bfloat16* __restrict__ sum, __nv_bfloat16* __restrict__ y,
                                                                 int64_t rows, int cols, float eps) {
  __shared__ float red[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int v = threadIdx.x;
  const bool active = v < (cols >> 3);
  float g[8];
  if (active) load8(w + 8 * v, g);
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    float f[8], d[8];
    float ss = 0.f;
    if (active) {
      load8(h + row * cols + 8 * v, f);
      load8(delta + row * cols + 8 * v, d);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        f[i] = __bfloat162float(__float2bfloat16(f[i] + d[i]));
        ss += f[i] * f[i];
      }
      store8(sum + row * cols + 8 * v, f);
    }
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float r = rsqrtf(tot / cols + eps);
    if (active) {
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = f[i] * r * g[i];
      store8(y + row * cols + 8 * v, f);
    }
    __syncthreads();     // `red` is rewritten by the next row
  }
}

// Shared memory of the backward warp kernel: one fp32 dw partial row per warp plus the weight as bf16.
static inline size_t rmsnorm_bwd_warp_smem(int cols) { return static_cast<size_t>(cols) * (4 * sizeof(float) + sizeof(__nv_bfloat16)); }

__device__ __forceinline__ void unpack8(const uint4& q, float (&f)[8]) {
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(b[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

// The row stays in registers as the packed bf16 it was loaded as (2·VPL 16-byte vectors per lane, all loads issued before the
// first use) and is unpacked once per pass; the dw partial of a warp lives in its own shared-memory row, updated with plain
// 16-byte read-modify-writes (a lane owns its columns), so the kernel needs ~100 registers instead of ~220 and four to five CTAs
// fit on an SM: enough loads in flight to keep HBM busy.
template <int VPL>
__global__ void __launch_bounds__(128, 4) rmsnorm_bwd_warp_kernel(const __nv_bfloat16* __restrict__ gy,
                                                                   const __nv_bfloat16* __restrict__ x,
                                                                   const __nv_bfloat16* __restrict__ w,
                                                                   const float* __restrict__ rstd, __nv_bfloat16* __restrict__ gx,
                                                                   float* __restrict__ gw_part, int64_t rows, int cols,
                                                                   const __nv_bfloat16* __restrict__ gres = nullptr) {
  // gres: gradient that reaches the normalised tensor along another path (the residual stream); it is added to gx here
  // instead of in a separate element-wise pass.
  extern __shared__ __align__(16) float gws[];   // [4][cols] per-warp dw partials, then the weight as bf16 [cols]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nvec = cols >> 3;
  __nv_bfloat16* ws = reinterpret_cast<__nv_bfloat16*>(gws + 4 * cols);
  for (int i = threadIdx.x; i < 4 * cols; i += 128) gws[i] = 0.f;
  for (int v = threadIdx.x; v < nvec; v += 128) reinterpret_cast<uint4*>(ws)[v] = reinterpret_cast<const uint4*>(w)[v];
  __syncthreads();
  float* mine = gws + warp * cols;
  for (int64_t row = blockIdx.x * 4 + warp; row < rows; row += static_cast<int64_t>(gridDim.x) * 4) {
    const __nv_bfloat16* xr = x + row * cols;
    const __nv_bfloat16* gr = gy + row * cols;
    uint4 rx[VPL], rg[VPL];
#pragma unroll
    for (int a = 0; a < VPL; ++a) {
      const int v = lane + 32 * a;
      if (v < nvec) {
        rx[a] = *reinterpret_cast<const uint4*>(xr + 8 * v);
        rg[a] = *reinterpret_cast<const uint4*>(gr + 8 * v);
      }
    }
    if (gres != nullptr) {   // start the residual-gradient row towards L2 while the reduction below runs
#pragma unroll
      for (int a = 0; a < VPL; ++a) {
        const int v = lane + 32 * a;
        if (v < nvec) asm volatile("prefetch.global.L2 [%0];" ::"l"(gres + row * cols + 8 * v));
      }
    }
    const float r = rstd[row];
    float dot = 0.f;
#pragma unroll
    for (int a = 0; a < VPL; ++a) {
      const int v = lane + 32 * a;
      if (v < nvec) {
        float fx[8], fg[8], fw[8];
        unpack8(rx[a], fx);
        unpack8(rg[a], fg);
        unpack8(reinterpret_cast<const uint4*>(ws)[v], fw);
#pragma unroll
        for (int i = 0; i < 8; ++i) dot += fg[i] * fw[i] * fx[i];
      }
    }
    dot = warp_sum(dot);
    const float c = dot * r * r * r / cols;
    __nv_bfloat16* gxr = gx + row * cols;
#pragma unroll
    for (int a = 0; a < VPL; ++a) {
      const int v = lane + 32 * a;
      if (v < nvec) {
        float fx[8], fg[8], fw[8], o[8];
        unpack8(rx[a], fx);
        unpack8(rg[a], fg);
        unpack8(reinterpret_cast<const uint4*>(ws)[v], fw);
        float4* acc = reinterpret_cast<float4*>(mine + 8 * v);
        float4 a0 = acc[0], a1 = acc[1];
        a0.x += fg[0] * fx[0] * r; a0.y += fg[1] * fx[1] * r; a0.z += fg[2] * fx[2] * r; a0.w += fg[3] * fx[3] * r;
        a1.x += fg[4] * fx[4] * r; a1.y += fg[5] * fx[5] * r; a1.z += fg[6] * fx[6] * r; a1.w += fg[7] * fx[7] * r;
        acc[0] = a0;
        acc[1] = a1;
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = fg[i] * fw[i] * r - fx[i] * c;
        if (gres != nullptr) {
          float fr[8];
          unpack8(*reinterpret_cast<const uint4*>(gres + row * cols + 8 * v), fr);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += fr[i];
        }
        store8(gxr + 8 * v, o);
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < cols; i += 128)
    gw_part[static_cast<size_t>(blockIdx.x) * cols + i] = (gws[i] + gws[cols + i]) + (gws[2 * cols + i] + gws[3 * cols + i]);
}

// SwiGLU: y = silu(g) * u with gu = [.., 2H] laid out as [gate | up] halves.
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ y, int64_t rows,
                                  int H) {
  const int64_t nvec = rows * (H >> 3);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = i / (H >> 3);
    const int c = static_cast<int>(i - row * (H >> 3)) * 8;
    float g[8], u[8], o[8];
    load8(gu + row * 2 * H + c, g);
    load8(gu + row * 2 * H + H + c, u);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = g[k] / (1.f + __expf(-g[k])) * u[k];
    store8(y + row * H + c, o);
  }
}
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gy, const __nv_bfloat16* __restrict__ gu,
                                  __nv_bfloat16* __restrict__ ggu, int64_t rows, int H) {
  const int64_t nvec = rows * (H >> 3);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = i / (H >> 3);
    const int c = static_cast<int>(i - row * (H >> 3)) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    load8(gu + row * 2 * H + c, g);
    load8(gu + row * 2 * H + H + c, u);
    load8(gy + row * H + c, d);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float s = 1.f / (1.f + __expf(-g[k]));
      const float silu = g[k] * s;
      du[k] = d[k] * silu;
      dg[k] = d[k] * u[k] * (s + silu * (1.f - s));
    }
    store8(ggu + row * 2 * H + c, dg);
    store8(ggu + row * 2 * H + H + c, du);
  }
}

// Split-half rotary on the trailing `rot` dims of each head: (x1, x2) -> (x1 c - x2 s, x2 c + x1 s),
// cos/sin tables [S, rot/2] fp32. `inverse` applies the transpose (backward). x: [B, S, H, D] bf16,
// the rotated slice starts at `off` inside D. In place when y == x.
__global__ void rope_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                            const float* __restrict__ cos_t, const float* __restrict__ sin_t, int64_t B, int S, int H,
                            int D, int off, int rot, int pos0, int inverse) {
  const int half = rot >> 1;
  const int64_t total = B * S * static_cast<int64_t>(H) * half;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int j = static_cast<int>(i % half);
    const int64_t bh = i / half;  // (b*S + s)*H + h
    const int s = static_cast<int>((bh / H) % S);
    const float c = cos_t[static_cast<int64_t>(s + pos0) * half + j];
    float sn = sin_t[static_cast<int64_t>(s + pos0) * half + j];
    if (inverse) sn = -sn;
    const __nv_bfloat16* xp = x + bh * D + off;
    __nv_bfloat16* yp = y + bh * D + off;
    const float a = __bfloat162float(xp[j]);
    const float b = __bfloat162float(xp[j + half]);
    yp[j] = __float2bfloat16(a * c - b * sn);
    yp[j + half] = __float2bfloat16(b * c + a * sn);
  }
}

}  // namespace cmb

extern "C" int cmb_rmsnorm_fwd(const void* x, const void* w, void* y, void* rstd, int64_t rows, int cols, float eps,
                               void* stream) {
  if (cols % 8) return 1;
  if (cols <= 2048 && rows >= 256) {   // whole row in registers, one warp per row (fewer rows: one CTA per row has more loads in flight)
    const int64_t want = (rows + 3) / 4;
    const int wgrid = static_cast<int>(want < 148 * 16 ? want : 148 * 16);
    cmb::rmsnorm_fwd_warp_kernel<8><<<wgrid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y),
        static_cast<float*>(rstd), rows, cols, eps);
    return cudaGetLastError() == cudaSuccess ? 0 : 2;
  }
  const int grid = static_cast<int>(rows < 148 * 16 ? rows : 148 * 16);
  cmb::rmsnorm_fwd_kernel<256><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y),
      static_cast<float*>(rstd), rows, cols, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// Training form of the fused residual add + norm: sum = bf16(h + delta), y = rmsnorm(sum)·w, rstd kept for the backward.
// cols a multiple of 8 and at most 2048.
extern "C" int cmb_add_rmsnorm_train(const void* h, const void* delta, const void* w, void* sum, void* y, void* rstd, int64_t rows, int cols,
                                     float eps, void* stream) {
  if (cols % 8 || cols > 2048 || rows <= 0) return 1;
  const int64_t want = (rows + 3) / 4;
  const int wgrid = static_cast<int>(want < 148 * 16 ? want : 148 * 16);
  cmb::rmsnorm_fwd_warp_kernel<8><<<wgrid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(h), static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y), static_cast<float*>(rstd), rows,
      cols, eps, static_cast<const __nv_bfloat16*>(delta), static_cast<__nv_bfloat16*>(sum));
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// gx = rmsnorm backward of gy + gres (the gradient arriving on the residual stream); same contract as cmb_rmsnorm_bwd otherwise.
// cols at most 2048, rows at least 4.
extern "C" int cmb_rmsnorm_bwd_add(const void* gy, const void* x, const void* w, const void* rstd, const void* gres, void* gx, void* gw_part,
                                   int64_t rows, int cols, int nblk, void* stream) {
  if (cols % 8 || cols > 2048 || rows < 4) return 1;
  cmb::rmsnorm_bwd_warp_kernel<8><<<nblk, 128, cmb::rmsnorm_bwd_warp_smem(cols), static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gy), static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
      static_cast<const float*>(rstd), static_cast<__nv_bfloat16*>(gx), static_cast<float*>(gw_part), rows, cols,
      static_cast<const __nv_bfloat16*>(gres));
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// sum = h + delta (bf16), y = rmsnorm(sum)·w.  cols a multiple of 8 and at most 2048; all tensors contiguous [rows, cols].
extern "C" int cmb_add_rmsnorm(const void* h, const void* delta, const void* w, void* sum, void* y, int64_t rows, int cols, float eps,
                               void* stream) {
  if (cols % 8 || cols > 2048 || rows <= 0) return 1;
  const int grid = static_cast<int>(rows < 148 * 8 ? rows : 148 * 8);
  cmb::add_rmsnorm_block_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(h), static_cast<const __nv_bfloat16*>(delta), static_cast<const __nv_bfloat16*>(w),
      static_cast<__nv_bfloat16*>(sum), static_cast<__nv_bfloat16*>(y), rows, cols, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

extern "C" int cmb_rmsnorm_bwd(const void* gy, const void* x, const void* w, const void* rstd, void* gx, void* gw_part,
                               int64_t rows, int cols, int nblk, void* stream) {
  if (cols % 8) return 1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cols <= 2048 && rows >= 4) {   // a CTA without rows still writes its (zero) dw partial
    cmb::rmsnorm_bwd_warp_kernel<8><<<nblk, 128, cmb::rmsnorm_bwd_warp_smem(cols), s>>>(
        static_cast<const __nv_bfloat16*>(gy), static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
        static_cast<const float*>(rstd), static_cast<__nv_bfloat16*>(gx), static_cast<float*>(gw_part), rows, cols);
    return cudaGetLastError() == cudaSuccess ? 0 : 2;
  }
  if ((cols >> 3) > 256 * 4) cudaMemsetAsync(gw_part, 0, sizeof(float) * static_cast<size_t>(nblk) * cols, s);
  cmb::rmsnorm_bwd_kernel<256><<<nblk, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(gy),
                                                      static_cast<const __nv_bfloat16*>(x),
                                                      static_cast<const __nv_bfloat16*>(w), static_cast<const float*>(rstd),
                                                      static_cast<__nv_bfloat16*>(gx), static_cast<float*>(gw_part), rows, cols);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

extern "C" int cmb_swiglu_fwd(const void* gu, void* y, int64_t rows, int H, void* stream) {
  if (H % 8) return 1;
  cmb::swiglu_fwd_kernel<<<148 * 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<__nv_bfloat16*>(y), rows, H);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
extern "C" int cmb_swiglu_bwd(const void* gy, const void* gu, void* ggu, int64_t rows, int H, void* stream) {
  if (H % 8) return 1;
  cmb::swiglu_bwd_kernel<<<148 * 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gy), static_cast<const __nv_bfloat16*>(gu), static_cast<__nv_bfloat16*>(ggu), rows, H);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
extern "C" int cmb_rope(const void* x, void* y, const void* cos_t, const void* sin_t, int64_t B, int S, int H, int D,
                        int off, int rot, int pos0, int inverse, void* stream) {
  if (rot % 2 || off + rot > D) return 1;
  cmb::rope_kernel<<<148 * 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), static_cast<const float*>(cos_t),
      static_cast<const float*>(sin_t), B, S, H, D, off, rot, pos0, inverse);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// ---------------------------------------------------------------------------------------------------------------
// RMSNorm backward for callers that cannot allocate device memory (declared in rmsnorm_noalloc.h).
//
// The regular entry point above hands the per-CTA partial sums of dW back to the caller, who has to provide that
// buffer. This variant keeps the partials in a fixed device array that lives inside the library image, and reduces
// them into the caller's dW vector itself, so a caller needs nothing but its inputs and outputs.
namespace cmb {

constexpr int NOALLOC_MAX_COLS = 8192;   // widest row the entry point accepts
constexpr int NOALLOC_MAX_BLOCKS = 148;  // partial rows (one per CTA, one CTA per SM)

// 148 × 8192 fp32 = 4.6 MiB, resident on every GPU that loads the library until the process exits.
static __device__ __align__(256) float g_rmsnorm_noalloc_partials[NOALLOC_MAX_BLOCKS * NOALLOC_MAX_COLS];

__global__ void rmsnorm_noalloc_reduce_kernel(const float* __restrict__ part, float* __restrict__ gw, int nblk, int cols) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float acc = 0.f;
  for (int b = 0; b < nblk; ++b) acc += part[static_cast<size_t>(b) * cols + c];
  gw[c] = acc;
}

}  // namespace cmb

extern "C" int cmb_rmsnorm_bwd_noalloc(const void* gy, const void* x, const void* w, const void* rstd, void* gx,
                                       float* gw, int64_t rows, int cols, void* stream) {
  if (gy == nullptr || x == nullptr || w == nullptr || rstd == nullptr || gx == nullptr || gw == nullptr) return -1;
  if (rows <= 0 || cols <= 0 || cols % 8 != 0) return -2;
  if (cols > cmb::NOALLOC_MAX_COLS) return -3;
  // The array's name is only a host-side handle; kernels need its device address, which differs per GPU. It is looked
  // up once per device (with that device current) on the first call made there and cached.
  static std::mutex mu;
  static float* dev_ptr[64] = {nullptr};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -4;
  float* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev_ptr[dev] == nullptr) {
      void* p = nullptr;
      if (cudaGetSymbolAddress(&p, cmb::g_rmsnorm_noalloc_partials) != cudaSuccess || p == nullptr) return -5;
      dev_ptr[dev] = static_cast<float*>(p);
    }
    scratch = dev_ptr[dev];
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int nblk = static_cast<int>(rows < cmb::NOALLOC_MAX_BLOCKS ? rows : cmb::NOALLOC_MAX_BLOCKS);
  // Every partial row that the reduction reads (rows 0..nblk-1, columns 0..cols-1) is fully overwritten by the first
  // kernel, so nothing left over from an earlier call can leak in and no clearing is needed.
  // Same kernel choice as cmb_rmsnorm_bwd, so both entry points return identical bits.
  if (cols <= 2048 && rows >= 4)
    cmb::rmsnorm_bwd_warp_kernel<8><<<nblk, 128, cmb::rmsnorm_bwd_warp_smem(cols), s>>>(
        static_cast<const __nv_bfloat16*>(gy), static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
        static_cast<const float*>(rstd), static_cast<__nv_bfloat16*>(gx), scratch, rows, cols);
  else
    cmb::rmsnorm_bwd_kernel<256><<<nblk, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(gy), static_cast<const __nv_bfloat16*>(x),
                                                      static_cast<const __nv_bfloat16*>(w), static_cast<const float*>(rstd),
                                                      static_cast<__nv_bfloat16*>(gx), scratch, rows, cols);
  if (cudaGetLastError() != cudaSuccess) return -6;
  cmb::rmsnorm_noalloc_reduce_kernel<<<(cols + 255) / 256, 256, 0, s>>>(scratch, gw, nblk, cols);
  return cudaGetLastError() == cudaSuccess ? 0 : -6;
}
