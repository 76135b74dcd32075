// Element-wise stages of the chunked Mamba3 scan (the GEMM-shaped stages run on the batched tcgen05
// GEMM; ops/mamba3_scan_cuda.py sequences both).  Shapes: x, z, y, dy … [B,S,H,P]; per-chunk vectors
// [B,nc,H,L]; chunk states [B,nc,H,P,N].  All index arithmetic is 64-bit.
//
// Recurrence being computed: h_t = exp(A_t dt_t) h_{t-1} + x_t ⊗ B_t,  y_t = C_t·h_t + D x_t,
// out_t = silu(z_t) y_t  — cppmega_mlx/nn/mamba3.py:339-408 (token loop) and
// cppmega_mlx/nn/_tilelang/mamba3.py:71-144 / :168-327 (the reference's per-lane Metal kernels).
#include "sm100.cuh"

namespace cmb {

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + __expf(-v)); }

// cum[b,c,h,t] = Σ_{t'≤t} A·dt over the chunk. One warp per (b,c,h); L ≤ 1024, L % 32 == 0.
__global__ void m3_cumsum_kernel(const float* __restrict__ A, const float* __restrict__ dt, float* __restrict__ cum,
                                 int Bn, int S, int H, int L) {
  const int nc = S / L;
  const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= static_cast<long long>(Bn) * nc * H) return;
  const int h = static_cast<int>(row % H);
  const int c = static_cast<int>((row / H) % nc);
  const int b = static_cast<int>(row / (static_cast<long long>(H) * nc));
  const int per = L / 32;
  float run = 0.f;
  float vals[32];
  const long long base = (static_cast<long long>(b) * S + static_cast<long long>(c) * L) * H + h;
  for (int i = 0; i < per; ++i) {
    const int t = lane * per + i;
    const long long idx = base + static_cast<long long>(t) * H;
    run += A[idx] * dt[idx];
    vals[i] = run;
  }
  // exclusive prefix of the lane totals
  float tot = run;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, tot, o);
    if (lane >= o) tot += n;
  }
  const float off = tot - run;
  float* out = cum + row * L;
  for (int i = 0; i < per; ++i) out[lane * per + i] = vals[i] + off;
}

// xw = x · exp(cum_L − cum_t)   (bf16 out, contiguous).  One thread per bf16 pair.
__global__ void m3_xw_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ cum,
                             __nv_bfloat16* __restrict__ xw, int Bn, int S, int H, int P, int L) {
  const int nc = S / L;
  const long long n2 = static_cast<long long>(Bn) * S * H * (P / 2);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n2;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long bsh = i / (P / 2);
    const int h = static_cast<int>(bsh % H);
    const long long bs = bsh / H;
    const int s = static_cast<int>(bs % S);
    const int b = static_cast<int>(bs / S);
    const int c = s / L, t = s - c * L;
    const float* cr = cum + ((static_cast<long long>(b) * nc + c) * H + h) * L;
    const float w = __expf(cr[L - 1] - cr[t]);
    const float2 v = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(x)[i]);
    reinterpret_cast<__nv_bfloat162*>(xw)[i] = __floats2bfloat162_rn(v.x * w, v.y * w);
  }
}

// 16-byte form of the above (P % 8 == 0): one thread per 8 channels.
__global__ void __launch_bounds__(256) m3_xw_w8_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ cum,
                                                        __nv_bfloat16* __restrict__ xw, int Bn, int S, int H, int P, int L) {
  const int nc = S / L, p8 = P >> 3;
  const long long n8 = static_cast<long long>(Bn) * S * H * p8;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint4 raw = reinterpret_cast<const uint4*>(x)[i];
    const long long bsh = i / p8;
    const int h = static_cast<int>(bsh % H);
    const long long bs = bsh / H;
    const int s = static_cast<int>(bs % S);
    const int b = static_cast<int>(bs / S);
    const int c = s / L, t = s - c * L;
    const float* cr = cum + ((static_cast<long long>(b) * nc + c) * H + h) * L;
    const float w = __expf(cr[L - 1] - cr[t]);
    float v[8];
    unpack8_bf16(raw, v);
    uint4 o;
    o.x = pack_bf16x2(v[0] * w, v[1] * w); o.y = pack_bf16x2(v[2] * w, v[3] * w);
    o.z = pack_bf16x2(v[4] * w, v[5] * w); o.w = pack_bf16x2(v[6] * w, v[7] * w);
    reinterpret_cast<uint4*>(xw)[i] = o;
  }
}

// Sequential carry over chunks: Hc[c] = state entering chunk c; state ← exp(cum_L[c]) state + S_loc[c].
__global__ void m3_state_pass_kernel(const float* __restrict__ sloc, const float* __restrict__ cum,
                                     const float* __restrict__ h0, __nv_bfloat16* __restrict__ hc,
                                     float* __restrict__ hlast, int Bn, int nc, int H, int PN, int L) {
  const long long n = static_cast<long long>(Bn) * H * PN;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int e = static_cast<int>(i % PN);
    const int h = static_cast<int>((i / PN) % H);
    const int b = static_cast<int>(i / (static_cast<long long>(PN) * H));
    float st = h0 != nullptr ? h0[i] : 0.f;
    for (int c = 0; c < nc; ++c) {
      const long long idx = ((static_cast<long long>(b) * nc + c) * H + h) * PN + e;
      hc[idx] = __float2bfloat16(st);
      const float d = __expf(cum[((static_cast<long long>(b) * nc + c) * H + h) * L + L - 1]);
      st = d * st + sloc[idx];
    }
    hlast[i] = st;
  }
}

// Four state entries per thread (PN % 4 == 0) and the chunk loop unrolled by four with the loads issued first: the recurrence
// is a dependent chain, the loads are not.
__global__ void __launch_bounds__(256) m3_state_pass_w4_kernel(const float* __restrict__ sloc, const float* __restrict__ cum,
                                                                const float* __restrict__ h0, __nv_bfloat16* __restrict__ hc,
                                                                float* __restrict__ hlast, int Bn, int nc, int H, int PN, int L) {
  const int pn4 = PN >> 2;
  const long long n4 = static_cast<long long>(Bn) * H * pn4;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int e = static_cast<int>(i % pn4) * 4;
    const int h = static_cast<int>((i / pn4) % H);
    const int b = static_cast<int>(i / (static_cast<long long>(pn4) * H));
    float4 st = h0 != nullptr ? reinterpret_cast<const float4*>(h0)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    for (int c0 = 0; c0 < nc; c0 += 4) {
      float4 sl[4];
      float d[4];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (c0 + k < nc) {
          const long long row = (static_cast<long long>(b) * nc + c0 + k) * H + h;
          sl[k] = *reinterpret_cast<const float4*>(sloc + row * PN + e);
          d[k] = cum[row * L + L - 1];
        }
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (c0 + k < nc) {
          const long long row = (static_cast<long long>(b) * nc + c0 + k) * H + h;
          uint2 o;
          o.x = pack_bf16x2(st.x, st.y);
          o.y = pack_bf16x2(st.z, st.w);
          *reinterpret_cast<uint2*>(hc + row * PN + e) = o;
          const float dk = __expf(d[k]);
          st.x = dk * st.x + sl[k].x; st.y = dk * st.y + sl[k].y; st.z = dk * st.z + sl[k].z; st.w = dk * st.w + sl[k].w;
        }
    }
    reinterpret_cast<float4*>(hlast)[i] = st;
  }
}

// y_pre = Y + D x ; out = silu(z) y_pre.   z may be a strided view (element strides zs_b, zs_s, zs_h).
__global__ void m3_finalize_fwd_kernel(const float* __restrict__ Y, const __nv_bfloat16* __restrict__ x,
                                       const __nv_bfloat16* __restrict__ z, const float* __restrict__ D,
                                       __nv_bfloat16* __restrict__ ypre, __nv_bfloat16* __restrict__ out, int Bn, int S,
                                       int H, int P, long long zs_b, long long zs_s, long long zs_h) {
  const long long n2 = static_cast<long long>(Bn) * S * H * (P / 2);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n2;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int pp = static_cast<int>(i % (P / 2));
    const long long bsh = i / (P / 2);
    const int h = static_cast<int>(bsh % H);
    const long long bs = bsh / H;
    const int s = static_cast<int>(bs % S);
    const int b = static_cast<int>(bs / S);
    const float2 xv = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(x)[i]);
    const float2 yv = reinterpret_cast<const float2*>(Y)[i];
    const float d = D[h];
    const float y0 = yv.x + d * xv.x, y1 = yv.y + d * xv.y;
    const __nv_bfloat162 zz = *reinterpret_cast<const __nv_bfloat162*>(z + b * zs_b + s * zs_s + h * zs_h + 2 * pp);
    const float2 zv = __bfloat1622float2(zz);
    reinterpret_cast<__nv_bfloat162*>(ypre)[i] = __floats2bfloat162_rn(y0, y1);
    reinterpret_cast<__nv_bfloat162*>(out)[i] = __floats2bfloat162_rn(silu_f(zv.x) * y0, silu_f(zv.y) * y1);
  }
}

// 16-byte form of the above (P % 8 == 0, z strides multiples of 8): one thread per 8 channels.
__global__ void __launch_bounds__(256) m3_finalize_fwd_w8_kernel(const float* __restrict__ Y, const __nv_bfloat16* __restrict__ x,
                                                                  const __nv_bfloat16* __restrict__ z, const float* __restrict__ D,
                                                                  __nv_bfloat16* __restrict__ ypre, __nv_bfloat16* __restrict__ out, int Bn,
                                                                  int S, int H, int P, long long zs_b, long long zs_s, long long zs_h) {
  const int p8 = P >> 3;
  const long long n8 = static_cast<long long>(Bn) * S * H * p8;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int pp = static_cast<int>(i % p8) * 8;
    const long long bsh = i / p8;
    const int h = static_cast<int>(bsh % H);
    const long long bs = bsh / H;
    const int s = static_cast<int>(bs % S);
    const int b = static_cast<int>(bs / S);
    const float4 y0 = reinterpret_cast<const float4*>(Y)[2 * i], y1 = reinterpret_cast<const float4*>(Y)[2 * i + 1];
    float xv[8], zv[8];
    unpack8_bf16(reinterpret_cast<const uint4*>(x)[i], xv);
    unpack8_bf16(*reinterpret_cast<const uint4*>(z + b * zs_b + s * zs_s + h * zs_h + pp), zv);
    const float d = D[h];
    const float yy[8] = {y0.x + d * xv[0], y0.y + d * xv[1], y0.z + d * xv[2], y0.w + d * xv[3],
                         y1.x + d * xv[4], y1.y + d * xv[5], y1.z + d * xv[6], y1.w + d * xv[7]};
    uint4 o;
    o.x = pack_bf16x2(yy[0], yy[1]); o.y = pack_bf16x2(yy[2], yy[3]); o.z = pack_bf16x2(yy[4], yy[5]); o.w = pack_bf16x2(yy[6], yy[7]);
    reinterpret_cast<uint4*>(ypre)[i] = o;
    o.x = pack_bf16x2(silu_f(zv[0]) * yy[0], silu_f(zv[1]) * yy[1]); o.y = pack_bf16x2(silu_f(zv[2]) * yy[2], silu_f(zv[3]) * yy[3]);
    o.z = pack_bf16x2(silu_f(zv[4]) * yy[4], silu_f(zv[5]) * yy[5]); o.w = pack_bf16x2(silu_f(zv[6]) * yy[6], silu_f(zv[7]) * yy[7]);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

// Intra-chunk matrices of all heads of a group from the group's score tile:  M[b,c,h,t,s] = CB[b,c,g,t,s] · exp(cum_h[t] − cum_h[s]) · [s ≤ t].
// C·Bᵀ is shared by the H/G heads of a group, so it is formed once per group (fp32) and expanded here per head, instead of running
// the product once per head with the decay in its epilogue (8× the tiles, each bound by that epilogue).  One thread per 8 columns.
__global__ void __launch_bounds__(256) m3_expand_decay_kernel(const float* __restrict__ CB, const float* __restrict__ cum,
                                                               __nv_bfloat16* __restrict__ M, int Bn, int nc, int H, int G, int L) {
  const int l8 = L >> 3, hg = H / G;
  const long long n8 = static_cast<long long>(Bn) * nc * H * L * l8;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int s = static_cast<int>(i % l8) * 8;
    const long long row = i / l8;                 // ((b·nc + c)·H + h)·L + t
    const int t = static_cast<int>(row % L);
    const long long bch = row / L;
    const int h = static_cast<int>(bch % H);
    const long long bc = bch / H;
    uint4 o = make_uint4(0u, 0u, 0u, 0u);
    if (s <= t) {
      const float* cb = CB + ((bc * G + h / hg) * L + t) * L + s;
      const float* cr = cum + bch * L;
      const float4 a0 = *reinterpret_cast<const float4*>(cb), a1 = *reinterpret_cast<const float4*>(cb + 4);
      const float4 c0 = *reinterpret_cast<const float4*>(cr + s), c1 = *reinterpret_cast<const float4*>(cr + s + 4);
      const float ct = cr[t];
      const float v[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
      float m[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) m[k] = (s + k <= t) ? v[k] * __expf(ct - cs[k]) : 0.f;
      o.x = pack_bf16x2(m[0], m[1]); o.y = pack_bf16x2(m[2], m[3]); o.z = pack_bf16x2(m[4], m[5]); o.w = pack_bf16x2(m[6], m[7]);
    }
    *reinterpret_cast<uint4*>(M + row * L + s) = o;
  }
}

// Backward prologue. One warp per (b,s,h):
//   dy = dout·silu(z) ; dz = dout·y_pre·silu'(z) ; dye = dy·exp(cum_t) ; dx_acc = D·dy (fp32)
//   dcum[b,c,h,t] = Σ_p dy·(y_pre − D x)      (row-factor part of d/dcum)
//   dD[h] += Σ dy·x                            (block-reduced, one atomic per block)
// Blocks are laid out so that the 8 warps of a block share h (consecutive s).
__global__ void __launch_bounds__(256) m3_bwd_pre_kernel(
    const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ z, const __nv_bfloat16* __restrict__ ypre,
    const __nv_bfloat16* __restrict__ x, const float* __restrict__ D, const float* __restrict__ cum,
    __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dz, __nv_bfloat16* __restrict__ dye,
    float* __restrict__ dx_acc, float* __restrict__ dcum, float* __restrict__ dD, int Bn, int S, int H, int P, int L,
    long long zs_b, long long zs_s, long long zs_h) {
  __shared__ float red[8];
  const int nc = S / L;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // block index → (b, s-block, h)
  const long long blk = blockIdx.x;
  const int h = static_cast<int>(blk % H);
  const long long q = blk / H;
  const int sblocks = (S + 7) / 8;
  const int sb = static_cast<int>(q % sblocks);
  const int b = static_cast<int>(q / sblocks);
  const int s = sb * 8 + warp;
  float dacc = 0.f;
  if (b < Bn && s < S) {
    const int c = s / L, t = s - c * L;
    const long long crow = ((static_cast<long long>(b) * nc + c) * H + h) * L;
    const float e = __expf(cum[crow + t]);
    const float d = D[h];
    const long long base = ((static_cast<long long>(b) * S + s) * H + h) * P;
    const __nv_bfloat16* zr = z + b * zs_b + s * zs_s + h * zs_h;
    float rsum = 0.f;
    for (int p = 2 * lane; p < P; p += 64) {
      const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dout + base + p));
      const float2 zv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(zr + p));
      const float2 yv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(ypre + base + p));
      const float2 xv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + base + p));
      const float s0 = 1.f / (1.f + __expf(-zv.x)), s1 = 1.f / (1.f + __expf(-zv.y));
      const float sl0 = zv.x * s0, sl1 = zv.y * s1;
      const float dy0 = g.x * sl0, dy1 = g.y * sl1;
      *reinterpret_cast<__nv_bfloat162*>(dy + base + p) = __floats2bfloat162_rn(dy0, dy1);
      *reinterpret_cast<__nv_bfloat162*>(dz + base + p) =
          __floats2bfloat162_rn(g.x * yv.x * (s0 + sl0 * (1.f - s0)), g.y * yv.y * (s1 + sl1 * (1.f - s1)));
      *reinterpret_cast<__nv_bfloat162*>(dye + base + p) = __floats2bfloat162_rn(dy0 * e, dy1 * e);
      *reinterpret_cast<float2*>(dx_acc + base + p) = make_float2(d * dy0, d * dy1);
      rsum += dy0 * (yv.x - d * xv.x) + dy1 * (yv.y - d * xv.y);
      dacc += dy0 * xv.x + dy1 * xv.y;
    }
    rsum = warp_sum(rsum);
    if (lane == 0) dcum[crow + t] = rsum;
  }
  dacc = warp_sum(dacc);
  if (lane == 0) red[warp] = dacc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += red[w];
    atomicAdd(&dD[h], t);
  }
}

// The same prologue with 16-byte accesses: a thread owns 8 consecutive channels of one (b,s,h) row, P/8 lanes share a row and a
// block covers 256·8/P consecutive tokens of one head.  P ∈ {32, 64, 128, 256}; z strides multiples of 8.
template <int LPR>   // lanes per row = P / 8
__global__ void __launch_bounds__(256) m3_bwd_pre_w8_kernel(
    const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ z, const __nv_bfloat16* __restrict__ ypre,
    const __nv_bfloat16* __restrict__ x, const float* __restrict__ D, const float* __restrict__ cum,
    __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dz, __nv_bfloat16* __restrict__ dye,
    float* __restrict__ dx_acc, float* __restrict__ dcum, float* __restrict__ dD, int Bn, int S, int H, int L,
    long long zs_b, long long zs_s, long long zs_h) {
  constexpr int P = LPR * 8, ROWS = 256 / LPR;
  __shared__ float red[8];
  const int nc = S / L;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long blk = blockIdx.x;
  const int h = static_cast<int>(blk % H);
  const long long q = blk / H;
  const int sblocks = (S + ROWS - 1) / ROWS;
  const int sb = static_cast<int>(q % sblocks);
  const int b = static_cast<int>(q / sblocks);
  const int s = sb * ROWS + threadIdx.x / LPR;
  const int p = (threadIdx.x % LPR) * 8;
  float dacc = 0.f, rsum = 0.f;
  const bool live = b < Bn && s < S;
  int c = 0, t = 0;
  long long crow = 0;
  if (live) {
    c = s / L;
    t = s - c * L;
    crow = ((static_cast<long long>(b) * nc + c) * H + h) * L;
    const float e = __expf(cum[crow + t]);
    const float d = D[h];
    const long long base = ((static_cast<long long>(b) * S + s) * H + h) * P + p;
    float g[8], zv[8], yv[8], xv[8], o_dy[8], o_dz[8], o_dye[8], o_dx[8];
    unpack8_bf16(*reinterpret_cast<const uint4*>(dout + base), g);
    unpack8_bf16(*reinterpret_cast<const uint4*>(z + b * zs_b + s * zs_s + h * zs_h + p), zv);
    unpack8_bf16(*reinterpret_cast<const uint4*>(ypre + base), yv);
    unpack8_bf16(*reinterpret_cast<const uint4*>(x + base), xv);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float sg = 1.f / (1.f + __expf(-zv[i]));
      const float sl = zv[i] * sg;
      const float dyi = g[i] * sl;
      o_dy[i] = dyi;
      o_dz[i] = g[i] * yv[i] * (sg + sl * (1.f - sg));
      o_dye[i] = dyi * e;
      o_dx[i] = d * dyi;
      rsum += dyi * (yv[i] - d * xv[i]);
      dacc += dyi * xv[i];
    }
    uint4 o;
    o.x = pack_bf16x2(o_dy[0], o_dy[1]); o.y = pack_bf16x2(o_dy[2], o_dy[3]); o.z = pack_bf16x2(o_dy[4], o_dy[5]); o.w = pack_bf16x2(o_dy[6], o_dy[7]);
    *reinterpret_cast<uint4*>(dy + base) = o;
    o.x = pack_bf16x2(o_dz[0], o_dz[1]); o.y = pack_bf16x2(o_dz[2], o_dz[3]); o.z = pack_bf16x2(o_dz[4], o_dz[5]); o.w = pack_bf16x2(o_dz[6], o_dz[7]);
    *reinterpret_cast<uint4*>(dz + base) = o;
    o.x = pack_bf16x2(o_dye[0], o_dye[1]); o.y = pack_bf16x2(o_dye[2], o_dye[3]); o.z = pack_bf16x2(o_dye[4], o_dye[5]); o.w = pack_bf16x2(o_dye[6], o_dye[7]);
    *reinterpret_cast<uint4*>(dye + base) = o;
    *reinterpret_cast<float4*>(dx_acc + base) = make_float4(o_dx[0], o_dx[1], o_dx[2], o_dx[3]);
    *reinterpret_cast<float4*>(dx_acc + base + 4) = make_float4(o_dx[4], o_dx[5], o_dx[6], o_dx[7]);
  }
#pragma unroll
  for (int off = LPR / 2; off > 0; off >>= 1) rsum += __shfl_xor_sync(0xffffffffu, rsum, off);
  if (live && (threadIdx.x % LPR) == 0) dcum[crow + t] = rsum;
  dacc = warp_sum(dacc);
  if (lane == 0) red[warp] = dacc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tt = 0.f;
    for (int w = 0; w < 8; ++w) tt += red[w];
    atomicAdd(&dD[h], tt);
  }
}

// [L,L] stage of the backward: per (b,c,g, 32-row block) loop over the heads of the group:
//   Q = dM∘M ; dcum[b,c,h,s] −= Σ_t Q[t,s] ; dG_g[t,s] = Σ_h dM_h[t,s]·exp(cum_h[t] − cum_h[s])·[s ≤ t]
// 8 warps × 4 rows; lane owns column pairs s = 2·lane + 64·j.  L ≤ 512, L % 64 == 0.
template <int MAXJ>
__global__ void __launch_bounds__(256) m3_bwd_q_kernel(const __nv_bfloat16* __restrict__ dM,
                                                        const __nv_bfloat16* __restrict__ Mm,
                                                        const float* __restrict__ cum, float* __restrict__ dcum,
                                                        __nv_bfloat16* __restrict__ dG, int Bn, int nc, int H, int G,
                                                        int L) {
  extern __shared__ float sm[];  // [L] cum of current head, [L] column sums
  float* scum = sm;
  float* scol = sm + L;
  const int hg = H / G;
  const int rblocks = L / 32;
  const long long blk = blockIdx.x;
  const int rb = static_cast<int>(blk % rblocks);
  const long long q = blk / rblocks;
  const int g = static_cast<int>(q % G);
  const int c = static_cast<int>((q / G) % nc);
  const int b = static_cast<int>(q / (static_cast<long long>(G) * nc));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r0 = rb * 32 + warp * 4;
  const int nj = L / 64;
  const int smax = rb * 32 + 32;  // columns ≥ smax are above the diagonal for every row of this block
  float acc[4][MAXJ][2];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int j = 0; j < MAXJ; ++j) acc[r][j][0] = acc[r][j][1] = 0.f;
  for (int hh = 0; hh < hg; ++hh) {
    const int h = g * hg + hh;
    const long long vrow = ((static_cast<long long>(b) * nc + c) * H + h) * L;
    __syncthreads();
    for (int i = threadIdx.x; i < L; i += 256) {
      scum[i] = cum[vrow + i];
      scol[i] = 0.f;
    }
    __syncthreads();
    const long long mbase = vrow * L;  // [b,c,h] matrix base (L×L)
    if (hh + 1 < hg) {  // the loop is latency-bound: ask L2 for the next head's rows of dM and M while this head is processed
      const long long nbase = mbase + static_cast<long long>(L) * L;
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int j = 0; j < MAXJ; ++j) {
          const int s = 2 * lane + 64 * j;
          if (j < nj && s < smax) {
            asm volatile("prefetch.global.L2 [%0];" ::"l"(dM + nbase + static_cast<long long>(r0 + r) * L + s));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(Mm + nbase + static_cast<long long>(r0 + r) * L + s));
          }
        }
    }
    float csum[MAXJ][2];
#pragma unroll
    for (int j = 0; j < MAXJ; ++j) csum[j][0] = csum[j][1] = 0.f;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int t = r0 + r;
      const float ct = scum[t];
#pragma unroll
      for (int j = 0; j < MAXJ; ++j) {
        const int s = 2 * lane + 64 * j;
        if (j < nj && s < smax) {
          const float2 dm = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dM + mbase + static_cast<long long>(t) * L + s));
          const float2 mm = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(Mm + mbase + static_cast<long long>(t) * L + s));
          if (s <= t) {
            csum[j][0] += dm.x * mm.x;
            acc[r][j][0] += dm.x * __expf(ct - scum[s]);
          }
          if (s + 1 <= t) {
            csum[j][1] += dm.y * mm.y;
            acc[r][j][1] += dm.y * __expf(ct - scum[s + 1]);
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < MAXJ; ++j) {
      const int s = 2 * lane + 64 * j;
      if (j < nj && s < smax) {
        atomicAdd(&scol[s], csum[j][0]);
        atomicAdd(&scol[s + 1], csum[j][1]);
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < smax && i < L; i += 256) atomicAdd(&dcum[vrow + i], -scol[i]);
  }
  const long long gbase = (((static_cast<long long>(b) * nc + c) * G + g) * L) * L;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int t = r0 + r;
#pragma unroll
    for (int j = 0; j < MAXJ; ++j) {
      const int s = 2 * lane + 64 * j;
      if (j < nj)
        *reinterpret_cast<__nv_bfloat162*>(dG + gbase + static_cast<long long>(t) * L + s) =
            __floats2bfloat162_rn(acc[r][j][0], acc[r][j][1]);
    }
  }
}

// The same stage for L a multiple of 256 with 16-byte accesses: a lane owns 8 consecutive columns s = 8·lane + 256·j, so a warp
// reads a whole 512-byte row segment per instruction and a thread has 8 wide loads in flight per head instead of 64 narrow ones
// (the narrow form is bound by the number of memory instructions, not by bytes).
template <int MAXJ>
__global__ void __launch_bounds__(256) m3_bwd_q_w8_kernel(const __nv_bfloat16* __restrict__ dM, const __nv_bfloat16* __restrict__ Mm,
                                                           const float* __restrict__ cum, float* __restrict__ dcum,
                                                           __nv_bfloat16* __restrict__ dG, int Bn, int nc, int H, int G, int L) {
  extern __shared__ __align__(16) float sm[];  // [L] cum of current head, [L] column sums
  float* scum = sm;
  float* scol = sm + L;
  const int hg = H / G;
  const int rblocks = L / 32;
  const long long blk = blockIdx.x;
  const int rb = static_cast<int>(blk % rblocks);
  const long long q = blk / rblocks;
  const int g = static_cast<int>(q % G);
  const int c = static_cast<int>((q / G) % nc);
  const int b = static_cast<int>(q / (static_cast<long long>(G) * nc));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r0 = rb * 32 + warp * 4;
  const int nj = L / 256;
  const int smax = rb * 32 + 32;  // columns ≥ smax are above the diagonal for every row of this block
  float acc[4][MAXJ][8];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int j = 0; j < MAXJ; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[r][j][i] = 0.f;
  for (int hh = 0; hh < hg; ++hh) {
    const int h = g * hg + hh;
    const long long vrow = ((static_cast<long long>(b) * nc + c) * H + h) * L;
    __syncthreads();
    for (int i = threadIdx.x; i < L; i += 256) {
      scum[i] = cum[vrow + i];
      scol[i] = 0.f;
    }
    __syncthreads();
    const long long mbase = vrow * L;  // [b,c,h] matrix base (L×L)
    uint4 rd[4][MAXJ], rm[4][MAXJ];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int j = 0; j < MAXJ; ++j) {
        const int s = 8 * lane + 256 * j;
        if (j < nj && s < smax) {
          rd[r][j] = *reinterpret_cast<const uint4*>(dM + mbase + static_cast<long long>(r0 + r) * L + s);
          rm[r][j] = *reinterpret_cast<const uint4*>(Mm + mbase + static_cast<long long>(r0 + r) * L + s);
        }
      }
    if (hh + 1 < hg) {  // ask L2 for the next head's rows while this head is processed
      const long long nbase = mbase + static_cast<long long>(L) * L;
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int j = 0; j < MAXJ; ++j) {
          const int s = 8 * lane + 256 * j;
          if (j < nj && s < smax && (lane & 7) == 0) {       // one request per 128-byte line
            asm volatile("prefetch.global.L2 [%0];" ::"l"(dM + nbase + static_cast<long long>(r0 + r) * L + s));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(Mm + nbase + static_cast<long long>(r0 + r) * L + s));
          }
        }
    }
#pragma unroll
    for (int j = 0; j < MAXJ; ++j) {
      const int s = 8 * lane + 256 * j;
      if (j < nj && s < smax) {
        float cs[8], csum[8];
        *reinterpret_cast<float4*>(cs) = *reinterpret_cast<const float4*>(scum + s);
        *reinterpret_cast<float4*>(cs + 4) = *reinterpret_cast<const float4*>(scum + s + 4);
#pragma unroll
        for (int i = 0; i < 8; ++i) csum[i] = 0.f;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int t = r0 + r;
          const float ct = scum[t];
          float dm[8], mm[8];
          unpack8_bf16(rd[r][j], dm);
          unpack8_bf16(rm[r][j], mm);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            if (s + i <= t) {
              csum[i] += dm[i] * mm[i];
              acc[r][j][i] += dm[i] * __expf(ct - cs[i]);
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) atomicAdd(&scol[s + i], csum[i]);
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < smax && i < L; i += 256) atomicAdd(&dcum[vrow + i], -scol[i]);
  }
  const long long gbase = (((static_cast<long long>(b) * nc + c) * G + g) * L) * L;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int t = r0 + r;
#pragma unroll
    for (int j = 0; j < MAXJ; ++j) {
      const int s = 8 * lane + 256 * j;
      if (j < nj) {
        uint4 o;
        o.x = pack_bf16x2(acc[r][j][0], acc[r][j][1]);
        o.y = pack_bf16x2(acc[r][j][2], acc[r][j][3]);
        o.z = pack_bf16x2(acc[r][j][4], acc[r][j][5]);
        o.w = pack_bf16x2(acc[r][j][6], acc[r][j][7]);
        *reinterpret_cast<uint4*>(dG + gbase + static_cast<long long>(t) * L + s) = o;
      }
    }
  }
}

// The 16-byte form for L = 64 and L = 128: LPR = L/8 lanes cover a row, so one warp-wide load fetches 32/LPR rows of the block's
// 32×L tile and each warp still owns 4 rows.
template <int LPR>
__global__ void __launch_bounds__(256) m3_bwd_q_w8s_kernel(const __nv_bfloat16* __restrict__ dM, const __nv_bfloat16* __restrict__ Mm,
                                                            const float* __restrict__ cum, float* __restrict__ dcum,
                                                            __nv_bfloat16* __restrict__ dG, int Bn, int nc, int H, int G) {
  constexpr int L = LPR * 8, RPL = 32 / LPR, NL = 4 / RPL;
  __shared__ __align__(16) float scum[L];
  __shared__ __align__(16) float spart[8][L];        // per-warp column sums (no atomics: a lane pair owns its columns inside a warp)
  const int hg = H / G;
  constexpr int rblocks = L / 32;
  const long long blk = blockIdx.x;
  const int rb = static_cast<int>(blk % rblocks);
  const long long q = blk / rblocks;
  const int g = static_cast<int>(q % G);
  const int c = static_cast<int>((q / G) % nc);
  const int b = static_cast<int>(q / (static_cast<long long>(G) * nc));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r0 = rb * 32 + warp * 4 + lane / LPR;   // this lane's row of load k is r0 + k·RPL
  const int s = (lane % LPR) * 8;
  const int smax = rb * 32 + 32;
  const bool live = s < smax;
  float acc[NL][8];
#pragma unroll
  for (int k = 0; k < NL; ++k)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[k][i] = 0.f;
  for (int hh = 0; hh < hg; ++hh) {
    const int h = g * hg + hh;
    const long long vrow = ((static_cast<long long>(b) * nc + c) * H + h) * L;
    const long long mbase = vrow * L;
    uint4 rd[NL], rm[NL];
    if (live) {
#pragma unroll
      for (int k = 0; k < NL; ++k) {
        rd[k] = *reinterpret_cast<const uint4*>(dM + mbase + static_cast<long long>(r0 + k * RPL) * L + s);
        rm[k] = *reinterpret_cast<const uint4*>(Mm + mbase + static_cast<long long>(r0 + k * RPL) * L + s);
      }
    }
    __syncthreads();                                  // the previous head's readers of scum / spart are done
    for (int i = threadIdx.x; i < L; i += 256) scum[i] = cum[vrow + i];
    __syncthreads();
    float csum[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) csum[i] = 0.f;
    if (live) {
      float cs[8];
      *reinterpret_cast<float4*>(cs) = *reinterpret_cast<const float4*>(scum + s);
      *reinterpret_cast<float4*>(cs + 4) = *reinterpret_cast<const float4*>(scum + s + 4);
#pragma unroll
      for (int k = 0; k < NL; ++k) {
        const int t = r0 + k * RPL;
        const float ct = scum[t];
        float dm[8], mm[8];
        unpack8_bf16(rd[k], dm);
        unpack8_bf16(rm[k], mm);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (s + i <= t) {
            csum[i] += dm[i] * mm[i];
            acc[k][i] += dm[i] * __expf(ct - cs[i]);
          }
      }
    }
    // the RPL lanes of a warp that share these 8 columns add up, then one of them publishes the warp's sums
#pragma unroll
    for (int off = LPR; off < 32; off <<= 1)
#pragma unroll
      for (int i = 0; i < 8; ++i) csum[i] += __shfl_xor_sync(0xffffffffu, csum[i], off);
    if (lane < LPR) {
      *reinterpret_cast<float4*>(&spart[warp][s]) = make_float4(csum[0], csum[1], csum[2], csum[3]);
      *reinterpret_cast<float4*>(&spart[warp][s + 4]) = make_float4(csum[4], csum[5], csum[6], csum[7]);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < smax && i < L; i += 256) {
      float tsum = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) tsum += spart[w][i];
      atomicAdd(&dcum[vrow + i], -tsum);
    }
  }
  const long long gbase = (((static_cast<long long>(b) * nc + c) * G + g) * L) * L;
#pragma unroll
  for (int k = 0; k < NL; ++k) {
    uint4 o;
    o.x = pack_bf16x2(acc[k][0], acc[k][1]);
    o.y = pack_bf16x2(acc[k][2], acc[k][3]);
    o.z = pack_bf16x2(acc[k][4], acc[k][5]);
    o.w = pack_bf16x2(acc[k][6], acc[k][7]);
    *reinterpret_cast<uint4*>(dG + gbase + static_cast<long long>(r0 + k * RPL) * L + s) = o;
  }
}

// Reverse carry. Block (b·H + h, slice): 256 threads × 4 state entries each, so the P·N entries of one (b,h) are spread over
// several blocks; the per-chunk scalar is combined with one atomic per block (dcumL must be zeroed by the caller).
//   dS[c] = dHtot_{c+1} ; dcumL[b,c,h] += Σ dHtot_{c+1}·H_c·decay_c ; dHtot_c = dHy_c + decay_c·dHtot_{c+1}
constexpr int SB_EPT = 4;
__global__ void __launch_bounds__(256) m3_state_bwd_kernel(const float* __restrict__ dHy,
                                                            const __nv_bfloat16* __restrict__ hc,
                                                            const float* __restrict__ cum,
                                                            const float* __restrict__ dhlast,
                                                            __nv_bfloat16* __restrict__ dS, float* __restrict__ dcumL,
                                                            float* __restrict__ dh0, int Bn, int nc, int H, int PN,
                                                            int L) {
  __shared__ float red[8];
  const int h = blockIdx.x % H;
  const int b = blockIdx.x / H;
  const int e0 = (blockIdx.y * 256 + threadIdx.x) * SB_EPT;
  float carry[SB_EPT];
#pragma unroll
  for (int k = 0; k < SB_EPT; ++k)
    carry[k] = (e0 + k < PN && dhlast != nullptr) ? dhlast[(static_cast<long long>(b) * H + h) * PN + e0 + k] : 0.f;
  for (int c = nc - 1; c >= 0; --c) {
    const long long row = (static_cast<long long>(b) * nc + c) * H + h;
    const float d = __expf(cum[row * L + L - 1]);
    float part = 0.f;
#pragma unroll
    for (int k = 0; k < SB_EPT; ++k) {
      if (e0 + k < PN) {
        const long long idx = row * PN + e0 + k;
        dS[idx] = __float2bfloat16(carry[k]);
        part += carry[k] * __bfloat162float(hc[idx]);
        carry[k] = dHy[idx] + d * carry[k];
      }
    }
    part = warp_sum(part);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = part;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int w = 0; w < 8; ++w) t += red[w];
      atomicAdd(&dcumL[row], t * d);
    }
  }
  if (dh0 != nullptr) {
#pragma unroll
    for (int k = 0; k < SB_EPT; ++k)
      if (e0 + k < PN) dh0[(static_cast<long long>(b) * H + h) * PN + e0 + k] = carry[k];
  }
}

// dXw stage. One warp per (b,s,h):  dx_acc += dXw·w ; dw = Σ_p dXw·x ; dcum[t] −= dw·w ; dcumL += dw·w.
__global__ void __launch_bounds__(256) m3_bwd_xw_kernel(const float* __restrict__ dXw, const __nv_bfloat16* __restrict__ x,
                                                         const float* __restrict__ cum, float* __restrict__ dx_acc,
                                                         float* __restrict__ dcum, float* __restrict__ dcumL, int Bn,
                                                         int S, int H, int P, int L) {
  const int nc = S / L;
  const long long wid = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= static_cast<long long>(Bn) * S * H) return;
  const int h = static_cast<int>(wid % H);
  const long long bs = wid / H;
  const int s = static_cast<int>(bs % S);
  const int b = static_cast<int>(bs / S);
  const int c = s / L, t = s - c * L;
  const long long crow = (static_cast<long long>(b) * nc + c) * H + h;
  const float w = __expf(cum[crow * L + L - 1] - cum[crow * L + t]);
  const long long base = wid * P;
  float dw = 0.f;
  for (int p = 2 * lane; p < P; p += 64) {
    const float2 g = *reinterpret_cast<const float2*>(dXw + base + p);
    const float2 xv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + base + p));
    float2 a = *reinterpret_cast<float2*>(dx_acc + base + p);
    a.x += g.x * w;
    a.y += g.y * w;
    *reinterpret_cast<float2*>(dx_acc + base + p) = a;
    dw += g.x * xv.x + g.y * xv.y;
  }
  dw = warp_sum(dw);
  if (lane == 0) {
    const float v = dw * w;
    atomicAdd(&dcum[crow * L + t], -v);
    atomicAdd(&dcumL[crow], v);
  }
}

// 16-byte form: a thread owns 8 channels, P/8 lanes share a (b,s,h) row and a block covers 256·8/P consecutive tokens of one head
// and one chunk (the row count divides L), so dcumL takes one atomic per block instead of one per token.
template <int LPR>
__global__ void __launch_bounds__(256) m3_bwd_xw_w8_kernel(const float* __restrict__ dXw, const __nv_bfloat16* __restrict__ x,
                                                            const float* __restrict__ cum, float* __restrict__ dx_acc,
                                                            float* __restrict__ dcum, float* __restrict__ dcumL, int Bn, int S, int H,
                                                            int L, __nv_bfloat16* __restrict__ gx) {
  constexpr int P = LPR * 8, ROWS = 256 / LPR;
  __shared__ float red[8];
  const int nc = S / L;
  const long long blk = blockIdx.x;
  const int h = static_cast<int>(blk % H);
  const long long q = blk / H;
  const int sblocks = S / ROWS;                  // S % L == 0 and L % ROWS == 0
  const int sb = static_cast<int>(q % sblocks);
  const int b = static_cast<int>(q / sblocks);
  const int s = sb * ROWS + threadIdx.x / LPR;
  const int p = (threadIdx.x % LPR) * 8;
  const int c = s / L, t = s - c * L;
  const long long crow = (static_cast<long long>(b) * nc + c) * H + h;
  const float w = __expf(cum[crow * L + L - 1] - cum[crow * L + t]);
  const long long base = ((static_cast<long long>(b) * S + s) * H + h) * P + p;
  const float4 g0 = *reinterpret_cast<const float4*>(dXw + base), g1 = *reinterpret_cast<const float4*>(dXw + base + 4);
  float4 a0 = *reinterpret_cast<const float4*>(dx_acc + base), a1 = *reinterpret_cast<const float4*>(dx_acc + base + 4);
  float xv[8];
  unpack8_bf16(*reinterpret_cast<const uint4*>(x + base), xv);
  a0.x += g0.x * w; a0.y += g0.y * w; a0.z += g0.z * w; a0.w += g0.w * w;
  a1.x += g1.x * w; a1.y += g1.y * w; a1.z += g1.z * w; a1.w += g1.w * w;
  if (gx != nullptr) {               // this is the last contribution to dx: emit the bf16 gradient instead of the fp32 accumulator
    uint4 o;
    o.x = pack_bf16x2(a0.x, a0.y); o.y = pack_bf16x2(a0.z, a0.w); o.z = pack_bf16x2(a1.x, a1.y); o.w = pack_bf16x2(a1.z, a1.w);
    *reinterpret_cast<uint4*>(gx + base) = o;
  } else {
    *reinterpret_cast<float4*>(dx_acc + base) = a0;
    *reinterpret_cast<float4*>(dx_acc + base + 4) = a1;
  }
  float dw = g0.x * xv[0] + g0.y * xv[1] + g0.z * xv[2] + g0.w * xv[3] + g1.x * xv[4] + g1.y * xv[5] + g1.z * xv[6] + g1.w * xv[7];
#pragma unroll
  for (int off = LPR / 2; off > 0; off >>= 1) dw += __shfl_xor_sync(0xffffffffu, dw, off);
  float v = 0.f;
  if ((threadIdx.x % LPR) == 0) {
    v = dw * w;
    atomicAdd(&dcum[crow * L + t], -v);
  }
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tt = 0.f;
    for (int k = 0; k < 8; ++k) tt += red[k];
    atomicAdd(&dcumL[crow], tt);
  }
}

// Final: dcum[L−1] += dcumL ; dla = reverse-cumsum(dcum) ; dA = dla·dt ; ddt = dla·A.  One warp per (b,c,h).
__global__ void m3_bwd_final_kernel(const float* __restrict__ dcum, const float* __restrict__ dcumL,
                                    const float* __restrict__ A, const float* __restrict__ dt, float* __restrict__ dA,
                                    float* __restrict__ ddt, int Bn, int S, int H, int L) {
  const int nc = S / L;
  const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= static_cast<long long>(Bn) * nc * H) return;
  const int h = static_cast<int>(row % H);
  const int c = static_cast<int>((row / H) % nc);
  const int b = static_cast<int>(row / (static_cast<long long>(H) * nc));
  const int per = L / 32;
  const float* in = dcum + row * L;
  float vals[32];
  float run = 0.f;
  // lane owns t in [lane·per, lane·per+per); build suffix sums inside the lane from the right
  for (int i = per - 1; i >= 0; --i) {
    const int t = lane * per + i;
    float v = in[t];
    if (t == L - 1) v += dcumL[row];
    run += v;
    vals[i] = run;
  }
  float tot = run;  // inclusive suffix over lanes to the right
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float n = __shfl_down_sync(0xffffffffu, tot, o);
    if (lane + o < 32) tot += n;
  }
  const float off = tot - run;
  const long long base = (static_cast<long long>(b) * S + static_cast<long long>(c) * L) * H + h;
  for (int i = 0; i < per; ++i) {
    const int t = lane * per + i;
    const long long idx = base + static_cast<long long>(t) * H;
    const float dla = vals[i] + off;
    dA[idx] = dla * dt[idx];
    ddt[idx] = dla * A[idx];
  }
}

// fp32 → bf16 cast with optional accumulate-free copy (used for dx, dB, dC).
__global__ void m3_cast_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, long long n2) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n2;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float2 v = reinterpret_cast<const float2*>(in)[i];
    reinterpret_cast<__nv_bfloat162*>(out)[i] = __floats2bfloat162_rn(v.x, v.y);
  }
}

static inline int grid1d(long long n, int per_block) {
  long long b = (n + per_block - 1) / per_block;
  const long long cap = 148LL * 32;
  return static_cast<int>(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace cmb

#define CMB_OK() (cudaGetLastError() == cudaSuccess ? 0 : 2)

extern "C" int cmb_m3_cumsum(const float* A, const float* dt, float* cum, int Bn, int S, int H, int L, void* stream) {
  if (L % 32 || L > 1024 || S % L) return 1;
  const long long rows = static_cast<long long>(Bn) * (S / L) * H;
  cmb::m3_cumsum_kernel<<<static_cast<int>((rows * 32 + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(A, dt, cum, Bn, S, H, L);
  return CMB_OK();
}
extern "C" int cmb_m3_xw(const void* x, const float* cum, void* xw, int Bn, int S, int H, int P, int L, void* stream) {
  if (P % 2) return 1;
  if (P % 8 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(xw)) & 15) == 0) {
    const long long n8 = static_cast<long long>(Bn) * S * H * (P / 8);
    cmb::m3_xw_w8_kernel<<<cmb::grid1d(n8, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(x), cum, static_cast<__nv_bfloat16*>(xw), Bn, S, H, P, L);
    return CMB_OK();
  }
  const long long n2 = static_cast<long long>(Bn) * S * H * (P / 2);
  cmb::m3_xw_kernel<<<cmb::grid1d(n2, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), cum, static_cast<__nv_bfloat16*>(xw), Bn, S, H, P, L);
  return CMB_OK();
}
extern "C" int cmb_m3_state_pass(const float* sloc, const float* cum, const float* h0, void* hc, float* hlast, int Bn,
                                 int nc, int H, int PN, int L, void* stream) {
  const long long n = static_cast<long long>(Bn) * H * PN;
  if (PN % 4 == 0 && ((reinterpret_cast<uintptr_t>(sloc) | reinterpret_cast<uintptr_t>(h0) | reinterpret_cast<uintptr_t>(hlast)) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(hc) & 7) == 0) {
    cmb::m3_state_pass_w4_kernel<<<cmb::grid1d(n / 4, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        sloc, cum, h0, static_cast<__nv_bfloat16*>(hc), hlast, Bn, nc, H, PN, L);
    return CMB_OK();
  }
  cmb::m3_state_pass_kernel<<<cmb::grid1d(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      sloc, cum, h0, static_cast<__nv_bfloat16*>(hc), hlast, Bn, nc, H, PN, L);
  return CMB_OK();
}
extern "C" int cmb_m3_finalize_fwd(const float* Y, const void* x, const void* z, const float* D, void* ypre, void* out,
                                   int Bn, int S, int H, int P, long long zs_b, long long zs_s, long long zs_h,
                                   void* stream) {
  if (P % 2) return 1;
  auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (P % 8 == 0 && zs_b % 8 == 0 && zs_s % 8 == 0 && zs_h % 8 == 0 && al16(Y) && al16(x) && al16(z) && al16(ypre) && al16(out)) {
    const long long n8 = static_cast<long long>(Bn) * S * H * (P / 8);
    cmb::m3_finalize_fwd_w8_kernel<<<cmb::grid1d(n8, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        Y, static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(z), D, static_cast<__nv_bfloat16*>(ypre),
        static_cast<__nv_bfloat16*>(out), Bn, S, H, P, zs_b, zs_s, zs_h);
    return CMB_OK();
  }
  const long long n2 = static_cast<long long>(Bn) * S * H * (P / 2);
  cmb::m3_finalize_fwd_kernel<<<cmb::grid1d(n2, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      Y, static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(z), D, static_cast<__nv_bfloat16*>(ypre),
      static_cast<__nv_bfloat16*>(out), Bn, S, H, P, zs_b, zs_s, zs_h);
  return CMB_OK();
}
extern "C" int cmb_m3_expand_decay(const float* CB, const float* cum, void* M, int Bn, int nc, int H, int G, int L, void* stream) {
  if (L % 8 || H % G) return 1;
  const long long n8 = static_cast<long long>(Bn) * nc * H * L * (L / 8);
  cmb::m3_expand_decay_kernel<<<cmb::grid1d(n8, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(CB, cum, static_cast<__nv_bfloat16*>(M), Bn, nc, H,
                                                                                                 G, L);
  return CMB_OK();
}
extern "C" int cmb_m3_bwd_pre(const void* dout, const void* z, const void* ypre, const void* x, const float* D,
                              const float* cum, void* dy, void* dz, void* dye, float* dx_acc, float* dcum, float* dD,
                              int Bn, int S, int H, int P, int L, long long zs_b, long long zs_s, long long zs_h,
                              void* stream) {
  if (P % 2) return 1;
  using bf = __nv_bfloat16;
  auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if ((P == 32 || P == 64 || P == 128 || P == 256) && zs_b % 8 == 0 && zs_s % 8 == 0 && zs_h % 8 == 0 && al16(dout) && al16(z) && al16(ypre) &&
      al16(x) && al16(dy) && al16(dz) && al16(dye) && al16(dx_acc)) {
    const int rows = 256 * 8 / P;
    const long long wblocks = static_cast<long long>(Bn) * ((S + rows - 1) / rows) * H;
    if (wblocks > 0x7fffffffLL) return 3;
    auto kern = P == 32 ? cmb::m3_bwd_pre_w8_kernel<4> : P == 64 ? cmb::m3_bwd_pre_w8_kernel<8> : P == 128 ? cmb::m3_bwd_pre_w8_kernel<16>
                                                                                                          : cmb::m3_bwd_pre_w8_kernel<32>;
    kern<<<static_cast<int>(wblocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const bf*>(dout), static_cast<const bf*>(z), static_cast<const bf*>(ypre), static_cast<const bf*>(x), D, cum,
        static_cast<bf*>(dy), static_cast<bf*>(dz), static_cast<bf*>(dye), dx_acc, dcum, dD, Bn, S, H, L, zs_b, zs_s, zs_h);
    return CMB_OK();
  }
  const long long blocks = static_cast<long long>(Bn) * ((S + 7) / 8) * H;
  if (blocks > 0x7fffffffLL) return 3;
  cmb::m3_bwd_pre_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const bf*>(dout), static_cast<const bf*>(z), static_cast<const bf*>(ypre), static_cast<const bf*>(x), D,
      cum, static_cast<bf*>(dy), static_cast<bf*>(dz), static_cast<bf*>(dye), dx_acc, dcum, dD, Bn, S, H, P, L, zs_b, zs_s,
      zs_h);
  return CMB_OK();
}
extern "C" int cmb_m3_bwd_q(const void* dM, const void* Mm, const float* cum, float* dcum, void* dG, int Bn, int nc, int H,
                            int G, int L, void* stream) {
  if (L % 64 || L > 512 || H % G) return 1;
  const long long blocks = static_cast<long long>(Bn) * nc * G * (L / 32);
  if (blocks > 0x7fffffffLL) return 3;
  using bf = __nv_bfloat16;
  if (L % 256 == 0 && ((reinterpret_cast<uintptr_t>(dM) | reinterpret_cast<uintptr_t>(Mm) | reinterpret_cast<uintptr_t>(dG)) & 15) == 0) {
    auto kern = L == 256 ? cmb::m3_bwd_q_w8_kernel<1> : cmb::m3_bwd_q_w8_kernel<2>;
    kern<<<static_cast<int>(blocks), 256, 2 * L * sizeof(float), static_cast<cudaStream_t>(stream)>>>(
        static_cast<const bf*>(dM), static_cast<const bf*>(Mm), cum, dcum, static_cast<bf*>(dG), Bn, nc, H, G, L);
    return CMB_OK();
  }
  if ((L == 64 || L == 128) && ((reinterpret_cast<uintptr_t>(dM) | reinterpret_cast<uintptr_t>(Mm) | reinterpret_cast<uintptr_t>(dG)) & 15) == 0) {
    auto kern = L == 64 ? cmb::m3_bwd_q_w8s_kernel<8> : cmb::m3_bwd_q_w8s_kernel<16>;
    kern<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const bf*>(dM), static_cast<const bf*>(Mm), cum, dcum,
                                                                                  static_cast<bf*>(dG), Bn, nc, H, G);
    return CMB_OK();
  }
  cmb::m3_bwd_q_kernel<8><<<static_cast<int>(blocks), 256, 2 * L * sizeof(float), static_cast<cudaStream_t>(stream)>>>(
      static_cast<const bf*>(dM), static_cast<const bf*>(Mm), cum, dcum, static_cast<bf*>(dG), Bn, nc, H, G, L);
  return CMB_OK();
}
extern "C" int cmb_m3_state_bwd(const float* dHy, const void* hc, const float* cum, const float* dhlast, void* dS,
                                float* dcumL, float* dh0, int Bn, int nc, int H, int PN, int L, void* stream) {
  using bf = __nv_bfloat16;
  const dim3 grid(Bn * H, (PN + 256 * cmb::SB_EPT - 1) / (256 * cmb::SB_EPT));
  cmb::m3_state_bwd_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      dHy, static_cast<const bf*>(hc), cum, dhlast, static_cast<bf*>(dS), dcumL, dh0, Bn, nc, H, PN, L);
  return CMB_OK();
}
// `gx` (optional, bf16 [B,S,H,P]): when given and the wide kernel applies, the finished gradient is written there in bf16 and dx_acc is
// left as it was; the return value 10 says so (0: dx_acc was updated and still has to be cast by the caller).
extern "C" int cmb_m3_bwd_xw(const float* dXw, const void* x, const float* cum, float* dx_acc, float* dcum, float* dcumL,
                             int Bn, int S, int H, int P, int L, void* gx, void* stream) {
  {
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    const int rows = (P == 32 || P == 64 || P == 128 || P == 256) ? 256 * 8 / P : 0;
    if (rows > 0 && L % rows == 0 && S % L == 0 && al16(dXw) && al16(x) && al16(dx_acc)) {
      const long long wblocks = static_cast<long long>(Bn) * (S / rows) * H;
      if (wblocks > 0x7fffffffLL) return 3;
      auto kern = P == 32 ? cmb::m3_bwd_xw_w8_kernel<4> : P == 64 ? cmb::m3_bwd_xw_w8_kernel<8> : P == 128 ? cmb::m3_bwd_xw_w8_kernel<16>
                                                                                                          : cmb::m3_bwd_xw_w8_kernel<32>;
      const bool fused = gx != nullptr && (reinterpret_cast<uintptr_t>(gx) & 15) == 0;
      kern<<<static_cast<int>(wblocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(dXw, static_cast<const __nv_bfloat16*>(x), cum, dx_acc, dcum,
                                                                                    dcumL, Bn, S, H, L,
                                                                                    fused ? static_cast<__nv_bfloat16*>(gx) : nullptr);
      if (cudaGetLastError() != cudaSuccess) return 2;
      return fused ? 10 : 0;
    }
  }
  const long long warps = static_cast<long long>(Bn) * S * H;
  cmb::m3_bwd_xw_kernel<<<static_cast<int>((warps * 32 + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      dXw, static_cast<const __nv_bfloat16*>(x), cum, dx_acc, dcum, dcumL, Bn, S, H, P, L);
  return CMB_OK();
}
extern "C" int cmb_m3_bwd_final(const float* dcum, const float* dcumL, const float* A, const float* dt, float* dA,
                                float* ddt, int Bn, int S, int H, int L, void* stream) {
  if (L % 32 || L > 1024) return 1;
  const long long rows = static_cast<long long>(Bn) * (S / L) * H;
  cmb::m3_bwd_final_kernel<<<static_cast<int>((rows * 32 + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      dcum, dcumL, A, dt, dA, ddt, Bn, S, H, L);
  return CMB_OK();
}
extern "C" int cmb_cast_f32_bf16(const float* in, void* out, long long n, void* stream) {
  if (n % 2) return 1;
  cmb::m3_cast_bf16_kernel<<<cmb::grid1d(n / 2, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      in, static_cast<__nv_bfloat16*>(out), n / 2);
  return CMB_OK();
}
