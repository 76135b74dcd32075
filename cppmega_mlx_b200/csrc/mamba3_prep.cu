// Mamba3 input preparation between the causal conv and the scan, forward and backward, as four small fused kernels
// (replaces ~150 element-wise framework launches per layer).  Single-rank B/C (no MIMO averaging).
//
//   per token t, head h (H heads, G groups, hg = H/G heads per group):
//     dt[h]   = softplus(dd_dt[h] + dt_bias[h])                A[h] = min(−softplus(dd_A[h]), −A_floor)
//     sc[h]   = dt_{t+1}[h]·(1 − σ(trap_{t+1}[h])) + dt_t[h]·σ(trap_t[h])      (the term of a missing successor is 0)
//     scale[g]= mean_{h in g} sc[h]                           inc[g,i] = angle[i] · dt[g]      (head index g < G, i < R)
//   cumulative phases ang = cumsum_t(inc) are formed between the kernels (a framework prefix sum over a small tensor), then
//   per token, group g, state index n (N = d_state):
//     B̂ = rmsnorm_N(B_raw)·wB + bB ;  Bg = rot(B̂ · scale[g], ang[g])        Ĉ = rmsnorm_N(C_raw)·wC + bC ;  Cg = rot(Ĉ, ang[g])
//   rot turns the interleaved pairs (2i, 2i+1), i < R, by ang[g,i]; the remaining columns pass through.
//
// Math parity: cppmega_mlx/nn/mamba3.py:227-310 (B/C norm + bias, trapezoid scale :238, phase accumulation and rotation :270).
#include "sm100.cuh"

namespace cmb {

__device__ __forceinline__ float softplusf(float x) { return x > 20.f ? x : log1pf(__expf(x)); }
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// tail row layout: [dd_dt (H) | dd_A (H) | trap (H) | angles (R)], bf16, row pitch ld_tail.
// One thread per (token, head).
__global__ void __launch_bounds__(256) m3_prep_dt_fwd_kernel(const __nv_bfloat16* __restrict__ tail, long long ld_tail,
                                                              const float* __restrict__ dt_bias, float* __restrict__ dt,
                                                              float* __restrict__ A, float* __restrict__ sc, float* __restrict__ inc,
                                                              int Bn, int S, int H, int G, int R, float a_floor) {
  const long long idx = blockIdx.x * 256LL + threadIdx.x;
  const long long total = static_cast<long long>(Bn) * S * H;
  if (idx >= total) return;
  const int h = static_cast<int>(idx % H);
  const long long tok = idx / H;
  const int s = static_cast<int>(tok % S);
  const __nv_bfloat16* row = tail + tok * ld_tail;
  const float bias = dt_bias[h];
  const float d = softplusf(__bfloat162float(row[h]) + bias);
  dt[idx] = d;
  A[idx] = fminf(-softplusf(__bfloat162float(row[H + h])), -a_floor);
  float v = d * sigmoidf_(__bfloat162float(row[2 * H + h]));
  if (s + 1 < S) {
    const __nv_bfloat16* nxt = row + ld_tail;
    v += softplusf(__bfloat162float(nxt[h]) + bias) * (1.f - sigmoidf_(__bfloat162float(nxt[2 * H + h])));
  }
  sc[idx] = v;
  if (h < G) {
    float* o = inc + (tok * G + h) * R;
    for (int i = 0; i < R; ++i) o[i] = __bfloat162float(row[3 * H + i]) * d;
  }
}

// One thread per (token, head). g_dt / g_A: gradients arriving from the scan; g_sc: gradient of sc (= g_scale[g]/hg, expanded by
// the caller); g_inc [B,S,G,R]. Writes the gradient of the whole tail row (bf16) and accumulates d dt_bias.
__global__ void __launch_bounds__(256) m3_prep_dt_bwd_kernel(const __nv_bfloat16* __restrict__ tail, long long ld_tail,
                                                              const float* __restrict__ dt_bias, const float* __restrict__ dt,
                                                              const float* __restrict__ g_dt, const float* __restrict__ g_A,
                                                              const float* __restrict__ g_scale, const float* __restrict__ g_inc,
                                                              __nv_bfloat16* __restrict__ g_tail, float* __restrict__ g_bias, int Bn, int S,
                                                              int H, int G, int R, float a_floor) {
  const long long idx = blockIdx.x * 256LL + threadIdx.x;
  const long long total = static_cast<long long>(Bn) * S * H;
  float gb = 0.f;
  int h = 0;
  if (idx < total) {
    h = static_cast<int>(idx % H);
    const long long tok = idx / H;
    const int s = static_cast<int>(tok % S);
    const int hg = H / G, g = h / hg;
    const __nv_bfloat16* row = tail + tok * ld_tail;
    const float pre = __bfloat162float(row[h]) + dt_bias[h];
    const float d = dt[idx];
    const float tr = __bfloat162float(row[2 * H + h]);
    const float sg = sigmoidf_(tr);
    const float gs_here = g_scale[tok * G + g] / hg;                        // d loss / d sc[t,h]
    const float gs_prev = s > 0 ? g_scale[(tok - 1) * G + g] / hg : 0.f;    // d loss / d sc[t−1,h]
    float gd = g_dt[idx] + gs_here * sg + gs_prev * (1.f - sg);
    if (h < G) {
      const float* gi = g_inc + (tok * G + h) * R;
      for (int i = 0; i < R; ++i) gd += gi[i] * __bfloat162float(row[3 * H + i]);
    }
    const float g_pre = gd * sigmoidf_(pre);                                  // softplus'
    const float g_trap = (gs_here - gs_prev) * d * sg * (1.f - sg);
    const float a_in = __bfloat162float(row[H + h]);
    const float g_a = (softplusf(a_in) > a_floor) ? -g_A[idx] * sigmoidf_(a_in) : 0.f;
    __nv_bfloat16* out = g_tail + tok * (3LL * H + R);
    out[h] = __float2bfloat16(g_pre);
    out[H + h] = __float2bfloat16(g_a);
    out[2 * H + h] = __float2bfloat16(g_trap);
    gb = g_pre;
    if (h < R) {   // the first R threads of a token also produce d angle[i]  (needs R ≤ H)
      float ga = 0.f;
      for (int gg = 0; gg < G; ++gg) ga += g_inc[(tok * G + gg) * R + h] * dt[tok * H + gg];
      out[3 * H + h] = __float2bfloat16(ga);
    }
  }
  // d dt_bias[h]: threads of a block cover consecutive (token, head) pairs; reduce per head through shared memory
  __shared__ float red[256];
  red[threadIdx.x] = gb;
  __syncthreads();
  if (threadIdx.x < H && H <= 256 && 256 % H == 0) {
    // blockDim (256) is a multiple of H: thread j < H sums the entries with the same head
    const int head = static_cast<int>((blockIdx.x * 256LL + threadIdx.x) % H);
    float t = 0.f;
    for (int j = threadIdx.x; j < 256; j += H) t += red[j];
    atomicAdd(&g_bias[head], t);
  } else if (!(H <= 256 && 256 % H == 0) && idx < total) {
    atomicAdd(&g_bias[h], gb);
  }
}

// One warp per (token, group); N ≤ 256, N % 64 == 0 (lane owns the pairs 2·lane + 64·j).
template <int NJ>
__global__ void __launch_bounds__(256) m3_prep_bc_fwd_kernel(const __nv_bfloat16* __restrict__ BC, const float* __restrict__ sc,
                                                              const float* __restrict__ ang, const __nv_bfloat16* __restrict__ wB,
                                                              const __nv_bfloat16* __restrict__ bB, const __nv_bfloat16* __restrict__ wC,
                                                              const __nv_bfloat16* __restrict__ bC, __nv_bfloat16* __restrict__ Bg,
                                                              __nv_bfloat16* __restrict__ Cg, float* __restrict__ rstd, float* __restrict__ scale_g,
                                                              long long rows, int H, int G, int N, int R, float eps) {
  const int lane = threadIdx.x & 31;
  const long long w = (blockIdx.x * 256LL + threadIdx.x) >> 5;     // (token, group)
  if (w >= rows) return;
  const int g = static_cast<int>(w % G);
  const long long tok = w / G;
  const int hg = H / G;
  float s = 0.f;
  for (int j = lane; j < hg; j += 32) s += sc[tok * H + g * hg + j];
  s = warp_sum(s) / hg;
  if (lane == 0) scale_g[w] = s;
  const __nv_bfloat16* braw = BC + tok * (2LL * G * N) + g * N;
  const __nv_bfloat16* craw = braw + G * N;
  float2 xb[NJ], xc[NJ];
  float ssb = 0.f, ssc = 0.f;
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    const int n = 2 * lane + 64 * j;
    xb[j] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(braw + n));
    xc[j] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(craw + n));
    ssb += xb[j].x * xb[j].x + xb[j].y * xb[j].y;
    ssc += xc[j].x * xc[j].x + xc[j].y * xc[j].y;
  }
  const float rb = rsqrtf(warp_sum(ssb) / N + eps), rc = rsqrtf(warp_sum(ssc) / N + eps);
  if (lane == 0) {
    rstd[2 * w] = rb;
    rstd[2 * w + 1] = rc;
  }
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    const int n = 2 * lane + 64 * j;
    const float2 wb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(wB + g * N + n));
    const float2 bb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(bB + g * N + n));
    const float2 wc = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(wC + g * N + n));
    const float2 bc = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(bC + g * N + n));
    float b0 = (xb[j].x * rb * wb.x + bb.x) * s, b1 = (xb[j].y * rb * wb.y + bb.y) * s;
    float c0 = xc[j].x * rc * wc.x + bc.x, c1 = xc[j].y * rc * wc.y + bc.y;
    const int i = n >> 1;
    if (i < R) {
      float sn, cs;
      __sincosf(ang[w * R + i], &sn, &cs);
      const float t0 = b0 * cs - b1 * sn, t1 = b0 * sn + b1 * cs;
      b0 = t0; b1 = t1;
      const float u0 = c0 * cs - c1 * sn, u1 = c0 * sn + c1 * cs;
      c0 = u0; c1 = u1;
    }
    *reinterpret_cast<__nv_bfloat162*>(Bg + w * N + n) = __floats2bfloat162_rn(b0, b1);
    *reinterpret_cast<__nv_bfloat162*>(Cg + w * N + n) = __floats2bfloat162_rn(c0, c1);
  }
}

// Backward of the above. Each warp walks `tokens_per_warp` tokens of one group so that the weight / bias gradients are
// accumulated in registers and flushed with one atomic per element per warp.
template <int NJ>
__global__ void __launch_bounds__(256) m3_prep_bc_bwd_kernel(const __nv_bfloat16* __restrict__ BC, const float* __restrict__ scale_g,
                                                              const float* __restrict__ ang, const float* __restrict__ rstd,
                                                              const __nv_bfloat16* __restrict__ wB, const __nv_bfloat16* __restrict__ bB,
                                                              const __nv_bfloat16* __restrict__ wC, const __nv_bfloat16* __restrict__ bC,
                                                              const __nv_bfloat16* __restrict__ gBg, const __nv_bfloat16* __restrict__ gCg,
                                                              __nv_bfloat16* __restrict__ gBC, float* __restrict__ g_scale, float* __restrict__ g_ang,
                                                              float* __restrict__ gwB, float* __restrict__ gbB, float* __restrict__ gwC,
                                                              float* __restrict__ gbC, long long tokens, int G, int N, int R, int tokens_per_warp) {
  const int lane = threadIdx.x & 31;
  const long long wid = (blockIdx.x * 256LL + threadIdx.x) >> 5;
  const int g = static_cast<int>(wid % G);
  const long long t0 = (wid / G) * tokens_per_warp;
  if (t0 >= tokens) return;
  float2 wb[NJ], bb[NJ], wc[NJ], bc[NJ], awb[NJ], abb[NJ], awc[NJ], abc[NJ];
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    const int n = 2 * lane + 64 * j;
    wb[j] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(wB + g * N + n));
    bb[j] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(bB + g * N + n));
    wc[j] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(wC + g * N + n));
    bc[j] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(bC + g * N + n));
    awb[j] = abb[j] = awc[j] = abc[j] = make_float2(0.f, 0.f);
  }
  const long long t1 = min(tokens, t0 + tokens_per_warp);
  for (long long tok = t0; tok < t1; ++tok) {
    const long long w = tok * G + g;
    const float s = scale_g[w], rb = rstd[2 * w], rc = rstd[2 * w + 1];
    const __nv_bfloat16* braw = BC + tok * (2LL * G * N) + g * N;
    const __nv_bfloat16* craw = braw + G * N;
    float2 xb[NJ], xc[NJ], db[NJ], dc[NJ];     // x̂ (normalised input) and the gradient wrt B̂ / Ĉ (after undoing rot / scale)
    float gs = 0.f, mb = 0.f, mc = 0.f;
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      const int n = 2 * lane + 64 * j;
      float2 gb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gBg + w * N + n));
      float2 gc = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gCg + w * N + n));
      xb[j] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(braw + n));
      xc[j] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(craw + n));
      xb[j].x *= rb; xb[j].y *= rb; xc[j].x *= rc; xc[j].y *= rc;
      const float nb0 = xb[j].x * wb[j].x + bb[j].x, nb1 = xb[j].y * wb[j].y + bb[j].y;    // B̂
      const float nc0 = xc[j].x * wc[j].x + bc[j].x, nc1 = xc[j].y * wc[j].y + bc[j].y;    // Ĉ
      const int i = n >> 1;
      if (i < R) {
        float sn, cs;
        __sincosf(ang[w * R + i], &sn, &cs);
        // outputs o = rot(v): d/dθ = −g0·o1 + g1·o0 ; gradient wrt v = rotᵀ g
        const float vb0 = nb0 * s, vb1 = nb1 * s;
        const float ob0 = vb0 * cs - vb1 * sn, ob1 = vb0 * sn + vb1 * cs;
        const float oc0 = nc0 * cs - nc1 * sn, oc1 = nc0 * sn + nc1 * cs;
        g_ang[w * R + i] = -gb.x * ob1 + gb.y * ob0 - gc.x * oc1 + gc.y * oc0;
        const float tb0 = gb.x * cs + gb.y * sn, tb1 = -gb.x * sn + gb.y * cs;
        const float tc0 = gc.x * cs + gc.y * sn, tc1 = -gc.x * sn + gc.y * cs;
        gb = make_float2(tb0, tb1);
        gc = make_float2(tc0, tc1);
      }
      gs += gb.x * nb0 + gb.y * nb1;
      db[j] = make_float2(gb.x * s, gb.y * s);
      dc[j] = gc;
      awb[j].x += db[j].x * xb[j].x; awb[j].y += db[j].y * xb[j].y; abb[j].x += db[j].x; abb[j].y += db[j].y;
      awc[j].x += dc[j].x * xc[j].x; awc[j].y += dc[j].y * xc[j].y; abc[j].x += dc[j].x; abc[j].y += dc[j].y;
      db[j].x *= wb[j].x; db[j].y *= wb[j].y; dc[j].x *= wc[j].x; dc[j].y *= wc[j].y;       // gradient wrt x̂
      mb += db[j].x * xb[j].x + db[j].y * xb[j].y;
      mc += dc[j].x * xc[j].x + dc[j].y * xc[j].y;
    }
    gs = warp_sum(gs);
    mb = warp_sum(mb) / N;
    mc = warp_sum(mc) / N;
    if (lane == 0) g_scale[w] = gs;
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      const int n = 2 * lane + 64 * j;
      __nv_bfloat16* ob = gBC + tok * (2LL * G * N) + g * N + n;
      *reinterpret_cast<__nv_bfloat162*>(ob) = __floats2bfloat162_rn(rb * (db[j].x - xb[j].x * mb), rb * (db[j].y - xb[j].y * mb));
      *reinterpret_cast<__nv_bfloat162*>(ob + G * N) = __floats2bfloat162_rn(rc * (dc[j].x - xc[j].x * mc), rc * (dc[j].y - xc[j].y * mc));
    }
  }
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    const int n = g * N + 2 * lane + 64 * j;
    atomicAdd(&gwB[n], awb[j].x); atomicAdd(&gwB[n + 1], awb[j].y); atomicAdd(&gbB[n], abb[j].x); atomicAdd(&gbB[n + 1], abb[j].y);
    atomicAdd(&gwC[n], awc[j].x); atomicAdd(&gwC[n + 1], awc[j].y); atomicAdd(&gbC[n], abc[j].x); atomicAdd(&gbC[n + 1], abc[j].y);
  }
}

}  // namespace cmb

using bf16 = __nv_bfloat16;

extern "C" int cmb_m3_prep_dt_fwd(const void* tail, long long ld_tail, const float* dt_bias, float* dt, float* A, float* sc, float* inc, int Bn,
                                  int S, int H, int G, int R, float a_floor, void* stream) {
  const long long total = static_cast<long long>(Bn) * S * H;
  if (total <= 0) return 0;
  if (H % G) return 1;
  cmb::m3_prep_dt_fwd_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const bf16*>(tail), ld_tail, dt_bias, dt, A, sc, inc, Bn, S, H, G, R, a_floor);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

extern "C" int cmb_m3_prep_dt_bwd(const void* tail, long long ld_tail, const float* dt_bias, const float* dt, const float* g_dt, const float* g_A,
                                  const float* g_scale, const float* g_inc, void* g_tail, float* g_bias, int Bn, int S, int H, int G, int R,
                                  float a_floor, void* stream) {
  const long long total = static_cast<long long>(Bn) * S * H;
  if (total <= 0) return 0;
  if (H % G || R > H) return 1;
  cmb::m3_prep_dt_bwd_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const bf16*>(tail), ld_tail, dt_bias, dt, g_dt, g_A, g_scale, g_inc, static_cast<bf16*>(g_tail), g_bias, Bn, S, H, G, R, a_floor);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

extern "C" int cmb_m3_prep_bc_fwd(const void* BC, const float* sc, const float* ang, const void* wB, const void* bB, const void* wC, const void* bC,
                                  void* Bg, void* Cg, float* rstd, float* scale_g, long long tokens, int H, int G, int N, int R, float eps,
                                  void* stream) {
  const long long rows = tokens * G;
  if (rows <= 0) return 0;
  if (N % 64 || N > 256 || H % G || 2 * R > N) return 1;
  const unsigned grid = static_cast<unsigned>((rows * 32 + 255) / 256);
  auto st = static_cast<cudaStream_t>(stream);
#define CMB_PREP_FWD(NJ_)                                                                                                          \
  cmb::m3_prep_bc_fwd_kernel<NJ_><<<grid, 256, 0, st>>>(static_cast<const bf16*>(BC), sc, ang, static_cast<const bf16*>(wB),       \
                                                         static_cast<const bf16*>(bB), static_cast<const bf16*>(wC),               \
                                                         static_cast<const bf16*>(bC), static_cast<bf16*>(Bg), static_cast<bf16*>(Cg), \
                                                         rstd, scale_g, rows, H, G, N, R, eps)
  switch (N / 64) {
    case 1: CMB_PREP_FWD(1); break;
    case 2: CMB_PREP_FWD(2); break;
    case 3: CMB_PREP_FWD(3); break;
    default: CMB_PREP_FWD(4); break;
  }
#undef CMB_PREP_FWD
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// gwB / gbB / gwC / gbC: fp32 [G, N], zeroed by the caller.
extern "C" int cmb_m3_prep_bc_bwd(const void* BC, const float* scale_g, const float* ang, const float* rstd, const void* wB, const void* bB,
                                  const void* wC, const void* bC, const void* gBg, const void* gCg, void* gBC, float* g_scale, float* g_ang,
                                  float* gwB, float* gbB, float* gwC, float* gbC, long long tokens, int G, int N, int R, void* stream) {
  if (tokens <= 0) return 0;
  if (N % 64 || N > 256 || 2 * R > N) return 1;
  const int tpw = 32;
  const long long warps = ((tokens + tpw - 1) / tpw) * G;
  const unsigned grid = static_cast<unsigned>((warps * 32 + 255) / 256);
  auto st = static_cast<cudaStream_t>(stream);
#define CMB_PREP_BWD(NJ_)                                                                                                          \
  cmb::m3_prep_bc_bwd_kernel<NJ_><<<grid, 256, 0, st>>>(static_cast<const bf16*>(BC), scale_g, ang, rstd, static_cast<const bf16*>(wB), \
                                                         static_cast<const bf16*>(bB), static_cast<const bf16*>(wC),               \
                                                         static_cast<const bf16*>(bC), static_cast<const bf16*>(gBg),              \
                                                         static_cast<const bf16*>(gCg), static_cast<bf16*>(gBC), g_scale, g_ang, gwB, gbB, \
                                                         gwC, gbC, tokens, G, N, R, tpw)
  switch (N / 64) {
    case 1: CMB_PREP_BWD(1); break;
    case 2: CMB_PREP_BWD(2); break;
    case 3: CMB_PREP_BWD(3); break;
    default: CMB_PREP_BWD(4); break;
  }
#undef CMB_PREP_BWD
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// ---------------------------------------------------------------------------------------------- prefix sum along the sequence
// out[b,t,c] = Σ_{t' ≤ t} in[b,t',c]  (or Σ_{t' ≥ t} with `reverse`), fp32, C contiguous.  Three tiny kernels: per-segment local
// scans (thread per (b, segment, c), c fastest → coalesced), an exclusive scan of the segment totals, and the offset add.
namespace cmb {
constexpr int SCAN_SEG = 64;

template <bool REV>
__global__ void scan_local_kernel(const float* __restrict__ in, float* __restrict__ out, float* __restrict__ totals, int S, int C, int nseg,
                                  long long total_threads) {
  const long long idx = blockIdx.x * 256LL + threadIdx.x;
  if (idx >= total_threads) return;
  const int c = static_cast<int>(idx % C);
  const int seg = static_cast<int>((idx / C) % nseg);
  const long long b = idx / (static_cast<long long>(C) * nseg);
  const int t0 = seg * SCAN_SEG, t1 = min(S, t0 + SCAN_SEG);
  float acc = 0.f;
  if (REV) {
    for (int t = t1 - 1; t >= t0; --t) {
      acc += in[(b * S + t) * C + c];
      out[(b * S + t) * C + c] = acc;
    }
  } else {
    for (int t = t0; t < t1; ++t) {
      acc += in[(b * S + t) * C + c];
      out[(b * S + t) * C + c] = acc;
    }
  }
  totals[(b * nseg + seg) * C + c] = acc;
}

template <bool REV>
__global__ void scan_totals_kernel(float* __restrict__ totals, int C, int nseg, long long cols) {
  const long long idx = blockIdx.x * 256LL + threadIdx.x;   // (b, c)
  if (idx >= cols) return;
  const int c = static_cast<int>(idx % C);
  const long long b = idx / C;
  float acc = 0.f;
  for (int k = 0; k < nseg; ++k) {
    const int seg = REV ? nseg - 1 - k : k;
    float* p = totals + (b * nseg + seg) * C + c;
    const float v = *p;
    *p = acc;          // exclusive offset for this segment
    acc += v;
  }
}

__global__ void scan_add_kernel(float* __restrict__ out, const float* __restrict__ offsets, int S, int C, int nseg, long long n) {
  const long long idx = blockIdx.x * 256LL + threadIdx.x;
  if (idx >= n) return;
  const int c = static_cast<int>(idx % C);
  const long long bt = idx / C;
  const int t = static_cast<int>(bt % S);
  const long long b = bt / S;
  out[idx] += offsets[(b * nseg + t / SCAN_SEG) * C + c];
}
}  // namespace cmb

// `totals` is scratch of Bn · ceil(S/64) · C floats.
extern "C" int cmb_cumsum_seq(const float* in, float* out, float* totals, int Bn, int S, int C, int reverse, void* stream) {
  if (Bn <= 0 || S <= 0 || C <= 0) return 0;
  const int nseg = (S + cmb::SCAN_SEG - 1) / cmb::SCAN_SEG;
  const long long th = static_cast<long long>(Bn) * nseg * C, cols = static_cast<long long>(Bn) * C, n = static_cast<long long>(Bn) * S * C;
  auto st = static_cast<cudaStream_t>(stream);
  const unsigned g1 = static_cast<unsigned>((th + 255) / 256), g2 = static_cast<unsigned>((cols + 255) / 256), g3 = static_cast<unsigned>((n + 255) / 256);
  if (reverse) {
    cmb::scan_local_kernel<true><<<g1, 256, 0, st>>>(in, out, totals, S, C, nseg, th);
    cmb::scan_totals_kernel<true><<<g2, 256, 0, st>>>(totals, C, nseg, cols);
  } else {
    cmb::scan_local_kernel<false><<<g1, 256, 0, st>>>(in, out, totals, S, C, nseg, th);
    cmb::scan_totals_kernel<false><<<g2, 256, 0, st>>>(totals, C, nseg, cols);
  }
  cmb::scan_add_kernel<<<g3, 256, 0, st>>>(out, totals, S, C, nseg, n);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
