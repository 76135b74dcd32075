// M2RNN matrix-state recurrence, forward and backward, as persistent time loops (sm_100a).
//
//   z_t = h_{t-1}·W + k_t ⊗ v_t          h ∈ R^{K×V}, W ∈ R^{V×V}
//   h_t = f_t·h_{t-1} + (1 − f_t)·tanh(z_t)
//   y_t = q_t · h_t                       (contracts K)
//
// The recurrence is nonlinear, so there is no parallel scan: the kernel is latency bound and is organised to keep the
// per-step critical path short.  One CTA per (batch, head); thread (k, j) owns the four state columns 4j..4j+3 of row k
// (V = 16 → four threads per row, K·4 threads per CTA).  W lives in shared memory (broadcast reads), the state in
// registers; the other 12 entries of a row come from the three quad neighbours by shuffle.  Inputs are staged through
// shared memory one chunk of 32 time steps at a time, and all cross-warp reductions (y, and in backward dv and df) are
// written as per-warp partials for the whole chunk and folded once per chunk, so a chunk costs two block barriers.
// Forward optionally records h_{t-1} (bf16) for every step; backward recomputes tanh(z_t) from it, walks t downwards
// carrying dh, accumulates dW in registers (64 per thread) and reduces it over the CTA once at the end.
//
// Reference kernels: cppmega_mlx/nn/_tilelang/m2rnn.py:128-248 (forward, one threadgroup per (b,h), K threads) and
// :300-485 (backward, replay + reverse sweep, host-side sum of dW over the batch).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace cmb {

constexpr int M2_V = 16;
constexpr int M2_CHUNK = 32;

struct M2Params {
  const __nv_bfloat16 *q, *k, *v;   // token stride ss_*, head slices contiguous
  const float* f;                    // [B,S,nf]
  const float* W;                    // [nw,V,V]
  const float* h0;                   // [B,H,K,V] or null
  __nv_bfloat16* y;                  // [B,S,H,V]
  float* h_last;                     // [B,H,K,V]
  __nv_bfloat16* hist;               // [B,H,S,K,V] h_{t-1}, or null
  long long sq_b, sq_s, sk_b, sk_s, sv_b, sv_s;   // element strides (batch, token)
  int B, S, H, nq, nk, nv, nw, nf;
  // backward only
  const __nv_bfloat16* dy;           // [B,S,H,V]
  const float* dh_last;              // [B,H,K,V] or null
  float *dq, *dk, *dv;               // [B,S,H,K] / [B,S,H,K] / [B,S,H,V] fp32, per expanded head
  float* df;                         // [B,S,H]
  float* dW;                         // [B,H,V,V] per-CTA result (summed over batch / shared heads by the caller)
  float* dh0;                        // [B,H,K,V]
};

__device__ __forceinline__ float fast_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Gather the full 16-entry row from the four quad lanes: out[4*j+i] = value i of lane (quad base + j).
__device__ __forceinline__ void quad_row(const float (&mine)[4], float (&row)[16], int lane) {
  const int base = lane & ~3;
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) row[4 * j + i] = __shfl_sync(0xffffffffu, mine[i], base + j);
}

template <int K>
__global__ void __launch_bounds__(K * 4, 1) m2rnn_fwd_kernel(const M2Params p) {
  constexpr int NT = K * 4;
  constexpr int NW = NT / 32;
  __shared__ float sW[M2_V * M2_V];
  __shared__ float sq[M2_CHUNK][K], sk[M2_CHUNK][K], sv[M2_CHUNK][M2_V], sf[M2_CHUNK];
  __shared__ float sy[M2_CHUNK][NW][M2_V];
  const int b = blockIdx.x / p.H, h = blockIdx.x % p.H;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int krow = tid >> 2, j = tid & 3;
  const int hq = h / (p.H / p.nq), hk = h / (p.H / p.nk), hv = h / (p.H / p.nv), hw = h / (p.H / p.nw), hf = h / (p.H / p.nf);
  for (int i = tid; i < M2_V * M2_V; i += NT) sW[i] = p.W[hw * M2_V * M2_V + i];
  float st[4];
  const long long hoff = ((static_cast<long long>(b) * p.H + h) * K + krow) * M2_V + 4 * j;
#pragma unroll
  for (int i = 0; i < 4; ++i) st[i] = p.h0 != nullptr ? p.h0[hoff + i] : 0.f;
  const __nv_bfloat16* qb = p.q + b * p.sq_b + static_cast<long long>(hq) * K;
  const __nv_bfloat16* kb = p.k + b * p.sk_b + static_cast<long long>(hk) * K;
  const __nv_bfloat16* vb = p.v + b * p.sv_b + static_cast<long long>(hv) * M2_V;
  const float* fb = p.f + static_cast<long long>(b) * p.S * p.nf + hf;
  __syncthreads();
  for (int t0 = 0; t0 < p.S; t0 += M2_CHUNK) {
    const int n = min(M2_CHUNK, p.S - t0);
    for (int i = tid; i < n * K; i += NT) {
      const int tt = i / K, c = i % K;
      sq[tt][c] = __bfloat162float(qb[(t0 + tt) * p.sq_s + c]);
      sk[tt][c] = __bfloat162float(kb[(t0 + tt) * p.sk_s + c]);
    }
    for (int i = tid; i < n * M2_V; i += NT) sv[i / M2_V][i % M2_V] = __bfloat162float(vb[(t0 + i / M2_V) * p.sv_s + i % M2_V]);
    for (int i = tid; i < n; i += NT) sf[i] = fb[static_cast<long long>(t0 + i) * p.nf];
    __syncthreads();
    for (int tt = 0; tt < n; ++tt) {
      if (p.hist != nullptr) {
        __nv_bfloat16* hp = p.hist + (((static_cast<long long>(b) * p.H + h) * p.S + t0 + tt) * K + krow) * M2_V + 4 * j;
        *reinterpret_cast<__nv_bfloat162*>(hp) = __floats2bfloat162_rn(st[0], st[1]);
        *reinterpret_cast<__nv_bfloat162*>(hp + 2) = __floats2bfloat162_rn(st[2], st[3]);
      }
      float row[16];
      quad_row(st, row, lane);
      const float kk = sk[tt][krow], ff = sf[tt], qq = sq[tt][krow];
      float part[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int w = 4 * j + i;
        float z = kk * sv[tt][w];
#pragma unroll
        for (int v = 0; v < M2_V; ++v) z = fmaf(row[v], sW[v * M2_V + w], z);
        st[i] = ff * st[i] + (1.f - ff) * fast_tanh(z);
        part[i] = qq * st[i];
      }
      // reduce over the 8 rows of this warp (lane bits 2..4), keeping the column (lane bits 0..1)
#pragma unroll
      for (int off = 4; off < 32; off <<= 1)
#pragma unroll
        for (int i = 0; i < 4; ++i) part[i] += __shfl_xor_sync(0xffffffffu, part[i], off);
      if (lane < 4) {
#pragma unroll
        for (int i = 0; i < 4; ++i) sy[tt][warp][4 * lane + i] = part[i];
      }
    }
    __syncthreads();
    for (int i = tid; i < n * M2_V; i += NT) {
      const int tt = i / M2_V, w = i % M2_V;
      float a = 0.f;
#pragma unroll
      for (int ww = 0; ww < NW; ++ww) a += sy[tt][ww][w];
      p.y[((static_cast<long long>(b) * p.S + t0 + tt) * p.H + h) * M2_V + w] = __float2bfloat16(a);
    }
    // sy / sq are rewritten only after the next chunk's load barrier
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) p.h_last[hoff + i] = st[i];
}

constexpr int M2_CHUNK_B = 16;

template <int K>
__global__ void __launch_bounds__(K * 4, 1) m2rnn_bwd_kernel(const M2Params p) {
  constexpr int NT = K * 4;
  constexpr int NW = NT / 32;
  __shared__ float sW[M2_V * M2_V];
  __shared__ float sWT[M2_V * 17];   // sWT[v*17 + w] = W[v][w], padded so that the four column groups hit distinct banks
  __shared__ float sq[M2_CHUNK_B][K], sk[M2_CHUNK_B][K], sv[M2_CHUNK_B][M2_V], sf[M2_CHUNK_B], sdy[M2_CHUNK_B][M2_V];
  __shared__ float sdq[M2_CHUNK_B][K], sdk[M2_CHUNK_B][K], sdv[M2_CHUNK_B][NW][M2_V], sdf[M2_CHUNK_B][NW];
  __shared__ float sdW[M2_V * M2_V];
  const int b = blockIdx.x / p.H, h = blockIdx.x % p.H;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int krow = tid >> 2, j = tid & 3;
  const int hq = h / (p.H / p.nq), hk = h / (p.H / p.nk), hv = h / (p.H / p.nv), hw = h / (p.H / p.nw), hf = h / (p.H / p.nf);
  for (int i = tid; i < M2_V * M2_V; i += NT) {
    const float w = p.W[hw * M2_V * M2_V + i];
    sW[i] = w;
    sWT[(i / M2_V) * 17 + (i % M2_V)] = w;
    sdW[i] = 0.f;
  }
  const long long bh = static_cast<long long>(b) * p.H + h;
  const long long hoff = (bh * K + krow) * M2_V + 4 * j;
  float dh[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) dh[i] = p.dh_last != nullptr ? p.dh_last[hoff + i] : 0.f;
  float acc[16][4];
#pragma unroll
  for (int v = 0; v < 16; ++v)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[v][i] = 0.f;
  const __nv_bfloat16* qb = p.q + b * p.sq_b + static_cast<long long>(hq) * K;
  const __nv_bfloat16* kb = p.k + b * p.sk_b + static_cast<long long>(hk) * K;
  const __nv_bfloat16* vb = p.v + b * p.sv_b + static_cast<long long>(hv) * M2_V;
  const float* fb = p.f + static_cast<long long>(b) * p.S * p.nf + hf;
  const int nchunks = (p.S + M2_CHUNK_B - 1) / M2_CHUNK_B;
  __syncthreads();
  for (int c = nchunks - 1; c >= 0; --c) {
    const int t0 = c * M2_CHUNK_B;
    const int n = min(M2_CHUNK_B, p.S - t0);
    for (int i = tid; i < n * K; i += NT) {
      const int tt = i / K, cc = i % K;
      sq[tt][cc] = __bfloat162float(qb[(t0 + tt) * p.sq_s + cc]);
      sk[tt][cc] = __bfloat162float(kb[(t0 + tt) * p.sk_s + cc]);
    }
    for (int i = tid; i < n * M2_V; i += NT) {
      const int tt = i / M2_V, w = i % M2_V;
      sv[tt][w] = __bfloat162float(vb[(t0 + tt) * p.sv_s + w]);
      sdy[tt][w] = __bfloat162float(p.dy[((static_cast<long long>(b) * p.S + t0 + tt) * p.H + h) * M2_V + w]);
    }
    for (int i = tid; i < n; i += NT) sf[i] = fb[static_cast<long long>(t0 + i) * p.nf];
    __syncthreads();
    for (int tt = n - 1; tt >= 0; --tt) {
      const __nv_bfloat16* hp = p.hist + ((bh * p.S + t0 + tt) * K + krow) * M2_V + 4 * j;
      const float2 a01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(hp));
      const float2 a23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(hp + 2));
      const float hprev[4] = {a01.x, a01.y, a23.x, a23.y};
      float hrow[16];
      quad_row(hprev, hrow, lane);
      const float kk = sk[tt][krow], ff = sf[tt], qq = sq[tt][krow];
      float dz[4], pdq = 0.f, pdk = 0.f, pdf = 0.f, pdv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int w = 4 * j + i;
        float z = kk * sv[tt][w];
#pragma unroll
        for (int v = 0; v < M2_V; ++v) z = fmaf(hrow[v], sW[v * M2_V + w], z);
        const float cnd = fast_tanh(z);
        const float ht = ff * hprev[i] + (1.f - ff) * cnd;
        const float dyw = sdy[tt][w];
        dh[i] = fmaf(qq, dyw, dh[i]);
        pdq = fmaf(dyw, ht, pdq);
        pdf = fmaf(dh[i], hprev[i] - cnd, pdf);
        dz[i] = (1.f - ff) * dh[i] * (1.f - cnd * cnd);
        pdk = fmaf(dz[i], sv[tt][w], pdk);
        pdv[i] = dz[i] * kk;
#pragma unroll
        for (int v = 0; v < M2_V; ++v) acc[v][i] = fmaf(hrow[v], dz[i], acc[v][i]);
      }
      float dzrow[16];
      quad_row(dz, dzrow, lane);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float s = ff * dh[i];
        const float* wt = sWT + (4 * j + i) * 17;
#pragma unroll
        for (int w = 0; w < M2_V; ++w) s = fmaf(dzrow[w], wt[w], s);
        dh[i] = s;   // now dL/dh_{t-1}
      }
      // quad reductions (row-wise sums over the 16 columns)
      pdq += __shfl_xor_sync(0xffffffffu, pdq, 1);
      pdq += __shfl_xor_sync(0xffffffffu, pdq, 2);
      pdk += __shfl_xor_sync(0xffffffffu, pdk, 1);
      pdk += __shfl_xor_sync(0xffffffffu, pdk, 2);
      if (j == 0) {
        sdq[tt][krow] = pdq;
        sdk[tt][krow] = pdk;
      }
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) pdf += __shfl_xor_sync(0xffffffffu, pdf, off);
#pragma unroll
      for (int off = 4; off < 32; off <<= 1)
#pragma unroll
        for (int i = 0; i < 4; ++i) pdv[i] += __shfl_xor_sync(0xffffffffu, pdv[i], off);
      if (lane == 0) sdf[tt][warp] = pdf;
      if (lane < 4) {
#pragma unroll
        for (int i = 0; i < 4; ++i) sdv[tt][warp][4 * lane + i] = pdv[i];
      }
    }
    __syncthreads();
    for (int i = tid; i < n * K; i += NT) {
      const int tt = i / K, cc = i % K;
      const long long o = ((static_cast<long long>(b) * p.S + t0 + tt) * p.H + h) * K + cc;
      p.dq[o] = sdq[tt][cc];
      p.dk[o] = sdk[tt][cc];
    }
    for (int i = tid; i < n * M2_V; i += NT) {
      const int tt = i / M2_V, w = i % M2_V;
      float a = 0.f;
#pragma unroll
      for (int ww = 0; ww < NW; ++ww) a += sdv[tt][ww][w];
      p.dv[((static_cast<long long>(b) * p.S + t0 + tt) * p.H + h) * M2_V + w] = a;
    }
    for (int i = tid; i < n; i += NT) {
      float a = 0.f;
#pragma unroll
      for (int ww = 0; ww < NW; ++ww) a += sdf[i][ww];
      p.df[(static_cast<long long>(b) * p.S + t0 + i) * p.H + h] = a;
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) p.dh0[hoff + i] = dh[i];
  // dW[v][w] = Σ_k acc: reduce over the rows held by this warp, then across warps through shared memory
#pragma unroll
  for (int v = 0; v < 16; ++v)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float a = acc[v][i];
#pragma unroll
      for (int off = 4; off < 32; off <<= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
      if (lane < 4) atomicAdd(&sdW[v * M2_V + 4 * lane + i], a);
    }
  __syncthreads();
  for (int i = tid; i < M2_V * M2_V; i += NT) p.dW[bh * M2_V * M2_V + i] = sdW[i];
}

}  // namespace cmb

static bool m2_ok(const cmb::M2Params& p, int K, int V) {
  if (V != cmb::M2_V || (K != 32 && K != 64)) return false;
  for (int n : {p.nq, p.nk, p.nv, p.nw, p.nf})
    if (n <= 0 || p.H % n) return false;
  return p.B > 0 && p.S > 0 && p.H > 0;
}

// ip = {B, S, H, K, V, nq, nk, nv, nw, nf}; lp = {sq_b, sq_s, sk_b, sk_s, sv_b, sv_s} (element strides; head slices of
// width K / V are contiguous inside a token). `hist` (bf16 [B,H,S,K,V]) may be null when no backward will follow.
extern "C" int cmb_m2rnn_fwd(const void* q, const void* k, const void* v, const float* f, const float* W, const float* h0, void* y,
                             float* h_last, void* hist, const int* ip, const long long* lp, void* stream) {
  cmb::M2Params p{};
  p.q = static_cast<const __nv_bfloat16*>(q); p.k = static_cast<const __nv_bfloat16*>(k); p.v = static_cast<const __nv_bfloat16*>(v);
  p.f = f; p.W = W; p.h0 = h0; p.y = static_cast<__nv_bfloat16*>(y); p.h_last = h_last; p.hist = static_cast<__nv_bfloat16*>(hist);
  p.B = ip[0]; p.S = ip[1]; p.H = ip[2]; p.nq = ip[5]; p.nk = ip[6]; p.nv = ip[7]; p.nw = ip[8]; p.nf = ip[9];
  p.sq_b = lp[0]; p.sq_s = lp[1]; p.sk_b = lp[2]; p.sk_s = lp[3]; p.sv_b = lp[4]; p.sv_s = lp[5];
  if (!m2_ok(p, ip[3], ip[4])) return -1;
  auto st = static_cast<cudaStream_t>(stream);
  if (ip[3] == 64) cmb::m2rnn_fwd_kernel<64><<<p.B * p.H, 256, 0, st>>>(p);
  else cmb::m2rnn_fwd_kernel<32><<<p.B * p.H, 128, 0, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Gradients are written per expanded head: dq,dk [B,S,H,K], dv [B,S,H,V], df [B,S,H], dW [B,H,V,V], dh0 [B,H,K,V] (fp32);
// the caller sums over the batch (dW) and over heads that share an input.
extern "C" int cmb_m2rnn_bwd(const void* q, const void* k, const void* v, const float* f, const float* W, const void* hist,
                             const void* dy, const float* dh_last, float* dq, float* dk, float* dv, float* df, float* dW, float* dh0,
                             const int* ip, const long long* lp, void* stream) {
  cmb::M2Params p{};
  p.q = static_cast<const __nv_bfloat16*>(q); p.k = static_cast<const __nv_bfloat16*>(k); p.v = static_cast<const __nv_bfloat16*>(v);
  p.f = f; p.W = W; p.hist = static_cast<__nv_bfloat16*>(const_cast<void*>(hist));
  p.dy = static_cast<const __nv_bfloat16*>(dy); p.dh_last = dh_last;
  p.dq = dq; p.dk = dk; p.dv = dv; p.df = df; p.dW = dW; p.dh0 = dh0;
  p.B = ip[0]; p.S = ip[1]; p.H = ip[2]; p.nq = ip[5]; p.nk = ip[6]; p.nv = ip[7]; p.nw = ip[8]; p.nf = ip[9];
  p.sq_b = lp[0]; p.sq_s = lp[1]; p.sk_b = lp[2]; p.sk_s = lp[3]; p.sv_b = lp[4]; p.sv_s = lp[5];
  if (!m2_ok(p, ip[3], ip[4]) || hist == nullptr) return -1;
  auto st = static_cast<cudaStream_t>(stream);
  if (ip[3] == 64) cmb::m2rnn_bwd_kernel<64><<<p.B * p.H, 256, 0, st>>>(p);
  else cmb::m2rnn_bwd_kernel<32><<<p.B * p.H, 128, 0, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// ---------------------------------------------------------------------------------------------------------------------
// One-token step for decoding: the state h [B,H,K,V] (fp32) is read, advanced by one token and written back, y = q·h.
// One CTA per (batch, head); thread (grp, w) owns column w of R = K / (256 / V) consecutive state rows, so W[v][w] is read once
// per thread (coalesced over w) and the state rows come from shared memory as broadcasts.  No history is kept.
namespace cmb {
template <int K, int V>
__global__ void __launch_bounds__(256) m2rnn_step_kernel(M2Params p) {
  constexpr int GROUPS = 256 / V, R = K / GROUPS;
  static_assert(GROUPS >= 1 && R >= 1 && R * GROUPS == K, "row split");
  __shared__ float hs[K * V];
  __shared__ float qs[K], ks[K];
  const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H, tid = threadIdx.x;
  const int hq = h / (p.H / p.nq), hk = h / (p.H / p.nk), hv = h / (p.H / p.nv), hw = h / (p.H / p.nw), hf = h / (p.H / p.nf);
  const long long hoff = static_cast<long long>(bh) * K * V;
  for (int i = tid; i < K * V; i += 256) hs[i] = p.h0 != nullptr ? p.h0[hoff + i] : 0.f;
  if (tid < K) {
    qs[tid] = __bfloat162float(p.q[b * p.sq_b + static_cast<long long>(hq) * K + tid]);
    ks[tid] = __bfloat162float(p.k[b * p.sk_b + static_cast<long long>(hk) * K + tid]);
  }
  __syncthreads();
  const int w = tid % V, r0 = (tid / V) * R;
  const float* Wh = p.W + static_cast<long long>(hw) * V * V;
  float acc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = 0.f;
  for (int v = 0; v < V; ++v) {
    const float wv = Wh[v * V + w];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = fmaf(hs[(r0 + r) * V + v], wv, acc[r]);
  }
  const float vt = __bfloat162float(p.v[b * p.sv_b + static_cast<long long>(hv) * V + w]);
  const float ft = p.f[static_cast<long long>(b) * p.nf + hf];
  float hn[R];
#pragma unroll
  for (int r = 0; r < R; ++r) hn[r] = ft * hs[(r0 + r) * V + w] + (1.f - ft) * tanhf(acc[r] + ks[r0 + r] * vt);
  __syncthreads();      // every thread has read the old rows it needs
#pragma unroll
  for (int r = 0; r < R; ++r) {
    hs[(r0 + r) * V + w] = hn[r];
    p.h_last[hoff + (r0 + r) * V + w] = hn[r];
  }
  __syncthreads();
  if (tid < V) {
    float y = 0.f;
#pragma unroll 8
    for (int kk = 0; kk < K; ++kk) y = fmaf(qs[kk], hs[kk * V + tid], y);
    p.y[static_cast<long long>(bh) * V + tid] = __float2bfloat16(y);
  }
}
}  // namespace cmb

// Same argument convention as cmb_m2rnn_fwd with S = 1 (the strides over tokens are unused); covers (K,V) = (32,16), (64,16), (64,128).
extern "C" int cmb_m2rnn_step(const void* q, const void* k, const void* v, const float* f, const float* W, const float* h0, void* y,
                              float* h_last, const int* ip, const long long* lp, void* stream) {
  cmb::M2Params p{};
  p.q = static_cast<const __nv_bfloat16*>(q); p.k = static_cast<const __nv_bfloat16*>(k); p.v = static_cast<const __nv_bfloat16*>(v);
  p.f = f; p.W = W; p.h0 = h0; p.y = static_cast<__nv_bfloat16*>(y); p.h_last = h_last;
  p.B = ip[0]; p.S = ip[1]; p.H = ip[2]; p.nq = ip[5]; p.nk = ip[6]; p.nv = ip[7]; p.nw = ip[8]; p.nf = ip[9];
  p.sq_b = lp[0]; p.sq_s = lp[1]; p.sk_b = lp[2]; p.sk_s = lp[3]; p.sv_b = lp[4]; p.sv_s = lp[5];
  if (p.S != 1 || p.B <= 0 || p.H <= 0 || h_last == nullptr || y == nullptr) return -1;
  for (int n : {p.nq, p.nk, p.nv, p.nw, p.nf})
    if (n <= 0 || p.H % n) return -1;
  auto st = static_cast<cudaStream_t>(stream);
  const int K = ip[3], V = ip[4];
  if (K == 32 && V == 16) cmb::m2rnn_step_kernel<32, 16><<<p.B * p.H, 256, 0, st>>>(p);
  else if (K == 64 && V == 16) cmb::m2rnn_step_kernel<64, 16><<<p.B * p.H, 256, 0, st>>>(p);
  else if (K == 64 && V == 128) cmb::m2rnn_step_kernel<64, 128><<<p.B * p.H, 256, 0, st>>>(p);
  else return -1;
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// ---------------------------------------------------------------------------------------------------------------------
// Post-recurrence gate of the M2RNN mixer in one pass each way:   out = (y + v·D) · silu(g)
// y [B,S,H,V] is the recurrence output (dense); v [B,S,nv,V] and g [B,S,ng,V] are strided slices of packed projections whose
// heads are shared by H/nv (H/ng) consecutive output heads; D [H,V].  Backward returns dy (dense), and per expanded head dv
// and dg (the caller folds heads that share an input) plus dD accumulated over all tokens.
// Reference fusion: cppmega_mlx/nn/_tilelang/m2rnn_path_c.py:2421 (forward), :2519 (backward).
namespace cmb {

struct M2PostParams {
  const __nv_bfloat16 *y, *v, *g;
  const float* D;                    // [H,V] or null (no residual)
  __nv_bfloat16* out;
  long long sv_b, sv_s, sg_b, sg_s;  // element strides of v and g (batch, token)
  int B, S, H, V, nv, ng;
  const __nv_bfloat16* dout;
  __nv_bfloat16* dy;
  float *dv, *dg, *dD;               // [B,S,H,V] ×2, [H,V] (dD pre-zeroed)
};

__global__ void __launch_bounds__(256) m2rnn_post_fwd_kernel(const M2PostParams p) {
  const int HV = p.H * p.V;
  const int hw = blockIdx.x * blockDim.x + threadIdx.x;
  if (hw >= HV) return;
  const int h = hw / p.V, w = hw % p.V;
  const int hv = h / (p.H / p.nv), hg = h / (p.H / p.ng);
  const float d = p.D != nullptr ? p.D[hw] : 0.f;
  const long long tokens = static_cast<long long>(p.B) * p.S;
  for (long long t = blockIdx.y; t < tokens; t += gridDim.y) {
    const long long b = t / p.S, s = t % p.S;
    const float yv = __bfloat162float(p.y[t * HV + hw]);
    const float vv = __bfloat162float(p.v[b * p.sv_b + s * p.sv_s + hv * p.V + w]);
    const float gv = __bfloat162float(p.g[b * p.sg_b + s * p.sg_s + hg * p.V + w]);
    const float sg = gv / (1.f + __expf(-gv));
    p.out[t * HV + hw] = __float2bfloat16((yv + vv * d) * sg);
  }
}

__global__ void __launch_bounds__(256) m2rnn_post_bwd_kernel(const M2PostParams p) {
  const int HV = p.H * p.V;
  const int hw = blockIdx.x * blockDim.x + threadIdx.x;
  if (hw >= HV) return;
  const int h = hw / p.V, w = hw % p.V;
  const int hv = h / (p.H / p.nv), hg = h / (p.H / p.ng);
  const float d = p.D != nullptr ? p.D[hw] : 0.f;
  const long long tokens = static_cast<long long>(p.B) * p.S;
  float accD = 0.f;
  for (long long t = blockIdx.y; t < tokens; t += gridDim.y) {
    const long long b = t / p.S, s = t % p.S;
    const float yv = __bfloat162float(p.y[t * HV + hw]);
    const float vv = __bfloat162float(p.v[b * p.sv_b + s * p.sv_s + hv * p.V + w]);
    const float gv = __bfloat162float(p.g[b * p.sg_b + s * p.sg_s + hg * p.V + w]);
    const float go = __bfloat162float(p.dout[t * HV + hw]);
    const float sig = 1.f / (1.f + __expf(-gv));
    const float sg = gv * sig;
    const float gy = go * sg;                       // ∂L/∂(y + v·D)
    p.dy[t * HV + hw] = __float2bfloat16(gy);
    p.dv[t * HV + hw] = gy * d;
    p.dg[t * HV + hw] = go * (yv + vv * d) * (sig * (1.f + gv * (1.f - sig)));
    accD = fmaf(gy, vv, accD);
  }
  if (p.dD != nullptr) atomicAdd(&p.dD[hw], accD);
}

}  // namespace cmb

// ip = {B, S, H, V, nv, ng}; lp = {sv_b, sv_s, sg_b, sg_s}.
extern "C" int cmb_m2rnn_post_fwd(const void* y, const void* v, const void* g, const float* D, void* out, const int* ip, const long long* lp,
                                  void* stream) {
  cmb::M2PostParams p{};
  p.y = static_cast<const __nv_bfloat16*>(y); p.v = static_cast<const __nv_bfloat16*>(v); p.g = static_cast<const __nv_bfloat16*>(g);
  p.D = D; p.out = static_cast<__nv_bfloat16*>(out);
  p.B = ip[0]; p.S = ip[1]; p.H = ip[2]; p.V = ip[3]; p.nv = ip[4]; p.ng = ip[5];
  p.sv_b = lp[0]; p.sv_s = lp[1]; p.sg_b = lp[2]; p.sg_s = lp[3];
  if (p.B <= 0 || p.S <= 0 || p.H <= 0 || p.V <= 0 || p.nv <= 0 || p.ng <= 0 || p.H % p.nv || p.H % p.ng) return -1;
  const int HV = p.H * p.V;
  dim3 grid((HV + 255) / 256, static_cast<unsigned>(min(static_cast<long long>(p.B) * p.S, 148LL * 16 / ((HV + 255) / 256) + 1)));
  cmb::m2rnn_post_fwd_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int cmb_m2rnn_post_bwd(const void* y, const void* v, const void* g, const float* D, const void* dout, void* dy, float* dv, float* dg,
                                  float* dD, const int* ip, const long long* lp, void* stream) {
  cmb::M2PostParams p{};
  p.y = static_cast<const __nv_bfloat16*>(y); p.v = static_cast<const __nv_bfloat16*>(v); p.g = static_cast<const __nv_bfloat16*>(g);
  p.D = D; p.dout = static_cast<const __nv_bfloat16*>(dout); p.dy = static_cast<__nv_bfloat16*>(dy); p.dv = dv; p.dg = dg; p.dD = dD;
  p.B = ip[0]; p.S = ip[1]; p.H = ip[2]; p.V = ip[3]; p.nv = ip[4]; p.ng = ip[5];
  p.sv_b = lp[0]; p.sv_s = lp[1]; p.sg_b = lp[2]; p.sg_s = lp[3];
  if (p.B <= 0 || p.S <= 0 || p.H <= 0 || p.V <= 0 || p.nv <= 0 || p.ng <= 0 || p.H % p.nv || p.H % p.ng) return -1;
  const int HV = p.H * p.V;
  dim3 grid((HV + 255) / 256, static_cast<unsigned>(min(static_cast<long long>(p.B) * p.S, 148LL * 16 / ((HV + 255) / 256) + 1)));
  cmb::m2rnn_post_bwd_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
