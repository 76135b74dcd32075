// Causal depthwise conv1d (+bias) followed by SiLU over channel-last activations, forward and backward.
//
//   pre[b,s,c] = bias[c] + Σ_k w[c,k] · in[b, s−K+1+k, c]        (zero left padding)
//   y          = silu(pre)
//
// The input is a column slice of a wider row-major matrix (row pitch `ld_in`, first channel `c_off`),
// e.g. the [x|B|C] part of Mamba3's packed projection or the [q|k|v] part of M2RNN's, so no split copy is
// needed; the output goes to two dense tensors (channels [0,C1) and [C1,C)).  Each thread owns one
// bf16 channel pair and a run of TS consecutive tokens, sliding a K-tap window through registers.
// Math parity: cppmega_mlx/nn/mamba3.py:322 (conv) followed by nn.silu at :715; weights are [C,K,1].
#include "sm100.cuh"

namespace cmb {

constexpr int CONV_TS = 8;
constexpr int CONV_RUN = 128;  // tokens per warp in the backward kernel
constexpr int CONV_MAXK = 8;

__device__ __forceinline__ float2 ld2(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}

template <int KC>  // KC > 0: compile-time tap count (everything stays in registers); 0: run-time K
__global__ void __launch_bounds__(256) conv_silu_fwd_kernel(const __nv_bfloat16* __restrict__ in, long long ld_in,
                                                             int c_off, const __nv_bfloat16* __restrict__ w,
                                                             const __nv_bfloat16* __restrict__ bias,
                                                             __nv_bfloat16* __restrict__ out1,
                                                             __nv_bfloat16* __restrict__ out2, int Bn, int S, int C,
                                                             int C1, int Krt) {
  const int K = KC > 0 ? KC : Krt;
  const int cp = blockIdx.x * 32 + (threadIdx.x & 31);  // channel pair
  const int c = cp * 2;
  const long long tile = blockIdx.y * 8LL + (threadIdx.x >> 5);
  const int tiles_per_seq = (S + CONV_TS - 1) / CONV_TS;
  if (c >= C || tile >= static_cast<long long>(Bn) * tiles_per_seq) return;
  const int b = static_cast<int>(tile / tiles_per_seq);
  const int s0 = static_cast<int>(tile % tiles_per_seq) * CONV_TS;
  float2 wk[CONV_MAXK];
#pragma unroll
  for (int k = 0; k < K; ++k) wk[k] = make_float2(__bfloat162float(w[c * K + k]), __bfloat162float(w[(c + 1) * K + k]));
  const float2 bs = bias != nullptr ? ld2(bias + c) : make_float2(0.f, 0.f);
  const __nv_bfloat16* ib = in + static_cast<long long>(b) * S * ld_in + c_off + c;
  float2 win[CONV_MAXK];  // win[k] = in[s-K+1+k]
#pragma unroll
  for (int k = 0; k < K - 1; ++k) {
    const int s = s0 - (K - 1) + k;
    win[k + 1] = s >= 0 ? ld2(ib + s * ld_in) : make_float2(0.f, 0.f);
  }
#pragma unroll
  for (int i = 0; i < CONV_TS; ++i) {
    const int s = s0 + i;
    if (s >= S) break;
#pragma unroll
    for (int k = 0; k < K - 1; ++k) win[k] = win[k + 1];
    win[K - 1] = ld2(ib + s * ld_in);
    float2 acc = bs;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      acc.x += wk[k].x * win[k].x;
      acc.y += wk[k].y * win[k].y;
    }
    const float y0 = acc.x / (1.f + __expf(-acc.x)), y1 = acc.y / (1.f + __expf(-acc.y));
    __nv_bfloat16* dst = c < C1 ? out1 + (static_cast<long long>(b) * S + s) * C1 + c
                                : out2 + (static_cast<long long>(b) * S + s) * (C - C1) + (c - C1);
    *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(y0, y1);
  }
}

// Backward. dy comes from the two dense gradient tensors; din is written with row pitch `ld_din` (so it can
// land directly inside the gradient of the packed projection);
// dw [C,K] and dbias [C] are fp32 and must be zeroed by the caller (block-reduced atomics).
template <int KC>
__global__ void __launch_bounds__(256) conv_silu_bwd_kernel(const __nv_bfloat16* __restrict__ in, long long ld_in,
                                                             int c_off, const __nv_bfloat16* __restrict__ w,
                                                             const __nv_bfloat16* __restrict__ bias,
                                                             const __nv_bfloat16* __restrict__ dy1,
                                                             const __nv_bfloat16* __restrict__ dy2,
                                                             __nv_bfloat16* __restrict__ din, long long ld_din,
                                                             float* __restrict__ dw, float* __restrict__ dbias, int Bn,
                                                             int S, int C, int C1, int Krt) {
  const int K = KC > 0 ? KC : Krt;
  __shared__ float red[8][32][2 * (CONV_MAXK + 1)];
  const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5;
  const int cp = blockIdx.x * 32 + lane;
  const int c = cp * 2;
  // each warp walks a run of CONV_RUN tokens in sub-tiles of CONV_TS, so the weight / bias partial sums are reduced (and the
  // atomics issued) once per run instead of once per sub-tile
  const long long tile = blockIdx.y * 8LL + wrp;
  const int tiles_per_seq = (S + CONV_RUN - 1) / CONV_RUN;
  const bool active = c < C && tile < static_cast<long long>(Bn) * tiles_per_seq;
  float2 dwk[CONV_MAXK];
  float2 db = make_float2(0.f, 0.f);
  for (int k = 0; k < CONV_MAXK; ++k) dwk[k] = make_float2(0.f, 0.f);
  if (active) {
    const int b = static_cast<int>(tile / tiles_per_seq);
    const int run0 = static_cast<int>(tile % tiles_per_seq) * CONV_RUN;
    float2 wk[CONV_MAXK];
#pragma unroll
    for (int k = 0; k < K; ++k) wk[k] = make_float2(__bfloat162float(w[c * K + k]), __bfloat162float(w[(c + 1) * K + k]));
    const float2 bs = bias != nullptr ? ld2(bias + c) : make_float2(0.f, 0.f);
    const __nv_bfloat16* ib = in + static_cast<long long>(b) * S * ld_in + c_off + c;
    const bool first = c < C1;
    const __nv_bfloat16* gb = first ? dy1 + static_cast<long long>(b) * S * C1 + c
                                    : dy2 + static_cast<long long>(b) * S * (C - C1) + (c - C1);
    const long long gld = first ? C1 : (C - C1);
    for (int s0 = run0; s0 < min(S, run0 + CONV_RUN); s0 += CONV_TS) {
    // The kernel is latency-bound (each sub-tile's loads are consumed right away): ask L2 for the rows the next sub-tile
    // will add to the window while this one is being computed.
    if (s0 + CONV_TS < min(S, run0 + CONV_RUN)) {
#pragma unroll
      for (int j = 0; j < CONV_TS; ++j) {
        const int sn = s0 + CONV_TS + (K - 1) + j;
        if (sn < S) {
          asm volatile("prefetch.global.L2 [%0];" ::"l"(ib + sn * ld_in));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(gb + sn * gld));
        }
      }
    }
    // inputs s0-(K-1) .. s0+TS+K-2 and dpre for s0 .. s0+TS+K-2
    constexpr int NI = CONV_TS + 2 * (CONV_MAXK - 1);
    float2 xin[NI];
    const int ni = CONV_TS + 2 * (K - 1);
#pragma unroll
    for (int j = 0; j < ni; ++j) {
      const int s = s0 - (K - 1) + j;
      xin[j] = (s >= 0 && s < S) ? ld2(ib + s * ld_in) : make_float2(0.f, 0.f);
    }
    constexpr int ND = CONV_TS + CONV_MAXK - 1;
    float2 dpre[ND];
    const int nd = CONV_TS + K - 1;
#pragma unroll
    for (int j = 0; j < nd; ++j) {
      const int s = s0 + j;
      if (s < S) {
        float2 acc = bs;
    #pragma unroll
#pragma unroll
    for (int k = 0; k < K; ++k) {  // pre[s] uses in[s-K+1+k] = xin[j+k]
          acc.x += wk[k].x * xin[j + k].x;
          acc.y += wk[k].y * xin[j + k].y;
        }
        const float2 g = ld2(gb + s * gld);
        const float sg0 = 1.f / (1.f + __expf(-acc.x)), sg1 = 1.f / (1.f + __expf(-acc.y));
        dpre[j] = make_float2(g.x * sg0 * (1.f + acc.x * (1.f - sg0)), g.y * sg1 * (1.f + acc.y * (1.f - sg1)));
      } else {
        dpre[j] = make_float2(0.f, 0.f);
      }
    }
#pragma unroll
    for (int i = 0; i < CONV_TS; ++i) {
      const int s = s0 + i;
      if (s >= S) break;
      // din[s] = Σ_k w[k] · dpre[s + K-1-k]
      float2 acc = make_float2(0.f, 0.f);
#pragma unroll
      for (int k = 0; k < K; ++k) {
        acc.x += wk[k].x * dpre[i + K - 1 - k].x;
        acc.y += wk[k].y * dpre[i + K - 1 - k].y;
      }
      *reinterpret_cast<__nv_bfloat162*>(din + (static_cast<long long>(b) * S + s) * ld_din + c) = __floats2bfloat162_rn(acc.x, acc.y);
      // this thread's own dpre positions feed dw / dbias exactly once
      db.x += dpre[i].x;
      db.y += dpre[i].y;
#pragma unroll
      for (int k = 0; k < K; ++k) {
        dwk[k].x += dpre[i].x * xin[i + k].x;
        dwk[k].y += dpre[i].y * xin[i + k].y;
      }
    }
    }
  }
#pragma unroll
  for (int k = 0; k < K; ++k) {
    red[wrp][lane][2 * k] = dwk[k].x;
    red[wrp][lane][2 * k + 1] = dwk[k].y;
  }
  red[wrp][lane][2 * K] = db.x;
  red[wrp][lane][2 * K + 1] = db.y;
  __syncthreads();
  if (wrp == 0 && c < C) {
    for (int j = 0; j < 2 * (K + 1); ++j) {
      float t = 0.f;
      for (int q = 0; q < 8; ++q) t += red[q][lane][j];
      const int which = j & 1;
      if (j < 2 * K)
        atomicAdd(&dw[(c + which) * K + (j >> 1)], t);
      else
        atomicAdd(&dbias[c + which], t);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Wide forms for K = 4 taps (the only tap count the models use), taken when channels, offsets and pitches allow 16- / 8-byte
// accesses.  The narrow kernels above issue one 4-byte load per thread and row and are bound by the number of memory
// instructions in flight; here a thread owns 8 (forward) or 4 (backward) channels, loads its rows a batch ahead of the
// arithmetic, and a warp reads 512 / 256 contiguous bytes of a row.
constexpr int CONV_WTS = 16;   // tokens per warp, forward
constexpr int CONV_WRUN = 64;  // tokens per warp, backward

__global__ void __launch_bounds__(256, 2) conv_silu_fwd_w8_kernel(const __nv_bfloat16* __restrict__ in, long long ld_in, int c_off,
                                                                const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ bias,
                                                                __nv_bfloat16* __restrict__ out1, __nv_bfloat16* __restrict__ out2, int Bn, int S,
                                                                int C, int C1) {
  constexpr int K = 4;
  const int c = (blockIdx.x * 32 + (threadIdx.x & 31)) * 8;
  const long long tile = blockIdx.y * 8LL + (threadIdx.x >> 5);
  const int tiles_per_seq = (S + CONV_WTS - 1) / CONV_WTS;
  if (c >= C || tile >= static_cast<long long>(Bn) * tiles_per_seq) return;
  const int b = static_cast<int>(tile / tiles_per_seq);
  const int s0 = static_cast<int>(tile % tiles_per_seq) * CONV_WTS;
  const int s1 = min(S, s0 + CONV_WTS);
  float wk[K][8], bs[8];
  {  // w is [C, K] row-major: the 8 channels' taps are 32 contiguous bf16
    const uint4* wp = reinterpret_cast<const uint4*>(w + static_cast<long long>(c) * K);
    float t[4][8];
#pragma unroll
    for (int i = 0; i < 4; ++i) unpack8_bf16(wp[i], t[i]);
#pragma unroll
    for (int ch = 0; ch < 8; ++ch)
#pragma unroll
      for (int k = 0; k < K; ++k) wk[k][ch] = t[(ch * K + k) >> 3][(ch * K + k) & 7];
    if (bias != nullptr) {
      unpack8_bf16(*reinterpret_cast<const uint4*>(bias + c), bs);
    } else {
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) bs[ch] = 0.f;
    }
  }
  const __nv_bfloat16* ib = in + static_cast<long long>(b) * S * ld_in + c_off + c;
  const bool first = c < C1;
  __nv_bfloat16* ob = first ? out1 + static_cast<long long>(b) * S * C1 + c : out2 + static_cast<long long>(b) * S * (C - C1) + (c - C1);
  const long long old = first ? C1 : (C - C1);
  float win[K][8];      // win[k] = in[s-K+1+k]; slot K-1 is the current row
#pragma unroll
  for (int k = 0; k < K - 1; ++k) {
    const int s = s0 - (K - 1) + k;
    if (s >= 0) {
      unpack8_bf16(*reinterpret_cast<const uint4*>(ib + s * ld_in), win[k + 1]);
    } else {
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) win[k + 1][ch] = 0.f;
    }
  }
  for (int sb = s0; sb < s1; sb += 4) {
    uint4 raw[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (sb + i < s1) raw[i] = *reinterpret_cast<const uint4*>(ib + (sb + i) * ld_in);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int sidx = sb + i;
      if (sidx >= s1) break;
#pragma unroll
      for (int k = 0; k < K - 1; ++k)
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) win[k][ch] = win[k + 1][ch];
      unpack8_bf16(raw[i], win[K - 1]);
      float y[8];
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        float acc = bs[ch];
#pragma unroll
        for (int k = 0; k < K; ++k) acc = fmaf(wk[k][ch], win[k][ch], acc);
        y[ch] = acc / (1.f + __expf(-acc));
      }
      uint4 o;
      o.x = pack_bf16x2(y[0], y[1]); o.y = pack_bf16x2(y[2], y[3]); o.z = pack_bf16x2(y[4], y[5]); o.w = pack_bf16x2(y[6], y[7]);
      *reinterpret_cast<uint4*>(ob + sidx * old) = o;
    }
  }
}

__global__ void __launch_bounds__(256, 2) conv_silu_bwd_w4_kernel(const __nv_bfloat16* __restrict__ in, long long ld_in, int c_off,
                                                                const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ bias,
                                                                const __nv_bfloat16* __restrict__ dy1, const __nv_bfloat16* __restrict__ dy2,
                                                                __nv_bfloat16* __restrict__ din, long long ld_din, float* __restrict__ dw,
                                                                float* __restrict__ dbias, int Bn, int S, int C, int C1) {
  constexpr int K = 4;
  __shared__ float red[8][32][4 * (K + 1) + 1];
  const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5;
  const int c = (blockIdx.x * 32 + lane) * 4;
  const long long tile = blockIdx.y * 8LL + wrp;
  const int tiles_per_seq = (S + CONV_WRUN - 1) / CONV_WRUN;
  const bool active = c < C && tile < static_cast<long long>(Bn) * tiles_per_seq;
  float dwk[K][4], db[4];
#pragma unroll
  for (int ch = 0; ch < 4; ++ch) {
    db[ch] = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) dwk[k][ch] = 0.f;
  }
  if (active) {
    const int b = static_cast<int>(tile / tiles_per_seq);
    const int run0 = static_cast<int>(tile % tiles_per_seq) * CONV_WRUN;
    const int run1 = min(S, run0 + CONV_WRUN);
    float wk[K][4], bs[4];
    {
      const uint2* wp = reinterpret_cast<const uint2*>(w + static_cast<long long>(c) * K);   // 16 contiguous bf16
      float t[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) unpack4_bf16(wp[i], t[i]);
#pragma unroll
      for (int ch = 0; ch < 4; ++ch)
#pragma unroll
        for (int k = 0; k < K; ++k) wk[k][ch] = t[ch][k];
      if (bias != nullptr) {
        unpack4_bf16(*reinterpret_cast<const uint2*>(bias + c), bs);
      } else {
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) bs[ch] = 0.f;
      }
    }
    const __nv_bfloat16* ib = in + static_cast<long long>(b) * S * ld_in + c_off + c;
    const bool first = c < C1;
    const __nv_bfloat16* gb = first ? dy1 + static_cast<long long>(b) * S * C1 + c : dy2 + static_cast<long long>(b) * S * (C - C1) + (c - C1);
    const long long gld = first ? C1 : (C - C1);
    __nv_bfloat16* db_out = din + static_cast<long long>(b) * S * ld_din + c;
    float xwin[K][4], dwin[K][4];      // xwin[k] = in[j-K+1+k], dwin[k] = dpre[j-K+1+k] for the current position j
#pragma unroll
    for (int k = 0; k < K; ++k)
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) dwin[k][ch] = 0.f;
#pragma unroll
    for (int k = 1; k < K; ++k) {
      const int s = run0 - K + k;
      if (s >= 0) {
        unpack4_bf16(*reinterpret_cast<const uint2*>(ib + s * ld_in), xwin[k]);
      } else {
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) xwin[k][ch] = 0.f;
      }
    }
    const int jend = run1 + K - 1;     // dpre of K-1 positions past the run feed the run's last din values
    for (int jb = run0; jb < jend; jb += 4) {
      uint2 rx[4], rg[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int j = jb + i;
        if (j < S && j < jend) {
          rx[i] = *reinterpret_cast<const uint2*>(ib + j * ld_in);
          rg[i] = *reinterpret_cast<const uint2*>(gb + j * gld);
        } else {
          rx[i] = make_uint2(0u, 0u);
          rg[i] = make_uint2(0u, 0u);
        }
      }
      if (jb + 8 < jend) {              // ask L2 for the batch after the next one
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (jb + 8 + i < S) {
            asm volatile("prefetch.global.L2 [%0];" ::"l"(ib + (jb + 8 + i) * ld_in));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(gb + (jb + 8 + i) * gld));
          }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int j = jb + i;
        if (j >= jend) break;
#pragma unroll
        for (int k = 0; k < K - 1; ++k)
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            xwin[k][ch] = xwin[k + 1][ch];
            dwin[k][ch] = dwin[k + 1][ch];
          }
        float g[4];
        unpack4_bf16(rx[i], xwin[K - 1]);
        unpack4_bf16(rg[i], g);
        const bool owned = j < run1;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          float pre = bs[ch];
#pragma unroll
          for (int k = 0; k < K; ++k) pre = fmaf(wk[k][ch], xwin[k][ch], pre);
          const float sg = 1.f / (1.f + __expf(-pre));
          const float d = (j < S) ? g[ch] * sg * (1.f + pre * (1.f - sg)) : 0.f;
          dwin[K - 1][ch] = d;
          if (owned) {
            db[ch] += d;
#pragma unroll
            for (int k = 0; k < K; ++k) dwk[k][ch] = fmaf(d, xwin[k][ch], dwk[k][ch]);
          }
        }
        const int sidx = j - (K - 1);
        if (sidx >= run0) {
          float o[4];
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            float acc = 0.f;
#pragma unroll
            for (int k = 0; k < K; ++k) acc = fmaf(wk[k][ch], dwin[K - 1 - k][ch], acc);
            o[ch] = acc;
          }
          uint2 ov;
          ov.x = pack_bf16x2(o[0], o[1]);
          ov.y = pack_bf16x2(o[2], o[3]);
          *reinterpret_cast<uint2*>(db_out + sidx * ld_din) = ov;
        }
      }
    }
  }
#pragma unroll
  for (int ch = 0; ch < 4; ++ch) {
#pragma unroll
    for (int k = 0; k < K; ++k) red[wrp][lane][ch * (K + 1) + k] = dwk[k][ch];
    red[wrp][lane][ch * (K + 1) + K] = db[ch];
  }
  __syncthreads();
  if (wrp < 4 && c + wrp < C) {        // warp `wrp` finishes channel c + wrp of every lane
    float t[K + 1];
#pragma unroll
    for (int j = 0; j <= K; ++j) {
      float a = 0.f;
      for (int q = 0; q < 8; ++q) a += red[q][lane][wrp * (K + 1) + j];
      t[j] = a;
    }
#pragma unroll
    for (int k = 0; k < K; ++k) atomicAdd(&dw[static_cast<long long>(c + wrp) * K + k], t[k]);
    atomicAdd(&dbias[c + wrp], t[K]);
  }
}

// Rows of `width` bytes between two pitched 2-D buffers (a dense gradient into its columns of a packed one): 16 bytes per
// thread and step when pointers, pitches and width allow, 2 bytes otherwise.
template <typename V>
__global__ void __launch_bounds__(256) copy2d_kernel(const uint8_t* __restrict__ src, long long src_pitch, uint8_t* __restrict__ dst,
                                                     long long dst_pitch, long long rows, int vec_per_row) {
  const long long total = rows * vec_per_row;
  const long long stride = gridDim.x * 256ll;
  for (long long i0 = blockIdx.x * 256ll + threadIdx.x; i0 < total; i0 += 4 * stride) {
    V v[4];
    long long off[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {      // four loads in flight per thread before the first store
      const long long i = i0 + u * stride;
      off[u] = -1;
      if (i < total) {
        const long long r = i / vec_per_row;
        const long long c = (i - r * vec_per_row) * static_cast<long long>(sizeof(V));
        v[u] = *reinterpret_cast<const V*>(src + r * src_pitch + c);
        off[u] = r * dst_pitch + c;
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (off[u] >= 0) *reinterpret_cast<V*>(dst + off[u]) = v[u];
  }
}

}  // namespace cmb

extern "C" int cmb_conv_silu_fwd(const void* in, long long ld_in, int c_off, const void* w, const void* bias, void* out1,
                                 void* out2, int Bn, int S, int C, int C1, int K, void* stream) {
  if (C % 2 || C1 % 2 || c_off % 2 || ld_in % 2 || K > cmb::CONV_MAXK || K < 1) return 1;
  using bf = __nv_bfloat16;
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (K == 4 && C % 8 == 0 && C1 % 8 == 0 && c_off % 8 == 0 && ld_in % 8 == 0 && al16(in) && al16(w) && al16(out1) && al16(out2) &&
      (bias == nullptr || al16(bias))) {
    const long long wt = static_cast<long long>(Bn) * ((S + cmb::CONV_WTS - 1) / cmb::CONV_WTS);
    dim3 wgrid((C / 8 + 31) / 32, static_cast<unsigned>((wt + 7) / 8));
    cmb::conv_silu_fwd_w8_kernel<<<wgrid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const bf*>(in), ld_in, c_off, static_cast<const bf*>(w), static_cast<const bf*>(bias), static_cast<bf*>(out1),
        static_cast<bf*>(out2), Bn, S, C, C1);
    return cudaGetLastError() == cudaSuccess ? 0 : 2;
  }
  const long long tiles = static_cast<long long>(Bn) * ((S + cmb::CONV_TS - 1) / cmb::CONV_TS);
  dim3 grid((C / 2 + 31) / 32, static_cast<unsigned>((tiles + 7) / 8));
  auto kern = K == 4 ? cmb::conv_silu_fwd_kernel<4> : cmb::conv_silu_fwd_kernel<0>;
  kern<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const bf*>(in), ld_in, c_off, static_cast<const bf*>(w),
                                                            static_cast<const bf*>(bias), static_cast<bf*>(out1), static_cast<bf*>(out2), Bn, S, C,
                                                            C1, K);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

extern "C" int cmb_conv_silu_bwd(const void* in, long long ld_in, int c_off, const void* w, const void* bias,
                                 const void* dy1, const void* dy2, void* din, long long ld_din, float* dw, float* dbias, int Bn,
                                 int S, int C, int C1, int K, void* stream) {
  if (C % 2 || C1 % 2 || c_off % 2 || ld_in % 2 || K > cmb::CONV_MAXK || K < 1) return 1;
  using bf = __nv_bfloat16;
  auto al8 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 7) == 0; };
  if (K == 4 && C % 4 == 0 && C1 % 4 == 0 && c_off % 4 == 0 && ld_in % 4 == 0 && ld_din % 4 == 0 && al8(in) && al8(w) && al8(dy1) && al8(dy2) &&
      al8(din) && (bias == nullptr || al8(bias))) {
    const long long wt = static_cast<long long>(Bn) * ((S + cmb::CONV_WRUN - 1) / cmb::CONV_WRUN);
    dim3 wgrid((C / 4 + 31) / 32, static_cast<unsigned>((wt + 7) / 8));
    cmb::conv_silu_bwd_w4_kernel<<<wgrid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const bf*>(in), ld_in, c_off, static_cast<const bf*>(w), static_cast<const bf*>(bias), static_cast<const bf*>(dy1),
        static_cast<const bf*>(dy2), static_cast<bf*>(din), ld_din, dw, dbias, Bn, S, C, C1);
    return cudaGetLastError() == cudaSuccess ? 0 : 2;
  }
  const long long tiles = static_cast<long long>(Bn) * ((S + cmb::CONV_RUN - 1) / cmb::CONV_RUN);
  dim3 grid((C / 2 + 31) / 32, static_cast<unsigned>((tiles + 7) / 8));
  auto kern = K == 4 ? cmb::conv_silu_bwd_kernel<4> : cmb::conv_silu_bwd_kernel<0>;
  kern<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const bf*>(in), ld_in, c_off, static_cast<const bf*>(w),
                                                            static_cast<const bf*>(bias), static_cast<const bf*>(dy1), static_cast<const bf*>(dy2),
                                                            static_cast<bf*>(din), ld_din, dw, dbias, Bn, S, C, C1, K);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// dst[r, 0:width) = src[r, 0:width) for `rows` rows; pitches and width in bytes (width even).
extern "C" int cmb_copy2d(const void* src, long long src_pitch, void* dst, long long dst_pitch, long long rows, long long width,
                          void* stream) {
  if (rows <= 0 || width <= 0) return 0;
  if (width % 2 || src_pitch % 2 || dst_pitch % 2) return 1;
  const auto a = reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) | static_cast<uintptr_t>(src_pitch) |
                 static_cast<uintptr_t>(dst_pitch) | static_cast<uintptr_t>(width);
  const int vb = (a & 15) == 0 ? 16 : 2;
  const long long total = rows * (width / vb);
  const int sms = cmb_host::sm_count_current_device();
  const int grid = static_cast<int>(std::min<long long>((total + 255) / 256, static_cast<long long>(sms) * 16));
  auto st = static_cast<cudaStream_t>(stream);
  if (vb == 16)
    cmb::copy2d_kernel<uint4><<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(src), src_pitch, static_cast<uint8_t*>(dst), dst_pitch, rows,
                                                    static_cast<int>(width / 16));
  else
    cmb::copy2d_kernel<uint16_t><<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(src), src_pitch, static_cast<uint8_t*>(dst), dst_pitch, rows,
                                                       static_cast<int>(width / 2));
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
