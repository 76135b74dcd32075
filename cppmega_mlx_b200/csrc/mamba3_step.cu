// One decode step of a Mamba3 mixer (rank-1 B/C) in a single launch: causal depthwise conv + SiLU on the packed
// projection, RMS-norm + bias of B and C, dt / decay / trapezoid terms, phase advance and rotation of B and C, completion of
// the previous token's look-ahead term, state update, read-out, D skip and SiLU(z) gate, and the next cache
// (phase, state, rotated B, x, conv window).  The layer math is that of the sequence path
// (cppmega_mlx/nn/mamba3.py:238 trapezoid, :270 state rotation, :339-408 recurrence, :182-189 decode cache); doing it with
// framework ops takes ~200 tiny launches per layer per token, which is what dominates small-batch decoding.
// One CTA per (head, batch row); everything out of place, so CTAs of one group may read the same previous cache rows.
#include "sm100.cuh"

namespace cmb {

struct M3StepParams {
  const __nv_bfloat16* proj;  // [B, total]: z | x B C | dd_dt dd_A trap angles
  long long ld_proj;
  const __nv_bfloat16* conv_w;     // [C, K]
  const __nv_bfloat16* conv_b;     // [C] or null
  const __nv_bfloat16* conv_prev;  // [B, K-1, C]
  __nv_bfloat16* conv_next;
  const __nv_bfloat16 *dt_bias, *Bw, *Bb, *Cw, *Cb, *D;  // [H], [G,N] ×4, [H]
  const __nv_bfloat16* ang_prev;   // [B,H,R]
  __nv_bfloat16* ang_next;
  const __nv_bfloat16* ssm_prev;   // [B,H,P,N]
  __nv_bfloat16* ssm_next;
  const __nv_bfloat16* k_prev;     // [B,H,N]
  __nv_bfloat16* k_next;
  const __nv_bfloat16* v_prev;     // [B,H,P]
  __nv_bfloat16* v_next;
  __nv_bfloat16* y;                // [B, H·P]
  int H, G, P, N, R, K, d_inner, C;
  float a_floor, eps;
};

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src) {
  const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(__expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x * sigmoid_f(x); }

// conv + SiLU of channel `ch` of row b (current input from proj, history from conv_prev); also forwards the window.
// All taps are loaded before any is used (K ≤ 16), so one call costs one memory latency, not one per tap.
// KC > 0 fixes the kernel width at compile time (the loops below then hold KC taps instead of 16 predicated ones, which is
// what keeps the register count low enough for every CTA of a 32-sequence batch to be resident at once); KC = 0 reads p.K.
template <int KC>
__device__ __forceinline__ float conv_silu_step(const M3StepParams& p, int b, int ch, bool write_window) {
  constexpr int KMAX = KC > 0 ? KC : 16;
  const int K = KC > 0 ? KC : p.K;
  const int hist = K - 1;
  const __nv_bfloat16 cur = p.proj[b * p.ld_proj + p.d_inner + ch];
  const __nv_bfloat16* prev = p.conv_prev + static_cast<long long>(b) * hist * p.C + ch;
  __nv_bfloat16 v[KMAX], w[KMAX];
#pragma unroll
  for (int j = 0; j < KMAX; ++j) {
    if (j < hist) v[j] = prev[static_cast<long long>(j) * p.C];
    if (j < K) w[j] = p.conv_w[ch * K + j];
  }
  float acc = p.conv_b != nullptr ? __bfloat162float(p.conv_b[ch]) : 0.f;
#pragma unroll
  for (int j = 0; j < KMAX; ++j) {
    if (j < hist) {
      acc = fmaf(__bfloat162float(w[j]), __bfloat162float(v[j]), acc);
      if (write_window && j > 0) p.conv_next[(static_cast<long long>(b) * hist + j - 1) * p.C + ch] = v[j];
    }
  }
  acc = fmaf(__bfloat162float(w[hist]), __bfloat162float(cur), acc);
  if (write_window && hist > 0) p.conv_next[(static_cast<long long>(b) * hist + hist - 1) * p.C + ch] = cur;
  return silu_f(acc);
}

// PRE: the CTA's previous state tile (P·N bf16, the one large read) is fetched into shared memory with cp.async at the very
// start, so that its latency overlaps the chain of small dependent loads before the update instead of following it.
template <int KC, bool PRE>
__global__ void __launch_bounds__(128, KC > 0 ? 7 : 2) mamba3_step_kernel(const M3StepParams p) {
  extern __shared__ __align__(16) float sm[];
  float* Bs = sm;             // [N] rotated, scaled B (scan input)
  float* Cr = Bs + p.N;       // [N] rotated C
  float* kp = Cr + p.N;       // [N] previous rotated B · late factor
  float* xs = kp + p.N;       // [P]
  float* vps = xs + p.P;      // [P] previous step's x (the look-ahead term's other factor)
  float* zs = vps + p.P;      // [P] gate input z of this head
  float* red = zs + p.P;      // [16]
  const int h = blockIdx.x, b = blockIdx.y;
  const int hpg = p.H / p.G, g = h / hpg;
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const long long sbase = (static_cast<long long>(b) * p.H + h) * p.P * p.N;
  __nv_bfloat16* stile = reinterpret_cast<__nv_bfloat16*>(sm + ((3 * p.N + 3 * p.P + 16 + 3) & ~3));   // 16-byte aligned
  if (PRE) {
    for (int i = t * 8; i < p.P * p.N; i += 128 * 8) cp_async_16(stile + i, p.ssm_prev + sbase + i);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  const __nv_bfloat16* tail = p.proj + b * p.ld_proj + p.d_inner + p.C;
  const int d_bc = p.G * p.N;
  const long long bh = static_cast<long long>(b) * p.H + h;
  const __nv_bfloat16* ang_in = tail + 3 * p.H;
  const int rr = min(p.R, p.N / 2);

  // ================= stage 1: every global read of the step, issued before the first barrier =================
  // (the stages below only touch shared memory and registers, so a CTA pays for one memory round trip, not for one per stage)
  // per-group scalars: one head per thread, folded over the CTA below (a group can span all heads)
  float scale_g = 0.f, late_g = 0.f;
  for (int i = t; i < hpg; i += 128) {
    const int hh = g * hpg + i;
    const float dth = softplus_f(__bfloat162float(tail[hh]) + __bfloat162float(p.dt_bias[hh]));
    const float sg = sigmoid_f(__bfloat162float(tail[2 * p.H + hh]));
    scale_g += dth * sg;
    late_g += dth * (1.f - sg);
  }
  const float dt_h = softplus_f(__bfloat162float(tail[h]) + __bfloat162float(p.dt_bias[h]));
  const float dt_gh = softplus_f(__bfloat162float(tail[g]) + __bfloat162float(p.dt_bias[g]));   // head index g drives group g's phase
  const float A_h = fminf(-softplus_f(__bfloat162float(tail[p.H + h])), -p.a_floor);
  const float decay = __expf(A_h * dt_h);
  const float Dh = __bfloat162float(p.D[h]);
  // first-iteration operands of the later loops (for N, R ≤ 128 that is all of them), fetched now
  float nw[4] = {0.f, 0.f, 0.f, 0.f}, a_rot = 0.f;
  if (t < p.N) {
    nw[0] = __bfloat162float(p.Bw[g * p.N + t]);
    nw[1] = __bfloat162float(p.Bb[g * p.N + t]);
    nw[2] = __bfloat162float(p.Cw[g * p.N + t]);
    nw[3] = __bfloat162float(p.Cb[g * p.N + t]);
  }
  if (t < rr) a_rot = __bfloat162float(ang_in[t]) * dt_gh + __bfloat162float(p.ang_prev[(static_cast<long long>(b) * p.H + g) * p.R + t]);
  for (int n = t; n < p.N; n += 128) kp[n] = __bfloat162float(p.k_prev[bh * p.N + n]);      // scaled by late_g in stage 4
  for (int i = t; i < p.P; i += 128) {
    vps[i] = __bfloat162float(p.v_prev[bh * p.P + i]);
    zs[i] = __bfloat162float(p.proj[b * p.ld_proj + h * p.P + i]);
  }
  // phase advance of the own head (cache only)
  for (int i = t; i < p.R; i += 128) {
    const float a = __bfloat162float(ang_in[i]) * dt_h + __bfloat162float(p.ang_prev[bh * p.R + i]);
    const float two_pi = 6.283185307179586f;
    p.ang_next[bh * p.R + i] = __float2bfloat16(a - two_pi * floorf(a / two_pi));
  }
  // B and C of this group: conv + SiLU (raw), sums of squares for the RMS norm
  float ssB = 0.f, ssC = 0.f;
  for (int n = t; n < p.N; n += 128) {
    const bool own = (h % hpg) == 0;   // the first head of a group forwards the group's conv window
    const float bv = conv_silu_step<KC>(p, b, p.d_inner + g * p.N + n, own);
    const float cv = conv_silu_step<KC>(p, b, p.d_inner + d_bc + g * p.N + n, own);
    Bs[n] = bv;
    Cr[n] = cv;
    ssB += bv * bv;
    ssC += cv * cv;
  }
  // x of this head: conv + SiLU (and the head's share of the conv window); v cache
  for (int i = t; i < p.P; i += 128) {
    const float xv = conv_silu_step<KC>(p, b, h * p.P + i, true);
    xs[i] = xv;
    p.v_next[bh * p.P + i] = __float2bfloat16(xv);
  }
  scale_g = warp_sum(scale_g);
  late_g = warp_sum(late_g);
  ssB = warp_sum(ssB);
  ssC = warp_sum(ssC);
  if (lane == 0) {
    red[warp] = scale_g;
    red[4 + warp] = late_g;
    red[8 + warp] = ssB;
    red[12 + warp] = ssC;
  }
  __syncthreads();
  // ================= stage 2: norm, weight + bias =================
  scale_g = (red[0] + red[1] + red[2] + red[3]) / hpg;
  late_g = (red[4] + red[5] + red[6] + red[7]) / hpg;
  const float rB = rsqrtf((red[8] + red[9] + red[10] + red[11]) / p.N + p.eps);
  const float rC = rsqrtf((red[12] + red[13] + red[14] + red[15]) / p.N + p.eps);
  for (int n = t; n < p.N; n += 128) {
    const bool first = n == t;
    const float bw = first ? nw[0] : __bfloat162float(p.Bw[g * p.N + n]), bb = first ? nw[1] : __bfloat162float(p.Bb[g * p.N + n]);
    const float cw = first ? nw[2] : __bfloat162float(p.Cw[g * p.N + n]), cb = first ? nw[3] : __bfloat162float(p.Cb[g * p.N + n]);
    Bs[n] = Bs[n] * rB * bw + bb;
    Cr[n] = Cr[n] * rC * cw + cb;
  }
  __syncthreads();
  // ================= stage 3: rotation of B, C by the phase of head index g =================
  for (int i = t; i < rr; i += 128) {
    const float a = i == t ? a_rot
                           : __bfloat162float(ang_in[i]) * dt_gh + __bfloat162float(p.ang_prev[(static_cast<long long>(b) * p.H + g) * p.R + i]);
    float sn, cs;
    __sincosf(a, &sn, &cs);
    const float b0 = Bs[2 * i], b1 = Bs[2 * i + 1], c0 = Cr[2 * i], c1 = Cr[2 * i + 1];
    Bs[2 * i] = b0 * cs - b1 * sn;
    Bs[2 * i + 1] = b0 * sn + b1 * cs;
    Cr[2 * i] = c0 * cs - c1 * sn;
    Cr[2 * i + 1] = c0 * sn + c1 * cs;
  }
  __syncthreads();
  // ================= stage 4: next-step cache of the rotated B, trapezoid scaling =================
  for (int n = t; n < p.N; n += 128) {
    p.k_next[bh * p.N + n] = __float2bfloat16(Bs[n]);   // rotated, not yet trapezoid-scaled: what the next step completes
    kp[n] *= late_g;
    Bs[n] *= scale_g;
  }
  if (PRE) asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();      // stage 4's shared-memory writes, and every thread's pieces of the state tile
  // ---- state update and read-out.  Warp w owns rows p ≡ w (mod 4), sixteen of them per pass; a lane owns two adjacent state
  // columns per 64-column chunk.  The per-column operands live in registers for the whole chunk and the read-out sums in
  // registers for the whole pass (shared-memory accumulators would force every operand to be re-read after each store),
  // so a state element costs one shared-memory read, a handful of FMAs and one global store.
  constexpr int RPW = 16;   // rows per warp and pass
  const __nv_bfloat16* sprev = PRE ? stile : p.ssm_prev + sbase;
  for (int pb = 0; pb < p.P; pb += 4 * RPW) {
    float yacc[RPW];
#pragma unroll
    for (int r = 0; r < RPW; ++r) yacc[r] = 0.f;
    for (int n = lane * 2; n < p.N; n += 64) {
      const float k0 = kp[n], k1 = kp[n + 1], b0 = Bs[n], b1 = Bs[n + 1], c0 = Cr[n], c1 = Cr[n + 1];
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        const int pr = pb + warp + 4 * r;
        if (pr < p.P) {
          const float2 s2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(sprev + pr * p.N + n));
          const float vp = vps[pr], xv = xs[pr];
          const float n0 = decay * (s2.x + vp * k0) + xv * b0;
          const float n1 = decay * (s2.y + vp * k1) + xv * b1;
          *reinterpret_cast<__nv_bfloat162*>(p.ssm_next + sbase + pr * p.N + n) = __floats2bfloat162_rn(n0, n1);
          yacc[r] = fmaf(n0, c0, fmaf(n1, c1, yacc[r]));
        }
      }
    }
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      const int pr = pb + warp + 4 * r;
      const float acc = warp_sum(yacc[r]);
      if (lane == 0 && pr < p.P) p.y[bh * p.P + pr] = __float2bfloat16((acc + Dh * xs[pr]) * silu_f(zs[pr]));
    }
  }
}

}  // namespace cmb

// ip = {B, H, G, P, N, R, K, d_inner, C}; pointers in `pp` in the order of M3StepParams (19 entries; conv_b may be null).
// Requirements: N even, H % G == 0, bf16 everywhere. Returns 1 for an unsupported shape.
extern "C" int cmb_mamba3_step(const void* const* pp, const int* ip, long long ld_proj, float a_floor, float eps, void* stream) {
  cmb::M3StepParams p{};
  const int B = ip[0];
  p.H = ip[1], p.G = ip[2], p.P = ip[3], p.N = ip[4], p.R = ip[5], p.K = ip[6], p.d_inner = ip[7], p.C = ip[8];
  if (B <= 0 || p.H <= 0 || p.G <= 0 || p.H % p.G || p.N % 2 || p.N > 1024 || p.P > 1024 || p.K < 1 || p.K > 16 || B > 65535) return 1;
  auto bf = [&](int i) { return static_cast<const __nv_bfloat16*>(pp[i]); };
  auto bfm = [&](int i) { return static_cast<__nv_bfloat16*>(const_cast<void*>(pp[i])); };
  p.proj = bf(0), p.ld_proj = ld_proj;
  p.conv_w = bf(1), p.conv_b = bf(2), p.conv_prev = bf(3), p.conv_next = bfm(4);
  p.dt_bias = bf(5), p.Bw = bf(6), p.Bb = bf(7), p.Cw = bf(8), p.Cb = bf(9), p.D = bf(10);
  p.ang_prev = bf(11), p.ang_next = bfm(12), p.ssm_prev = bf(13), p.ssm_next = bfm(14);
  p.k_prev = bf(15), p.k_next = bfm(16), p.v_prev = bf(17), p.v_next = bfm(18), p.y = bfm(19);
  p.a_floor = a_floor, p.eps = eps;
  const size_t base = ((3 * p.N + 3 * p.P + 16 + 3) & ~3) * sizeof(float);
  const size_t tile = static_cast<size_t>(p.P) * p.N * sizeof(__nv_bfloat16);
  // the prefetch needs 16-byte pieces (tile size and base pointer) and a tile small enough for seven CTAs per SM
  const bool pre = p.K == 4 && (static_cast<size_t>(p.P) * p.N) % 8 == 0 && (reinterpret_cast<uintptr_t>(pp[13]) & 15) == 0 &&
                   base + tile <= 30 * 1024;
  auto st = static_cast<cudaStream_t>(stream);
  if (pre) cmb::mamba3_step_kernel<4, true><<<dim3(p.H, B), 128, base + tile, st>>>(p);
  else if (p.K == 4) cmb::mamba3_step_kernel<4, false><<<dim3(p.H, B), 128, base, st>>>(p);
  else cmb::mamba3_step_kernel<0, false><<<dim3(p.H, B), 128, base, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
