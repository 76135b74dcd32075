// Gated delta rule (GDN: scalar log-decay per head and token; KDA: one per key dimension) as a persistent time loop, forward only:
// the no-gradient path of the V4 linear-attention blocks (prefill of a serving request, evaluation, one-token decode).
//
//   S ← S ⊙ exp(g_t) ;  u_t = β_t (v_t − Sᵀ k_t) ;  S ← S + k_t u_tᵀ ;  o_t = Sᵀ (scale · q_t)          S ∈ R^{K×V} per (batch, head)
//
// One CTA of 256 threads per (batch, value head).  The fp32 state lives in registers: TPC = 256 / V threads share a column v and
// own R = K / TPC consecutive rows of it, so both contractions over K are R fused multiply-adds per thread plus a log2(TPC)-step
// shuffle reduction inside a warp (the TPC threads of a column are adjacent lanes).  The token's q, k, g rows are staged in shared
// memory one token ahead of their use.  Training keeps the chunked WY form (GEMM-shaped, differentiable).
// Recurrence: cppmega_v4/nn/_external/fla_naive_gated_delta_rule.py:41-99, fla_naive_kda.py:38-98; the reference's own kernels for
// it are cppmega_v4/_tilelang/linear_attention_path_b.py:112-195 and kda_path_b.py:112-196.
#include "sm100.cuh"

namespace cmb {

struct DeltaParams {
  const float* q;      // [B,T,H,K]
  const float* k;      // [B,T,H,K]
  const float* v;      // [B,T,HV,D]
  const float* beta;   // [B,T,HV]
  const float* g;      // [B,T,HV] or [B,T,HV,K]
  const float* s0;     // [B,HV,K,D] or null
  float* o;            // [B,T,HV,D]
  float* s_out;        // [B,HV,K,D]
  int B, T, H, HV;
  int g_per_dim;       // 1: KDA
  float scale;
};

template <int K>      // K == V == D
__global__ void __launch_bounds__(256) delta_rule_fwd_kernel(DeltaParams p) {
  constexpr int V = K, TPC = 256 / V, R = K / TPC;
  static_assert(TPC >= 1 && TPC <= 32 && R >= 1 && R * TPC == K, "thread layout");
  __shared__ float sq[2][K], sk[2][K], sg[2][K];
  const int bh = blockIdx.x, b = bh / p.HV, hv = bh % p.HV, h = hv / (p.HV / p.H);
  const int tid = threadIdx.x, v = tid / TPC, r0 = (tid % TPC) * R;
  float S[R];
  const long long sbase = static_cast<long long>(bh) * K * V;
#pragma unroll
  for (int r = 0; r < R; ++r) S[r] = p.s0 != nullptr ? p.s0[sbase + static_cast<long long>(r0 + r) * V + v] : 0.f;
  auto stage = [&](int t, int buf) {
    if (tid < K) {
      const long long qk = ((static_cast<long long>(b) * p.T + t) * p.H + h) * K + tid;
      sq[buf][tid] = p.q[qk] * p.scale;
      sk[buf][tid] = p.k[qk];
      const long long gi = (static_cast<long long>(b) * p.T + t) * p.HV + hv;
      sg[buf][tid] = __expf(p.g_per_dim ? p.g[gi * K + tid] : p.g[gi]);
    }
  };
  if (p.T > 0) stage(0, 0);
  __syncthreads();
  for (int t = 0; t < p.T; ++t) {
    const int buf = t & 1;
    if (t + 1 < p.T) stage(t + 1, buf ^ 1);          // the other buffer was last read two barriers ago
    const long long tv = (static_cast<long long>(b) * p.T + t) * p.HV + hv;
    const float vt = p.v[tv * V + v];
    const float bt = p.beta[tv];
    float dot = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      S[r] *= sg[buf][r0 + r];
      dot = fmaf(S[r], sk[buf][r0 + r], dot);
    }
#pragma unroll
    for (int off = TPC / 2; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
    const float u = bt * (vt - dot);
    float out = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      S[r] = fmaf(sk[buf][r0 + r], u, S[r]);
      out = fmaf(S[r], sq[buf][r0 + r], out);
    }
#pragma unroll
    for (int off = TPC / 2; off > 0; off >>= 1) out += __shfl_xor_sync(0xffffffffu, out, off);
    if ((tid % TPC) == 0) p.o[tv * V + v] = out;
    __syncthreads();                                   // token t + 1 is staged; buffer `buf` is free for token t + 2
  }
#pragma unroll
  for (int r = 0; r < R; ++r) p.s_out[sbase + static_cast<long long>(r0 + r) * V + v] = S[r];
}

}  // namespace cmb

// ip = {B, T, H, HV, K, V, g_per_dim}.  fp32 contiguous tensors; K == V ∈ {16, 32, 64, 128}; HV % H == 0.
extern "C" int cmb_delta_rule_fwd(const float* q, const float* k, const float* v, const float* beta, const float* g, const float* s0, float* o,
                                  float* s_out, const int* ip, float scale, void* stream) {
  cmb::DeltaParams p{q, k, v, beta, g, s0, o, s_out, ip[0], ip[1], ip[2], ip[3], ip[6], scale};
  const int K = ip[4], V = ip[5];
  if (K != V || p.B <= 0 || p.T < 0 || p.H <= 0 || p.HV <= 0 || p.HV % p.H) return 1;
  auto st = static_cast<cudaStream_t>(stream);
  const int grid = p.B * p.HV;
  switch (K) {
    case 16: cmb::delta_rule_fwd_kernel<16><<<grid, 256, 0, st>>>(p); break;
    case 32: cmb::delta_rule_fwd_kernel<32><<<grid, 256, 0, st>>>(p); break;
    case 64: cmb::delta_rule_fwd_kernel<64><<<grid, 256, 0, st>>>(p); break;
    case 128: cmb::delta_rule_fwd_kernel<128><<<grid, 256, 0, st>>>(p); break;
    default: return 1;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
