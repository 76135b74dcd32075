// M2RNN recurrence with wide value heads (K = 64, V = 128) on tcgen05: forward, and backward with chunk checkpoints + replay.
//
//   z_t = h_{t-1}·W + k_t ⊗ v_t        h ∈ R^{K×V}, W ∈ R^{V×V}
//   h_t = f_t·h_{t-1} + (1 − f_t)·tanh(z_t)
//   y_t = q_t·h_t                       (contracts K)
//
// The per-step product h·W is 64×128×128: tensor-core work, but on the critical path of a nonlinear recurrence, so the
// kernel is organised around that one dependent chain.  One CTA per (batch, head), everything transposed so that thread w
// of 128 owns column w of the state for all 64 rows:
//
//   zᵀ[128 w, 64 k] = Wᵀ·hᵀ   one tcgen05.mma chain per step (A = Wᵀ resident in shared memory, B = the bf16 image of h
//                             that the owning threads rewrite each step; fp32 state stays in registers); the accumulator
//                             comes back with tcgen05.ld (64 columns per thread); tanh, the forget-gate blend and
//                             y_t[w] = Σ_k q_k h[k,w] are thread-local — no cross-thread reduction in the forward pass.
//
// Backward keeps fp32 states only at chunk boundaries (every 64 steps, written by the forward pass).  Per chunk, last to
// first, it replays the forward recurrence from the checkpoint while storing the bf16 operand image of every h_{t-1} into
// a per-CTA scratch ring with bulk copies, then sweeps the chunk in reverse: recompute z_t from that image (same MMA),
// form dz in registers, write dzᵀ once to shared memory and use it twice — as the A operand of dWᵀ += dzᵀ·h_{t-1}
// (accumulated in TMEM over the whole sequence) and, read MN-major, as the B operand of dh_{t-1}ᵀ = f·dhᵀ + W·dzᵀ.  The two
// reductions over V (dq, dk) go through staggered shared-memory atomics, dv is thread-local.
//
// Every mbarrier wait is bounded (sm100.cuh).  Math and layouts of the reference kernels: cppmega_mlx/nn/_tilelang/m2rnn.py:128-248
// (forward), :300-485 (replay + reverse sweep); packed q|k|v input and head mapping cppmega_mlx/nn/_tilelang/m2rnn_path_c.py:726-1064.
#include "sm100.cuh"

namespace cmb {

constexpr int MT_K = 64, MT_V = 128;
constexpr int MT_CHUNK = 32;        // steps staged per input chunk
constexpr int MT_CKPT = 64;         // steps between state checkpoints (two input chunks)
constexpr int MT_TILE = MT_K * MT_V * 2;   // bytes of the bf16 operand image of one state (16 KB)
constexpr int MT_THREADS = 160;     // warps 0-3: one state column each; warp 4: MMA / bulk-copy issuer

struct M2TcParams {
  const __nv_bfloat16 *q, *k, *v;   // token stride s*_s, batch stride s*_b, head slices contiguous (width K / V)
  const float* f;                   // [B,S,nf]
  const float* W;                   // [nw,V,V]
  const float* h0;                  // [B,H,K,V] or null
  __nv_bfloat16* y;                 // [B,S,H,V]
  float* h_last;                    // [B,H,K,V]
  float* ckpt;                      // [B,H,nchk,V,K] fp32 state at the start of every checkpoint interval (null: inference)
  long long sq_b, sq_s, sk_b, sk_s, sv_b, sv_s;
  int B, S, H, nq, nk, nv, nw, nf;
  // backward only
  const __nv_bfloat16* dy;          // [B,S,H,V]
  const float* dh_last;             // [B,H,K,V] or null
  float *dq, *dk, *dv, *df;         // per expanded head: [B,S,H,K] ×2, [B,S,H,V], [B,S,H]
  float* dW;                        // [B,H,V,V]
  float* dh0;                       // [B,H,K,V]
  uint8_t* scratch;                 // [B·H][MT_CKPT][MT_TILE] operand images of h_{t-1} for the chunk being swept
  int* status;
};

__device__ __forceinline__ float mt_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Byte offset of element (row k, column v) in the operand image of h: K-major for the MMA's B operand, two blocks of
// [64 rows × 64 columns], 128-byte rows, 16-byte chunks XOR-swizzled by the row.
__device__ __forceinline__ uint32_t mt_h_off(int k, int v) {
  return static_cast<uint32_t>((v >> 6) * (MT_K * 128) + k * 128 + ((((v & 63) >> 3) ^ (k & 7)) << 4) + (v & 7) * 2);
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* ssrc, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(ssrc)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_load(void* sdst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(sdst)), "l"(gsrc),
               "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

struct MtSmem {
  static constexpr int WT = 0;                         // Wᵀ  K-major [128 w × 128 v] (2 blocks of 16 KB): A of the z product
  static constexpr int WN = WT + 32768;                // W   K-major [128 w' × 128 w]                    : A of the dh product (backward)
  static constexpr int HB = WN + 32768;                // 2 operand images of h (16 KB each)
  static constexpr int DZ = HB + 2 * MT_TILE;          // dzᵀ K-major [128 w × 64 k] (backward)
  static constexpr int IN = DZ + 16384;                // staged inputs of one chunk
  static constexpr int IN_Q = 0, IN_K = MT_CHUNK * MT_K * 2, IN_V = 2 * MT_CHUNK * MT_K * 2, IN_DY = IN_V + MT_CHUNK * MT_V * 2,
                       IN_F = IN_DY + MT_CHUNK * MT_V * 2, IN_BYTES = IN_F + MT_CHUNK * 4;
  static constexpr int RED = IN + IN_BYTES;            // backward: dq / dk / df slots of the chunk [CHUNK][64+64+1(+pad)] fp32
  static constexpr int RED_BYTES = MT_CHUNK * 132 * 4;
  static constexpr int CTL = RED + RED_BYTES;
  static constexpr int TOTAL = CTL + 256 + 1024;
};

// Stage q, k, v (and dy), f of steps [t0, t0+n) into shared memory; all 128 compute threads take part.
__device__ __forceinline__ void mt_stage_inputs(const M2TcParams& p, uint8_t* in, int b, int h, int t0, int n, bool with_dy, int tid) {
  const int hq = h / (p.H / p.nq), hk = h / (p.H / p.nk), hv = h / (p.H / p.nv), hf = h / (p.H / p.nf);
  const __nv_bfloat16* qb = p.q + b * p.sq_b + static_cast<long long>(hq) * MT_K;
  const __nv_bfloat16* kb = p.k + b * p.sk_b + static_cast<long long>(hk) * MT_K;
  const __nv_bfloat16* vb = p.v + b * p.sv_b + static_cast<long long>(hv) * MT_V;
  for (int i = tid; i < n * (MT_K / 8); i += 128) {
    const int tt = i / (MT_K / 8), c = i % (MT_K / 8);
    *reinterpret_cast<uint4*>(in + MtSmem::IN_Q + (tt * MT_K + c * 8) * 2) = *reinterpret_cast<const uint4*>(qb + (t0 + tt) * p.sq_s + c * 8);
    *reinterpret_cast<uint4*>(in + MtSmem::IN_K + (tt * MT_K + c * 8) * 2) = *reinterpret_cast<const uint4*>(kb + (t0 + tt) * p.sk_s + c * 8);
  }
  for (int i = tid; i < n * (MT_V / 8); i += 128) {
    const int tt = i / (MT_V / 8), c = i % (MT_V / 8);
    *reinterpret_cast<uint4*>(in + MtSmem::IN_V + (tt * MT_V + c * 8) * 2) = *reinterpret_cast<const uint4*>(vb + (t0 + tt) * p.sv_s + c * 8);
    if (with_dy)
      *reinterpret_cast<uint4*>(in + MtSmem::IN_DY + (tt * MT_V + c * 8) * 2) =
          *reinterpret_cast<const uint4*>(p.dy + ((static_cast<long long>(b) * p.S + t0 + tt) * p.H + h) * MT_V + c * 8);
  }
  for (int i = tid; i < n; i += 128)
    *reinterpret_cast<float*>(in + MtSmem::IN_F + i * 4) = p.f[(static_cast<long long>(b) * p.S + t0 + i) * p.nf + hf];
}

// W → shared memory as bf16 operand tiles: Wᵀ (rows w, contraction v) and, for the backward pass, W (rows w', contraction w).
__device__ __forceinline__ void mt_load_w(const M2TcParams& p, uint8_t* smem, int h, bool both, int tid) {
  const float* Wg = p.W + static_cast<long long>(h / (p.H / p.nw)) * MT_V * MT_V;
  for (int i = tid; i < MT_V * MT_V; i += 128) {
    const int r = i / MT_V, c = i % MT_V;            // W[r][c]
    const __nv_bfloat16 x = __float2bfloat16(Wg[i]);
    // Wᵀ tile: row = c, contraction = r
    *reinterpret_cast<__nv_bfloat16*>(smem + MtSmem::WT + (r >> 6) * 16384 + c * 128 + ((((r & 63) >> 3) ^ (c & 7)) << 4) + (r & 7) * 2) = x;
    if (both)   // W tile: row = r, contraction = c
      *reinterpret_cast<__nv_bfloat16*>(smem + MtSmem::WN + (c >> 6) * 16384 + r * 128 + ((((c & 63) >> 3) ^ (r & 7)) << 4) + (c & 7) * 2) = x;
  }
}

// zᵀ = Wᵀ · hᵀ: 8 MMAs of 128×64×16 (contraction over the 128 state columns).
__device__ __forceinline__ void mt_issue_z(uint32_t tmem_z, uint32_t wt_addr, uint32_t h_addr) {
  constexpr uint32_t idesc = make_idesc(MT_V, MT_K, 1, 1, 0, 0);
#pragma unroll
  for (int kb = 0; kb < 2; ++kb)
#pragma unroll
    for (int ks = 0; ks < 4; ++ks)
      umma_f16(tmem_z, make_smem_desc_sw128(wt_addr + kb * 16384 + ks * 32, 16, 1024),
               make_smem_desc_sw128(h_addr + kb * (MT_K * 128) + ks * 32, 16, 1024), idesc, (kb > 0 || ks > 0) ? 1u : 0u);
}

// One forward step for the calling thread's column: consumes z (64 accumulator values), updates the fp32 state, returns y.
__device__ __forceinline__ float mt_forward_column(const uint32_t (&z)[64], float (&h)[64], const uint8_t* in, int tt, int w, uint8_t* h_next) {
  const __nv_bfloat16* qs = reinterpret_cast<const __nv_bfloat16*>(in + MtSmem::IN_Q) + tt * MT_K;
  const __nv_bfloat16* ks = reinterpret_cast<const __nv_bfloat16*>(in + MtSmem::IN_K) + tt * MT_K;
  const float vw = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(in + MtSmem::IN_V)[tt * MT_V + w]);
  const float ff = reinterpret_cast<const float*>(in + MtSmem::IN_F)[tt];
  float y = 0.f;
#pragma unroll
  for (int kk = 0; kk < MT_K; kk += 2) {
    const float2 kv2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(ks + kk));
    const float2 qv2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(qs + kk));
    const float c0 = mt_tanh(fmaf(kv2.x, vw, __uint_as_float(z[kk])));
    const float c1 = mt_tanh(fmaf(kv2.y, vw, __uint_as_float(z[kk + 1])));
    h[kk] = fmaf(ff, h[kk] - c0, c0);
    h[kk + 1] = fmaf(ff, h[kk + 1] - c1, c1);
    y = fmaf(qv2.x, h[kk], y);
    y = fmaf(qv2.y, h[kk + 1], y);
    if (h_next != nullptr) {
      *reinterpret_cast<__nv_bfloat16*>(h_next + mt_h_off(kk, w)) = __float2bfloat16(h[kk]);
      *reinterpret_cast<__nv_bfloat16*>(h_next + mt_h_off(kk + 1, w)) = __float2bfloat16(h[kk + 1]);
    }
  }
  return y;
}

// Shared control block.
struct MtCtl {
  uint64_t z_full, h_ready, g_full, dz_ready, tile_full[2];
  uint32_t tmem_slot;
  int abort_flag;
};

// --------------------------------------------------------------------------------------------------------------- forward
__global__ void __launch_bounds__(MT_THREADS, 1) m2rnn_tc_fwd_kernel(const M2TcParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  MtCtl* ctl = reinterpret_cast<MtCtl*>(smem + MtSmem::CTL);
  volatile int* abort_flag = &ctl->abort_flag;
  uint8_t* in = smem + MtSmem::IN;
  const int b = blockIdx.x / p.H, h = blockIdx.x % p.H;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    mbar_init(&ctl->z_full, 1);
    mbar_init(&ctl->h_ready, 128);
    ctl->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 4) {
    tmem_alloc(&ctl->tmem_slot, 64);
    tmem_relinquish();
  }
  float hst[64];
  const long long bh = static_cast<long long>(b) * p.H + h;
  if (warp < 4) {
    mt_load_w(p, smem, h, false, tid);
#pragma unroll
    for (int kk = 0; kk < MT_K; ++kk) {
      hst[kk] = p.h0 != nullptr ? p.h0[(bh * MT_K + kk) * MT_V + tid] : 0.f;
      *reinterpret_cast<__nv_bfloat16*>(smem + MtSmem::HB + mt_h_off(kk, tid)) = __float2bfloat16(hst[kk]);
    }
    fence_proxy_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_z = ctl->tmem_slot;
  const uint32_t wt_addr = smem_u32(smem + MtSmem::WT), hb_addr = smem_u32(smem + MtSmem::HB);

  if (warp == 4) {
    if (lane == 0) {
      for (int t = 0; t < p.S; ++t) {
        // step t reads the image of h_{t-1} in buffer t & 1 (written by the compute threads during step t − 1)
        if (t > 0 && !mbar_wait(&ctl->h_ready, (t - 1) & 1, abort_flag, p.status, ST_TIMEOUT_FULL)) break;
        tc_fence_after();
        mt_issue_z(tmem_z, wt_addr, hb_addr + (t & 1) * MT_TILE);
        umma_commit(&ctl->z_full);
      }
    }
  } else {
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    for (int t0 = 0; t0 < p.S; t0 += MT_CHUNK) {
      const int n = min(MT_CHUNK, p.S - t0);
      named_bar_sync(1, 128);                       // everyone is done with the previous chunk's inputs
      mt_stage_inputs(p, in, b, h, t0, n, false, tid);
      if (p.ckpt != nullptr && t0 % MT_CKPT == 0) {
        float* cp = p.ckpt + ((bh * ((p.S + MT_CKPT - 1) / MT_CKPT) + t0 / MT_CKPT) * MT_V + tid) * MT_K;
#pragma unroll
        for (int kk = 0; kk < MT_K; kk += 4) *reinterpret_cast<float4*>(cp + kk) = make_float4(hst[kk], hst[kk + 1], hst[kk + 2], hst[kk + 3]);
      }
      named_bar_sync(1, 128);
      bool ok = true;
      for (int tt = 0; tt < n; ++tt) {
        const int t = t0 + tt;
        if (!mbar_wait(&ctl->z_full, t & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) {
          ok = false;
          break;
        }
        tc_fence_after();
        uint32_t z[64];
        {
          uint32_t r[32];
          tmem_ld_x32(tmem_z + lane_addr, r);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) z[i] = r[i];
          tmem_ld_x32(tmem_z + lane_addr + 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) z[32 + i] = r[i];
        }
        const float y = mt_forward_column(z, hst, in, tt, tid, smem + MtSmem::HB + ((t + 1) & 1) * MT_TILE);
        p.y[((static_cast<long long>(b) * p.S + t) * p.H + h) * MT_V + tid] = __float2bfloat16(y);
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(&ctl->h_ready);
      }
      if (!ok) break;
    }
#pragma unroll
    for (int kk = 0; kk < MT_K; ++kk) p.h_last[(bh * MT_K + kk) * MT_V + tid] = hst[kk];
  }
  __syncwarp();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_z, 64);
  }
}

// -------------------------------------------------------------------------------------------------------------- backward
// Sum over the 32 lanes of a warp of 32 per-lane values at once: after the call lane j holds Σ_lanes v[j] in v[0]
// (31 shuffles instead of 32 × 5; every register index is static).
__device__ __forceinline__ float mt_transpose_reduce(float (&v)[32], int lane) {
#pragma unroll
  for (int step = 16; step >= 1; step >>= 1) {
    const bool up = (lane & step) != 0;
#pragma unroll
    for (int i = 0; i < step; ++i) {
      const float send = up ? v[i] : v[i + step];
      const float keep = up ? v[i + step] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, step);
    }
  }
  return v[0];
}

// Barrier protocol (each role counts the phases of the barriers it waits on; every phase is waited exactly once per waiter):
//   z_full    issuer → compute   a z product has completed               (replay and sweep: one per step)
//   h_ready   compute → issuer   an operand image of h is in place       (replay: one per step)
//   tile_full bulk load → both   an archived image is back in its buffer (sweep: one per step, alternating buffers)
//   dz_ready  compute → issuer   dzᵀ of the step is in shared memory     (sweep)
//   g_full    issuer → both      the dW and W·dzᵀ products have completed (sweep)
__global__ void __launch_bounds__(MT_THREADS, 1) m2rnn_tc_bwd_kernel(const M2TcParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  MtCtl* ctl = reinterpret_cast<MtCtl*>(smem + MtSmem::CTL);
  volatile int* abort_flag = &ctl->abort_flag;
  uint8_t* in = smem + MtSmem::IN;
  float* red = reinterpret_cast<float*>(smem + MtSmem::RED);     // [CHUNK][132]: dq[0..63], dk[64..127], df[128]
  const int b = blockIdx.x / p.H, h = blockIdx.x % p.H;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long long bh = static_cast<long long>(b) * p.H + h;
  uint8_t* scratch = p.scratch + bh * (static_cast<long long>(MT_CKPT) * MT_TILE);
  if (tid == 0) {
    mbar_init(&ctl->z_full, 1);
    mbar_init(&ctl->h_ready, 128);
    mbar_init(&ctl->g_full, 1);
    mbar_init(&ctl->dz_ready, 128);
    mbar_init(&ctl->tile_full[0], 1);
    mbar_init(&ctl->tile_full[1], 1);
    ctl->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 4) {
    tmem_alloc(&ctl->tmem_slot, 256);
    tmem_relinquish();
  }
  if (warp < 4) mt_load_w(p, smem, h, true, tid);
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_slot;
  const uint32_t tmem_z = tmem_base, tmem_g = tmem_base + 64, tmem_dw = tmem_base + 128;
  const uint32_t wt_addr = smem_u32(smem + MtSmem::WT), wn_addr = smem_u32(smem + MtSmem::WN), hb_addr = smem_u32(smem + MtSmem::HB),
                 dz_addr = smem_u32(smem + MtSmem::DZ);
  const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
  const int nchk = (p.S + MT_CKPT - 1) / MT_CKPT;
  uint32_t ph_z = 0, ph_h = 0, ph_g = 0, ph_dz = 0, ph_tile[2] = {0, 0};
  bool dw_started = false;
  bool ok = true;

  float dh[64];
  if (warp < 4) {
#pragma unroll
    for (int kk = 0; kk < MT_K; ++kk) dh[kk] = p.dh_last != nullptr ? p.dh_last[(bh * MT_K + kk) * MT_V + tid] : 0.f;
  }

  for (int c = nchk - 1; c >= 0 && ok; --c) {
    const int s0 = c * MT_CKPT;
    const int ns = min(MT_CKPT, p.S - s0);
    // ------------------------------------------------------------------------------------------------ replay
    // Steps s0 .. s0+ns-1 forward from the checkpoint; the image of h_{t-1} of step t goes to scratch[t − s0].
    if (warp == 4) {
      if (lane == 0) {
        for (int i = 0; i < ns; ++i) {
          if (!mbar_wait(&ctl->h_ready, ph_h & 1, abort_flag, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          ++ph_h;
          tc_fence_after();
          // the archive copy issued one step ago read the buffer that the compute threads fill during this step: it must be
          // done reading before this step's product (whose completion releases them) is issued
          tma_store_wait_read<0>();
          mt_issue_z(tmem_z, wt_addr, hb_addr + (i & 1) * MT_TILE);
          umma_commit(&ctl->z_full);
          bulk_store(scratch + static_cast<long long>(i) * MT_TILE, smem + MtSmem::HB + (i & 1) * MT_TILE, MT_TILE);
          tma_store_commit();
        }
        tma_store_wait<0>();          // the archive is complete in global memory before the sweep reads it back
      }
    } else {
      float hst[64];
      const float* cp = p.ckpt + ((bh * nchk + c) * MT_V + tid) * MT_K;
#pragma unroll
      for (int kk = 0; kk < MT_K; kk += 4) {
        const float4 v4 = *reinterpret_cast<const float4*>(cp + kk);
        hst[kk] = v4.x; hst[kk + 1] = v4.y; hst[kk + 2] = v4.z; hst[kk + 3] = v4.w;
      }
#pragma unroll
      for (int kk = 0; kk < MT_K; ++kk)
        *reinterpret_cast<__nv_bfloat16*>(smem + MtSmem::HB + mt_h_off(kk, tid)) = __float2bfloat16(hst[kk]);
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&ctl->h_ready);                    // image of h_{s0-1} is in buffer 0
      for (int i0 = 0; i0 < ns && ok; i0 += MT_CHUNK) {
        const int n = min(MT_CHUNK, ns - i0);
        named_bar_sync(1, 128);
        mt_stage_inputs(p, in, b, h, s0 + i0, n, false, tid);
        named_bar_sync(1, 128);
        for (int tt = 0; tt < n; ++tt) {
          const int i = i0 + tt;
          if (!mbar_wait(&ctl->z_full, ph_z & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
          ++ph_z;
          if (i == ns - 1) break;                    // the state after the chunk's last step is not needed by the sweep
          tc_fence_after();
          uint32_t z[64];
          {
            uint32_t r[32];
            tmem_ld_x32(tmem_z + lane_addr, r);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) z[j] = r[j];
            tmem_ld_x32(tmem_z + lane_addr + 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) z[32 + j] = r[j];
          }
          mt_forward_column(z, hst, in, tt, tid, smem + MtSmem::HB + ((i + 1) & 1) * MT_TILE);
          fence_proxy_async_smem();
          tc_fence_before();
          mbar_arrive(&ctl->h_ready);
        }
      }
    }
    ok = __syncthreads_and(ok);                      // products, archive copies and image writes of the replay are all complete
    if (!ok) break;
    // ------------------------------------------------------------------------------------------------ reverse sweep
    if (warp == 4) {
      if (lane == 0) {
        mbar_arrive_expect_tx(&ctl->tile_full[(ns - 1) & 1], MT_TILE);
        bulk_load(smem + MtSmem::HB + ((ns - 1) & 1) * MT_TILE, scratch + static_cast<long long>(ns - 1) * MT_TILE, MT_TILE,
                  &ctl->tile_full[(ns - 1) & 1]);
        for (int i = ns - 1; i >= 0; --i) {
          const int bf = i & 1;
          if (!mbar_wait(&ctl->tile_full[bf], ph_tile[bf] & 1, abort_flag, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          ++ph_tile[bf];
          tc_fence_after();
          mt_issue_z(tmem_z, wt_addr, hb_addr + bf * MT_TILE);       // recompute z_t from the archived h_{t-1}
          umma_commit(&ctl->z_full);
          if (i > 0) {   // the other buffer was last read by step i + 1, whose products completed before its g_full wait returned
            mbar_arrive_expect_tx(&ctl->tile_full[bf ^ 1], MT_TILE);
            bulk_load(smem + MtSmem::HB + (bf ^ 1) * MT_TILE, scratch + static_cast<long long>(i - 1) * MT_TILE, MT_TILE, &ctl->tile_full[bf ^ 1]);
          }
          if (!mbar_wait(&ctl->dz_ready, ph_dz & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
          ++ph_dz;
          tc_fence_after();
          // dWᵀ[w, v] += Σ_k dzᵀ[w, k] · h_{t-1}[k, v]      (A = dzᵀ K-major, B = the image read MN-major)
          constexpr uint32_t idesc_dw = make_idesc(MT_V, MT_V, 1, 1, 0, 1);
#pragma unroll
          for (int ks = 0; ks < MT_K / 16; ++ks)
            umma_f16(tmem_dw, make_smem_desc_sw128(dz_addr + ks * 32, 16, 1024),
                     make_smem_desc_sw128(hb_addr + bf * MT_TILE + ks * 2048, MT_K * 128, 1024), idesc_dw, (dw_started || ks > 0) ? 1u : 0u);
          dw_started = true;
          // Gᵀ[w', k] = Σ_w W[w', w] · dzᵀ[w, k]              (A = W K-major, B = dzᵀ read MN-major)
          constexpr uint32_t idesc_g = make_idesc(MT_V, MT_K, 1, 1, 0, 1);
#pragma unroll
          for (int kb = 0; kb < 2; ++kb)
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              umma_f16(tmem_g, make_smem_desc_sw128(wn_addr + kb * 16384 + ks * 32, 16, 1024),
                       make_smem_desc_sw128(dz_addr + (kb * 4 + ks) * 2048, 16384, 1024), idesc_g, (kb > 0 || ks > 0) ? 1u : 0u);
          umma_commit(&ctl->g_full);
          if (!mbar_wait(&ctl->g_full, ph_g & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
          ++ph_g;
        }
      }
    } else {
      for (int i0 = ((ns - 1) / MT_CHUNK) * MT_CHUNK; i0 >= 0 && ok; i0 -= MT_CHUNK) {
        const int n = min(MT_CHUNK, ns - i0);
        named_bar_sync(1, 128);
        mt_stage_inputs(p, in, b, h, s0 + i0, n, true, tid);
        for (int j = tid; j < n * 132; j += 128) red[j] = 0.f;
        named_bar_sync(1, 128);
        const long long tok0 = static_cast<long long>(b) * p.S + s0 + i0;
        for (int tt = n - 1; tt >= 0; --tt) {
          const int i = i0 + tt;
          const int bf = i & 1;
          const uint8_t* himg = smem + MtSmem::HB + bf * MT_TILE;
          if (!mbar_wait(&ctl->tile_full[bf], ph_tile[bf] & 1, abort_flag, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          ++ph_tile[bf];
          if (!mbar_wait(&ctl->z_full, ph_z & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
          ++ph_z;
          tc_fence_after();
          uint32_t z[64];
          {
            uint32_t r[32];
            tmem_ld_x32(tmem_z + lane_addr, r);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) z[j] = r[j];
            tmem_ld_x32(tmem_z + lane_addr + 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) z[32 + j] = r[j];
          }
          const __nv_bfloat16* qs = reinterpret_cast<const __nv_bfloat16*>(in + MtSmem::IN_Q) + tt * MT_K;
          const __nv_bfloat16* ks_ = reinterpret_cast<const __nv_bfloat16*>(in + MtSmem::IN_K) + tt * MT_K;
          const float vw = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(in + MtSmem::IN_V)[tt * MT_V + tid]);
          const float dyw = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(in + MtSmem::IN_DY)[tt * MT_V + tid]);
          const float ff = reinterpret_cast<const float*>(in + MtSmem::IN_F)[tt];
          float* rq = red + tt * 132;
          float pdf = 0.f, pdv = 0.f;
          uint32_t dzp[32];
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            float rdq[32], rdk[32];
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              float dzv[2];
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const int kk = half * 32 + j + e;
                const float hp = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(himg + mt_h_off(kk, tid)));
                const float kv = __bfloat162float(ks_[kk]);
                const float qv = __bfloat162float(qs[kk]);
                const float cnd = mt_tanh(fmaf(kv, vw, __uint_as_float(z[kk])));
                const float ht = fmaf(ff, hp - cnd, cnd);
                const float d = fmaf(qv, dyw, dh[kk]);            // ∂L/∂h_t including this step's read-out
                pdf = fmaf(d, hp - cnd, pdf);
                const float dzk = (1.f - ff) * d * (1.f - cnd * cnd);
                dzv[e] = dzk;
                pdv = fmaf(dzk, kv, pdv);
                dh[kk] = ff * d;                                  // the W·dz term is added once that product has run
                rdq[j + e] = ht * dyw;
                rdk[j + e] = dzk * vw;
              }
              dzp[(half * 32 + j) >> 1] = pack_bf16x2(dzv[0], dzv[1]);
            }
            // reductions over the 128 state columns: transpose-reduce inside the warp, then one conflict-free atomic per lane
            const float sq_ = mt_transpose_reduce(rdq, lane);
            const float sk_ = mt_transpose_reduce(rdk, lane);
            atomicAdd(&rq[half * 32 + lane], sq_);
            atomicAdd(&rq[64 + half * 32 + lane], sk_);
          }
          p.dv[((tok0 + tt) * p.H + h) * MT_V + tid] = pdv;
          pdf = warp_sum(pdf);
          if (lane == 0) atomicAdd(&rq[128], pdf);
          // dzᵀ row of this column: 64 bf16 = one 128-byte swizzled line
          uint8_t* drow = smem + MtSmem::DZ + tid * 128;
#pragma unroll
          for (int ch = 0; ch < 8; ++ch)
            *reinterpret_cast<uint4*>(drow + ((ch ^ (tid & 7)) << 4)) = make_uint4(dzp[4 * ch], dzp[4 * ch + 1], dzp[4 * ch + 2], dzp[4 * ch + 3]);
          fence_proxy_async_smem();
          tc_fence_before();
          mbar_arrive(&ctl->dz_ready);
          if (!mbar_wait(&ctl->g_full, ph_g & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
          ++ph_g;
          tc_fence_after();
          {
            uint32_t r[32];
            tmem_ld_x32(tmem_g + lane_addr, r);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) dh[j] += __uint_as_float(r[j]);
            tmem_ld_x32(tmem_g + lane_addr + 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) dh[32 + j] += __uint_as_float(r[j]);
          }
          tc_fence_before();
        }
        if (!ok) break;
        named_bar_sync(1, 128);                     // all atomics of the chunk have landed
        for (int j = tid; j < n * MT_K; j += 128) {
          const int tt = j / MT_K, kk = j % MT_K;
          p.dq[((tok0 + tt) * p.H + h) * MT_K + kk] = red[tt * 132 + kk];
          p.dk[((tok0 + tt) * p.H + h) * MT_K + kk] = red[tt * 132 + 64 + kk];
        }
        for (int j = tid; j < n; j += 128) p.df[(tok0 + j) * p.H + h] = red[j * 132 + 128];
      }
    }
    ok = __syncthreads_and(ok);
  }

  if (ok && warp < 4) {
#pragma unroll
    for (int kk = 0; kk < MT_K; ++kk) p.dh0[(bh * MT_K + kk) * MT_V + tid] = dh[kk];
    // dW[v][w] = accumulator[w][v]: thread w writes column w (the accumulator was started by the first sweep step; S ≥ 1)
    tc_fence_after();
    for (int cchunk = 0; cchunk < MT_V / 32; ++cchunk) {
      uint32_t r[32];
      tmem_ld_x32(tmem_dw + lane_addr + cchunk * 32, r);
      tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < 32; ++j) p.dW[(bh * MT_V + cchunk * 32 + j) * MT_V + tid] = __uint_as_float(r[j]);
    }
  }
  __syncwarp();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

}  // namespace cmb

static bool mt_fill(cmb::M2TcParams& p, const int* ip, const long long* lp) {
  p.B = ip[0]; p.S = ip[1]; p.H = ip[2]; p.nq = ip[5]; p.nk = ip[6]; p.nv = ip[7]; p.nw = ip[8]; p.nf = ip[9];
  p.sq_b = lp[0]; p.sq_s = lp[1]; p.sk_b = lp[2]; p.sk_s = lp[3]; p.sv_b = lp[4]; p.sv_s = lp[5];
  if (ip[3] != cmb::MT_K || ip[4] != cmb::MT_V || p.B <= 0 || p.S <= 0 || p.H <= 0) return false;
  for (int n : {p.nq, p.nk, p.nv, p.nw, p.nf})
    if (n <= 0 || p.H % n) return false;
  for (int i = 0; i < 6; ++i)
    if (lp[i] & 7) return false;     // 16-byte vector loads of the head slices
  return true;
}

// Forward for K = 64, V = 128. ip / lp as in cmb_m2rnn_fwd. `ckpt` (fp32 [B,H,ceil(S/64),V,K]) may be null when no backward follows.
extern "C" int cmb_m2rnn_tc_fwd(const void* q, const void* k, const void* v, const float* f, const float* W, const float* h0, void* y,
                                float* h_last, float* ckpt, const int* ip, const long long* lp, int* status, void* stream) {
  cmb::M2TcParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q); p.k = static_cast<const __nv_bfloat16*>(k); p.v = static_cast<const __nv_bfloat16*>(v);
  p.f = f; p.W = W; p.h0 = h0; p.y = static_cast<__nv_bfloat16*>(y); p.h_last = h_last; p.ckpt = ckpt; p.status = status;
  if (!mt_fill(p, ip, lp)) return -1;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15) return -1;
  static std::atomic<unsigned long long> attr_done{0};
  if (cmb_host::set_smem_limit_once_per_device(attr_done, reinterpret_cast<const void*>(cmb::m2rnn_tc_fwd_kernel), cmb::MtSmem::TOTAL)) return -3;
  cmb::m2rnn_tc_fwd_kernel<<<p.B * p.H, cmb::MT_THREADS, cmb::MtSmem::TOTAL, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Backward. `ckpt` from the forward call; `scratch` ≥ B·H·64·16384 bytes (16-byte aligned). Gradients per expanded head as in cmb_m2rnn_bwd.
extern "C" int cmb_m2rnn_tc_bwd(const void* q, const void* k, const void* v, const float* f, const float* W, const float* ckpt, const void* dy,
                                const float* dh_last, float* dq, float* dk, float* dv, float* df, float* dW, float* dh0, void* scratch,
                                const int* ip, const long long* lp, int* status, void* stream) {
  cmb::M2TcParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q); p.k = static_cast<const __nv_bfloat16*>(k); p.v = static_cast<const __nv_bfloat16*>(v);
  p.f = f; p.W = W; p.ckpt = const_cast<float*>(ckpt); p.dy = static_cast<const __nv_bfloat16*>(dy); p.dh_last = dh_last;
  p.dq = dq; p.dk = dk; p.dv = dv; p.df = df; p.dW = dW; p.dh0 = dh0; p.scratch = static_cast<uint8_t*>(scratch); p.status = status;
  if (!mt_fill(p, ip, lp) || ckpt == nullptr || scratch == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(dy) |
       reinterpret_cast<uintptr_t>(scratch)) & 15)
    return -1;
  static std::atomic<unsigned long long> attr_done{0};
  if (cmb_host::set_smem_limit_once_per_device(attr_done, reinterpret_cast<const void*>(cmb::m2rnn_tc_bwd_kernel), cmb::MtSmem::TOTAL)) return -3;
  cmb::m2rnn_tc_bwd_kernel<<<p.B * p.H, cmb::MT_THREADS, cmb::MtSmem::TOTAL, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
