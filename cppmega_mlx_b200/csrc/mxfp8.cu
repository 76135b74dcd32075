// MXFP8: 1×32 block quantisation (e4m3 data + one e8m0 scale per 32 contiguous elements) and the block-scaled
// GEMM on tcgen05 (`kind::mxf8f6f4.block_scale`), sm_100a.
//
//   quant   : x bf16 [R, C]  →  q e4m3 [R, C],  sf e8m0     scale = 2^ceil(log2(amax/448)), q = rn_sat(x / scale)
//   gemm    : C[M,N] bf16 = Σ_k (A[m,k]·2^(sfa[m,k/32]−127)) · (B[n,k]·2^(sfb[n,k/32]−127))     A: M×K, B: N×K, K-major
//
// Scale factors are stored tiled for the tensor core: the scales of a 128-row × 128-column block (128 rows × 4 k-blocks)
// form one 512-byte atom with byte offset (r%32)·16 + (r/32)·4 + kb, atoms ordered [row block][k block].  One atom is
// exactly what `tcgen05.cp.32x128b.warpx4` moves from shared memory into four TMEM columns, and what one 128-deep
// pipeline stage of the GEMM needs per operand, so the producer fetches it with a single 512-byte bulk copy.
// GEMM structure: persistent CTAs; warp 0 = TMA producer (A tile, B tile, SFA atom, SFB atom per stage), warp 1 = MMA
// issuer (per stage: 2 × tcgen05.cp of the scale atoms, then four 128×128×32 MMAs whose scale byte is picked by the
// sf_id field of the instruction descriptor), warps 2-5 = epilogue (TMEM → bf16 → swizzled staging → TMA store) working
// on the other of two TMEM accumulators.  Every mbarrier wait is bounded and reports through `status`.
//
// Semantics follow `mx.quantize(mode="mxfp8")` as used by cppmega_mlx/nn/_tilelang/sparse_mla_blockscaled.py:60-78 and the
// operand contract of cppmega_mlx/nn/_mxfp8_bridge.py:117-130 (A_u8[M,K], SFA[M,K/32] e8m0, B[N,K], SFB, bf16 out; M,N,K
// multiples of 128 there — here only K must be a multiple of 128).  The reference only wraps an external sm_120 kernel.
#include <cuda_fp8.h>

#include "sm100.cuh"

namespace cmb {

// ------------------------------------------------------------------------------------------- quantisation
__device__ __forceinline__ long long sf_tiled_offset(int r, int kb, int kblocks128) {
  return (static_cast<long long>(r >> 7) * kblocks128 + (kb >> 2)) * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (kb & 3);
}

// Quantise the 8 values of this thread (one quad = one 32-element block) and store data + scale byte.
__device__ __forceinline__ void mxfp8_quant8(const float (&v)[8], bool live, uint8_t* __restrict__ q, long long ldq, uint8_t* __restrict__ sf_tiled,
                                             uint8_t* __restrict__ sf_plain, long long r, int c8, int cols) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  // smallest power of two s with amax / s ≤ 448
  int e = 0;  // unbiased exponent of the scale
  if (amax > 0.f && isfinite(amax)) {
    const float t = amax * (1.f / 448.f);
    const int bits = __float_as_int(t);
    e = ((bits >> 23) & 0xff) - 127 + ((bits & 0x7fffff) ? 1 : 0);
  } else if (amax == 0.f) {
    e = -127;
  }
  e = max(-127, min(127, e));
  const float inv = __int_as_float((127 - e) << 23 | 0);  // 2^-e   (e = 127 → 2^-127 is subnormal: handled below)
  const float invs = (e == 127) ? 5.877471754111438e-39f : ((e == -127) ? 1.7014118346046923e38f : inv);
  if (live) {
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_fp8x2_storage_t p = __nv_cvt_float2_to_fp8x2(make_float2(v[2 * i] * invs, v[2 * i + 1] * invs), __NV_SATFINITE, __NV_E4M3);
      if (i < 2) lo |= static_cast<uint32_t>(p) << (16 * i);
      else hi |= static_cast<uint32_t>(p) << (16 * (i - 2));
    }
    *reinterpret_cast<uint2*>(q + r * ldq + c8 * 8) = make_uint2(lo, hi);
    if ((c8 & 3) == 0) {
      const int kb = c8 >> 2;
      const uint8_t byte = static_cast<uint8_t>(e + 127);
      if (sf_tiled != nullptr) sf_tiled[sf_tiled_offset(static_cast<int>(r), kb, (cols + 127) >> 7)] = byte;
      if (sf_plain != nullptr) sf_plain[r * (cols >> 5) + kb] = byte;
    }
  }
}

// One thread per 8 elements; four threads (one quad) per 32-element block.
__global__ void mxfp8_quant_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ q, long long ldq,
                                   uint8_t* __restrict__ sf_tiled, uint8_t* __restrict__ sf_plain, int rows, int cols) {
  const long long gid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int per_row = cols >> 3;
  const long long r = gid / per_row;
  const int c8 = static_cast<int>(gid % per_row);
  const bool live = r < rows;
  float v[8];
  if (live) {
    unpack8_bf16(*reinterpret_cast<const uint4*>(x + r * ldx + c8 * 8), v);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.f;
  }
  mxfp8_quant8(v, live, q, ldq, sf_tiled, sf_plain, r, c8, cols);
}

// SwiGLU and the quantiser of the following block-scaled product in one pass: gu [rows, 2H] = [gate | up] → y = silu(gate)·up as
// bf16 [rows, H] (kept for the backward pass) and the same values (after the bf16 rounding, so the result is bit-identical to
// quantising y in a second pass) as e4m3 + e8m0 scales.  Saves one read of y per expert layer.
__global__ void swiglu_mxfp8_quant_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ y, uint8_t* __restrict__ q,
                                          uint8_t* __restrict__ sf_tiled, int rows, int H) {
  const long long gid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int per_row = H >> 3;
  const long long r = gid / per_row;
  const int c8 = static_cast<int>(gid % per_row);
  const bool live = r < rows;
  float v[8];
  if (live) {
    float g[8], u[8];
    unpack8_bf16(*reinterpret_cast<const uint4*>(gu + r * 2 * H + c8 * 8), g);
    unpack8_bf16(*reinterpret_cast<const uint4*>(gu + r * 2 * H + H + c8 * 8), u);
    uint4 o;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float a = g[2 * i] / (1.f + __expf(-g[2 * i])) * u[2 * i], b = g[2 * i + 1] / (1.f + __expf(-g[2 * i + 1])) * u[2 * i + 1];
      const __nv_bfloat162 h2 = __floats2bfloat162_rn(a, b);
      ow[i] = *reinterpret_cast<const uint32_t*>(&h2);
      const float2 back = __bfloat1622float2(h2);
      v[2 * i] = back.x;
      v[2 * i + 1] = back.y;
    }
    *reinterpret_cast<uint4*>(y + r * H + c8 * 8) = o;
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.f;
  }
  mxfp8_quant8(v, live, q, H, sf_tiled, nullptr, r, c8, H);
}

__global__ void mxfp8_dequant_kernel(const uint8_t* __restrict__ q, long long ldq, const uint8_t* __restrict__ sf_tiled,
                                     __nv_bfloat16* __restrict__ out, long long ldo, int rows, int cols) {
  const long long gid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long r = gid / cols;
  const int c = static_cast<int>(gid % cols);
  if (r >= rows) return;
  const int e = sf_tiled[sf_tiled_offset(static_cast<int>(r), c >> 5, (cols + 127) >> 7)];
  const __half_raw hr = __nv_cvt_fp8_to_halfraw(q[r * ldq + c], __NV_E4M3);
  out[r * ldo + c] = __float2bfloat16(__half2float(__half(hr)) * exp2f(static_cast<float>(e - 127)));
}

// ------------------------------------------------------------------------------------------- block-scaled GEMM
constexpr int MX_BM = 128;
constexpr int MX_BK = 128;      // fp8 elements = bytes = one 128-byte swizzle line
constexpr int MX_EPI_WARPS = 4;
constexpr int MX_THREADS = 64 + 32 * MX_EPI_WARPS;
constexpr int MX_A_BYTES = MX_BM * MX_BK;
constexpr int MX_SF_BYTES = 512;
constexpr int MX_CBOX_BYTES = 32 * 128;
constexpr int MX_TMEM_COLS = 512;

// BN = 128: two accumulators (the epilogue of one tile overlaps the next tile's mainloop), 6 stages.
// BN = 256: one accumulator (TMEM has 512 columns and the scale factors need some), 4 stages; halves the shared-memory
//           traffic per FLOP, which is what bounds 8-bit MMAs on 128-wide tiles.
template <int BN>
struct MxCfg {
  static constexpr int STAGES = BN == 256 ? 4 : 6;
  static constexpr int NBUF = BN == 256 ? 1 : 2;
  static constexpr int B_BYTES = BN * MX_BK;
  static constexpr int SFB_ATOMS = BN / 128;
  static constexpr int STAGE_BYTES = MX_A_BYTES + B_BYTES + (1 + SFB_ATOMS) * MX_SF_BYTES;
  static constexpr int SF_COLS = 4 * (1 + SFB_ATOMS);     // TMEM columns of scale factors per stage
  static constexpr int TMEM_SF0 = NBUF * BN;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + MX_EPI_WARPS * MX_CBOX_BYTES + 1024 + 256;
  static_assert(TMEM_SF0 + STAGES * SF_COLS <= MX_TMEM_COLS, "TMEM budget");
};

struct MxParams {
  int M, N, K;
  const uint8_t* sfa;   // tiled atoms [ceil(M/128)][K/128][512]
  const uint8_t* sfb;   // tiled atoms [ceil(N/128)][K/128][512]
  int* status;
  const int* tile_group;   // grouped (MoE) mode: expert of each 128-row tile of A / C; B is the experts' weights stacked [E·N, K]
};

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
               "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

template <int BN>
__global__ void __launch_bounds__(MX_THREADS, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmC, const MxParams p) {
  using Cfg = MxCfg<BN>;
  constexpr int MX_STAGES = Cfg::STAGES;
  constexpr int MX_STAGE_BYTES = Cfg::STAGE_BYTES;
  constexpr int MX_B_BYTES = Cfg::B_BYTES;
  constexpr int MX_BN = BN;
  constexpr int NBUF = Cfg::NBUF;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* csmem = smem + MX_STAGES * MX_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(csmem + MX_EPI_WARPS * MX_CBOX_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + MX_STAGES;
  uint64_t* tfull_bar = bars + 2 * MX_STAGES;
  uint64_t* tempty_bar = bars + 2 * MX_STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * MX_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m = (p.M + MX_BM - 1) / MX_BM, num_n = (p.N + MX_BN - 1) / MX_BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = p.K / MX_BK;
  int* status = p.status;

  if (threadIdx.x == 0) {
    for (int s = 0; s < MX_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], MX_EPI_WARPS);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, MX_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int tm = t % num_m, tn = t / num_m;
        // grouped mode: the B rows (and their scale atoms) of this tile start at expert·N
        const int brow0 = (p.tile_group != nullptr ? p.tile_group[tm] * p.N : 0) + tn * MX_BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, status, ST_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * MX_STAGE_BYTES;
          uint8_t* sb = sa + MX_A_BYTES;
          uint8_t* ssfa = sb + MX_B_BYTES;
          uint8_t* ssfb = ssfa + MX_SF_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], MX_STAGE_BYTES);
          tma_load_2d(sa, &tmA, &full_bar[stage], kb * MX_BK, tm * MX_BM);
          tma_load_2d(sb, &tmB, &full_bar[stage], kb * MX_BK, brow0);
          bulk_load(ssfa, p.sfa + (static_cast<long long>(tm) * num_kb + kb) * MX_SF_BYTES, MX_SF_BYTES, &full_bar[stage]);
#pragma unroll
          for (int a = 0; a < Cfg::SFB_ATOMS; ++a)   // a tile past the last row block reads the (zeroed) padding atoms
            bulk_load(ssfb + a * MX_SF_BYTES, p.sfb + (static_cast<long long>(brow0 / 128 + a) * num_kb + kb) * MX_SF_BYTES,
                      MX_SF_BYTES, &full_bar[stage]);
          if (++stage == MX_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int buf = NBUF == 2 ? (local & 1) : 0;
        const uint32_t aphase = NBUF == 2 ? ((local >> 1) & 1) : (local & 1);
        ++local;
        if (!mbar_wait(&tempty_bar[buf], aphase ^ 1, abort_flag, status, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * MX_BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, status, ST_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * MX_STAGE_BYTES);
          const uint32_t sb = sa + MX_A_BYTES;
          const uint32_t ssfa = sb + MX_B_BYTES;
          const uint32_t ssfb = ssfa + MX_SF_BYTES;
          const uint32_t t_sfa = tmem_base + Cfg::TMEM_SF0 + stage * Cfg::SF_COLS;
          const uint32_t t_sfb = t_sfa + 4;
          tmem_cp_32x128b_warpx4(t_sfa, make_smem_desc_noswizzle(ssfa, 16, 128));
#pragma unroll
          for (int a = 0; a < Cfg::SFB_ATOMS; ++a)
            tmem_cp_32x128b_warpx4(t_sfb + 4 * a, make_smem_desc_noswizzle(ssfb + a * MX_SF_BYTES, 16, 128));
#pragma unroll
          for (int k = 0; k < MX_BK / 32; ++k) {
            const uint64_t adesc = make_smem_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t bdesc = make_smem_desc_sw128(sb + k * 32, 16, 1024);
            umma_mxf8(tmem_d, adesc, bdesc, make_idesc_mx(MX_BM, MX_BN, 0, 0, k, k), t_sfa, t_sfb, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == MX_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(&tfull_bar[buf]);
      }
    }
  } else {
    const int ew = warp - 2;
    const int quarter = warp & 3;
    uint8_t* cbox = csmem + ew * MX_CBOX_BYTES;
    int local = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      const int tm = t % num_m, tn = t / num_m;
      const int buf = NBUF == 2 ? (local & 1) : 0;
      const uint32_t aphase = NBUF == 2 ? ((local >> 1) & 1) : (local & 1);
      ++local;
      if (!mbar_wait(&tfull_bar[buf], aphase, abort_flag, status, ST_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after();
      const int row0 = tm * MX_BM + quarter * 32;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * MX_BN;
#pragma unroll 1
      for (int c = 0; c < MX_BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_x32(taddr + c * 32, r);
        tmem_wait_ld();
        if ((c & 1) == 0) {
          if (lane == 0) tma_store_wait_read<0>();
          __syncwarp();
        }
        uint8_t* rowp = cbox + lane * 128;
        const int chbase = (c & 1) * 4;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          uint4 v;
          v.x = pack_bf16x2(__uint_as_float(r[8 * ch]), __uint_as_float(r[8 * ch + 1]));
          v.y = pack_bf16x2(__uint_as_float(r[8 * ch + 2]), __uint_as_float(r[8 * ch + 3]));
          v.z = pack_bf16x2(__uint_as_float(r[8 * ch + 4]), __uint_as_float(r[8 * ch + 5]));
          v.w = pack_bf16x2(__uint_as_float(r[8 * ch + 6]), __uint_as_float(r[8 * ch + 7]));
          *reinterpret_cast<uint4*>(rowp + (((chbase + ch) ^ (lane & 7)) << 4)) = v;
        }
        if ((c & 1) == 1) {
          fence_proxy_async_smem();
          __syncwarp();
          const int bcol0 = tn * MX_BN + (c - 1) * 32;
          if (lane == 0 && row0 < p.M && bcol0 < p.N) {
            tma_store_2d(&tmC, cbox, bcol0, row0);
            tma_store_commit();
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
    }
    if (lane == 0) tma_store_wait<0>();
  }
  __syncwarp();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, MX_TMEM_COLS);
  }
}

}  // namespace cmb

// x bf16 [rows, cols] (pitch ldx) → q e4m3 [rows, cols] (pitch ldq) + scales. cols % 32 == 0. `sf_tiled` must hold
// ceil(rows/128)·ceil(cols/128)·512 bytes (zero it once: rows past `rows` are never written); `sf_plain` [rows, cols/32]
// is optional. Either scale pointer may be null.
extern "C" int cmb_mxfp8_quant(const void* x, long long ldx, void* q, long long ldq, void* sf_tiled, void* sf_plain, int rows, int cols,
                               void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (cols % 32 || ldx % 8 || ldq % 8) return -1;
  const long long threads = static_cast<long long>(rows) * (cols / 8);
  const int block = 256;
  const long long grid = (threads + block - 1) / block;
  if (grid > 0x7fffffffLL) return -3;
  cmb::mxfp8_quant_kernel<<<static_cast<unsigned>(grid), block, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), ldx, static_cast<uint8_t*>(q), ldq, static_cast<uint8_t*>(sf_tiled),
      static_cast<uint8_t*>(sf_plain), rows, cols);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// gu bf16 [rows, 2H] contiguous → y bf16 [rows, H], q e4m3 [rows, H], tiled scales (zeroed once by the caller).  H % 32 == 0.
extern "C" int cmb_swiglu_mxfp8_quant(const void* gu, void* y, void* q, void* sf_tiled, int rows, int H, void* stream) {
  if (rows <= 0 || H <= 0) return 0;
  if (H % 32) return -1;
  const long long threads = static_cast<long long>(rows) * (H / 8);
  const long long grid = (threads + 255) / 256;
  if (grid > 0x7fffffffLL) return -3;
  cmb::swiglu_mxfp8_quant_kernel<<<static_cast<unsigned>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<__nv_bfloat16*>(y), static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf_tiled), rows, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int cmb_mxfp8_dequant(const void* q, long long ldq, const void* sf_tiled, void* out, long long ldo, int rows, int cols,
                                 void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  const long long n = static_cast<long long>(rows) * cols;
  cmb::mxfp8_dequant_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(q), ldq, static_cast<const uint8_t*>(sf_tiled), static_cast<__nv_bfloat16*>(out), ldo, rows, cols);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// C[M,N] bf16 (pitch ldc) = A[M,K] · B[N,K]ᵀ with 1×32 e8m0 block scales in the tiled layout. K % 128 == 0, pitches % 16 == 0.
template <int BN>
static int launch_mx(const void* A, const void* sfa, const void* B, const void* sfb, void* C, int M, int N, int K, long long lda,
                     long long ldb, long long ldc, int* status, int max_ctas, void* stream, const int* tile_group = nullptr, int groups = 1) {
  using Cfg = cmb::MxCfg<BN>;
  CUtensorMap tmA, tmB, tmC;
  int rc = cmb_host::make_tmap_2d(&tmA, A, 1, M, K, lda, cmb::MX_BM, cmb::MX_BK, 128);
  if (rc) return rc;
  rc = cmb_host::make_tmap_2d(&tmB, B, 1, static_cast<uint64_t>(N) * groups, K, ldb, BN, cmb::MX_BK, 128);
  if (rc) return rc + 10000;
  rc = cmb_host::make_tmap_2d(&tmC, C, 2, M, N, ldc, 32, 64, 128);
  if (rc) return rc + 20000;
  static std::atomic<unsigned long long> attr_done{0};
  if (cmb_host::set_smem_limit_once_per_device(attr_done, reinterpret_cast<const void*>(cmb::gemm_mxfp8_kernel<BN>), Cfg::SMEM_BYTES)) return 103;
  const int sms = cmb_host::sm_count_current_device();
  const long long tiles = static_cast<long long>((M + cmb::MX_BM - 1) / cmb::MX_BM) * ((N + BN - 1) / BN);
  int grid = sms;
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (tiles < grid) grid = static_cast<int>(tiles);
  cmb::MxParams p{M, N, K, static_cast<const uint8_t*>(sfa), static_cast<const uint8_t*>(sfb), status, tile_group};
  cmb::gemm_mxfp8_kernel<BN><<<grid, cmb::MX_THREADS, Cfg::SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(tmA, tmB, tmC, p);
  return cudaGetLastError() == cudaSuccess ? 0 : 104;
}

// `bn_hint`: 0 = choose, 128 / 256 = force the tile width.
extern "C" int cmb_gemm_mxfp8(const void* A, const void* sfa, const void* B, const void* sfb, void* C, int M, int N, int K,
                              long long lda, long long ldb, long long ldc, int* status, int max_ctas, int bn_hint, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % cmb::MX_BK) return 110;
  // 256-wide tiles need the B scale atoms of both row blocks of a tile to exist: the scale buffer of B must cover
  // ceil(N/256)·2 row blocks (the quantiser's buffer does when N is padded to 256 by the caller; otherwise use 128).
  const bool wide = N >= 256 && (N % 256 == 0 || bn_hint == 256) && bn_hint != 128;
  return wide ? launch_mx<256>(A, sfa, B, sfb, C, M, N, K, lda, ldb, ldc, status, max_ctas, stream)
              : launch_mx<128>(A, sfa, B, sfb, C, M, N, K, lda, ldb, ldc, status, max_ctas, stream);
}

// Grouped (MoE) form: A [M, K] rows sorted by expert in 128-row aligned segments, `tile_group[i]` = expert of the i-th 128-row
// tile, B = the experts' weights stacked [groups·N, K] (N a multiple of the tile width), scales of B tiled over groups·N rows.
extern "C" int cmb_gemm_mxfp8_grouped(const void* A, const void* sfa, const void* B, const void* sfb, void* C, const int* tile_group,
                                      int groups, int M, int N, int K, long long lda, long long ldb, long long ldc, int* status,
                                      void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || groups <= 0) return 0;
  if (K % cmb::MX_BK || M % 128 || tile_group == nullptr) return 110;
  if (N % 256 == 0) return launch_mx<256>(A, sfa, B, sfb, C, M, N, K, lda, ldb, ldc, status, 0, stream, tile_group, groups);
  if (N % 128 == 0) return launch_mx<128>(A, sfa, B, sfb, C, M, N, K, lda, ldb, ldc, status, 0, stream, tile_group, groups);
  return 111;
}
