// Fused causal attention under an optional key bitmask (the dense form of sparse MLA / DSA), forward pass, on tcgen05.
//
//   O[t] = softmax_s( scale · q[t]·k[s]  |  s ≤ t  ∧  bit s of mask row t ) · v[s]          per (batch, head)
//
// One CTA owns 128 consecutive queries of one (batch, head) and streams the key / value tiles up to its diagonal:
//
//   S   = Q · K_tileᵀ          tcgen05.mma 128×128×16, fp32 in TMEM (two S buffers)
//   P   = exp2(S·c − m)        eight softmax warps read S with tcgen05.ld (a row per thread, half a tile's columns per
//                              warp group), apply mask ∧ causal ∧ range, keep a lazily re-referenced running maximum and
//                              write P as bf16 into shared memory in the MMA's K-major swizzled layout
//   O  += P · V_tile           tcgen05.mma 128×Dv×16 into the resident O accumulator in TMEM (V read MN-major in place)
//
// Neither S nor P ever reaches global memory; the score product is formed once.  The running maximum is only moved when
// a tile exceeds it by 2⁸ (probabilities then stay below 2⁸, well inside bf16 / fp32 range, and numerator and denominator
// share the reference, so the lazy reference is exact up to rounding); O is rescaled in TMEM only then.  Output: O (bf16) and the log-sum-exp per row.
//
// Roles in a 320-thread CTA: warp 0 TMA producer (Q once; K as a ring of [128 keys × 64 columns] blocks so that a
// 192-wide head needs 5 blocks of buffering instead of two whole tiles; V double-buffered), warp 1 issues every MMA,
// warps 2-9 softmax / correction / epilogue.  Every TMA load is a plain per-CTA load; every wait is bounded (sm100.cuh).
//
// Semantics: cppmega_mlx/nn/sparse_mla.py:125-210 (masked softmax over the listed keys in fp32, zeros and lse = −inf for
// a query with no key); kernel counterparts cppmega_mlx/nn/_tilelang/sparse_mla_path_c.py:2135-2260 (one threadgroup per
// (b, s, h), scalar FMAs) and the library SDPA call of cppmega_mlx/nn/attention.py:953-986.
#include <cstring>

#include "sm100.cuh"

namespace cmb {

constexpr int FA_BM = 128;
constexpr int FA_BN = 128;
constexpr int FA_BLK = 128 * 128;   // bytes of one [128 rows × 64 bf16] block
constexpr int FA_THREADS = 320;
constexpr float FA_RESCALE = 8.f;   // log2 units a tile maximum may exceed the reference before O is rescaled

struct FlashParams {
  int B, S, H, Hk;
  float scale_log2;                 // softmax scale · log2(e)
  const unsigned* mask;             // [B, S, mask_words] bit s of row t allows key s; nullptr = causal only
  long long mask_sb;                // words between batches
  int mask_words;
  __nv_bfloat16* out;               // [B, S, H, Dv] with element strides o_sb, o_ss, o_sh
  long long o_sb, o_ss, o_sh;
  float* lse;                       // [B, H, S] natural-log units; +inf for rows without any key (exp(s − lse) = 0)
  int* status;
};

template <int DQB, int DVB>
struct FlashCfg {
  static constexpr int KSLOTS = DQB == 3 ? 5 : 2 * DQB;
  static constexpr int Q_BYTES = DQB * FA_BLK;
  static constexpr int P_BYTES = 2 * FA_BLK;
  static constexpr int K_BYTES = KSLOTS * FA_BLK;
  static constexpr int V_STAGE = DVB * FA_BLK;
  static constexpr int CTL_BYTES = 3072;   // barriers (first 1 KB) + the softmax warps' exchange area (2 KB)
  // No alignment slack: the 192-wide variant uses the whole 227 KB; the dynamic segment is declared 1024-byte aligned and the
  // kernel refuses to run (status word) if the base address ever is not.
  static constexpr int SMEM_BYTES = Q_BYTES + P_BYTES + K_BYTES + 2 * V_STAGE + CTL_BYTES;
  static constexpr int TMEM_COLS = 512;
  static constexpr int O_COL = 256;
};

template <int DQB, int DVB>
__global__ void __launch_bounds__(FA_THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const FlashParams p) {
  using Cfg = FlashCfg<DQB, DVB>;
  constexpr int KSLOTS = Cfg::KSLOTS;
  constexpr int DVH = DVB * 32;      // output columns per softmax thread (half of Dv)
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023u) {   // swizzled TMA / MMA tiles need 1024-byte aligned buffers
    if (threadIdx.x == 0 && p.status != nullptr && atomicCAS(p.status, 0, ST_BAD_ARGUMENT) == 0) p.status[1] = -1024;
    return;
  }
  uint8_t* qs = smem;
  uint8_t* ps = qs + Cfg::Q_BYTES;
  uint8_t* ks = ps + Cfg::P_BYTES;
  uint8_t* vs = ks + Cfg::K_BYTES;
  uint8_t* ctl = vs + 2 * Cfg::V_STAGE;
  uint64_t* q_full = reinterpret_cast<uint64_t*>(ctl);
  uint64_t* k_full = q_full + 1;              // [KSLOTS]
  uint64_t* k_empty = k_full + KSLOTS;        // [KSLOTS]
  uint64_t* v_full = k_empty + KSLOTS;        // [2]
  uint64_t* v_empty = v_full + 2;             // [2]
  uint64_t* s_full = v_empty + 2;             // [2]
  uint64_t* s_free = s_full + 2;              // [2]
  uint64_t* p_full = s_free + 2;
  uint64_t* o_done = p_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* xch = reinterpret_cast<float*>(ctl + 1024);   // [2 tiles parity][2 halves][128 rows] maxima, then row sums

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_qt = (p.S + FA_BM - 1) / FA_BM;
  const int qt = num_qt - 1 - static_cast<int>(blockIdx.x);   // longest rows first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.H / p.Hk);
  const int q0 = qt * FA_BM;
  const int T = min(qt + 1, (p.S + FA_BN - 1) / FA_BN);       // key tiles up to the diagonal
  int* status = p.status;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < KSLOTS; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 256);
    }
    mbar_init(p_full, 256);
    mbar_init(o_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, Cfg::Q_BYTES);
#pragma unroll
      for (int kb = 0; kb < DQB; ++kb) tma_load_4d(qs + kb * FA_BLK, &tmQ, q_full, kb * 64, q0, h, b);
      int n = 0;
      bool ok = true;
      for (int j = 0; j < T && ok; ++j) {
#pragma unroll 1
        for (int kb = 0; kb < DQB; ++kb, ++n) {
          const int slot = n % KSLOTS;
          if (!mbar_wait(&k_empty[slot], ((n / KSLOTS) & 1) ^ 1, abort_flag, status, ST_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&k_full[slot], FA_BLK);
          tma_load_4d(ks + slot * FA_BLK, &tmK, &k_full[slot], kb * 64, j * FA_BN, hk, b);
        }
        if (!ok) break;
        const int st = j & 1;
        if (!mbar_wait(&v_empty[st], ((j >> 1) & 1) ^ 1, abort_flag, status, ST_TIMEOUT_EMPTY)) break;
        mbar_arrive_expect_tx(&v_full[st], Cfg::V_STAGE);
#pragma unroll
        for (int vb = 0; vb < DVB; ++vb)
          tma_load_4d(vs + st * Cfg::V_STAGE + vb * FA_BLK, &tmV, &v_full[st], vb * 64, j * FA_BN, hk, b);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (one thread)
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(FA_BM, FA_BN, 1, 1, 0, 0);
      constexpr uint32_t idesc_o = make_idesc(FA_BM, DVB * 64, 1, 1, 0, 1);
      const uint32_t q_addr = smem_u32(qs), k_addr = smem_u32(ks), p_addr = smem_u32(ps), v_addr = smem_u32(vs);
      int n = 0;
      bool ok = mbar_wait(q_full, 0, abort_flag, status, ST_TIMEOUT_FULL);
      auto issue_s = [&](int j) {
        const int buf = j & 1;
        if (!mbar_wait(&s_free[buf], ((j >> 1) & 1) ^ 1, abort_flag, status, ST_TIMEOUT_TMEM_EMPTY)) return false;
        tc_fence_after();
#pragma unroll 1
        for (int kb = 0; kb < DQB; ++kb, ++n) {
          const int slot = n % KSLOTS;
          if (!mbar_wait(&k_full[slot], (n / KSLOTS) & 1, abort_flag, status, ST_TIMEOUT_FULL)) return false;
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16(tmem_base + buf * FA_BN, make_smem_desc_sw128(q_addr + kb * FA_BLK + k * 32, 16, 1024),
                     make_smem_desc_sw128(k_addr + slot * FA_BLK + k * 32, 16, 1024), idesc_s, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(&k_empty[slot]);
        }
        umma_commit(&s_full[buf]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < T && ok; ++j) {
        if (j + 1 < T && !issue_s(j + 1)) break;
        const int st = j & 1;
        if (!mbar_wait(p_full, j & 1, abort_flag, status, ST_TIMEOUT_TMEM_FULL)) break;
        if (!mbar_wait(&v_full[st], (j >> 1) & 1, abort_flag, status, ST_TIMEOUT_FULL)) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < FA_BN / 16; ++k)
          umma_f16(tmem_base + Cfg::O_COL, make_smem_desc_sw128(p_addr + (k >> 2) * FA_BLK + (k & 3) * 32, 16, 1024),
                   make_smem_desc_sw128(v_addr + st * Cfg::V_STAGE + k * 2048, FA_BLK, 1024), idesc_o, (j > 0 || k > 0) ? 1u : 0u);
        umma_commit(&v_empty[st]);
        umma_commit(o_done);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax / correction / epilogue (8 warps)
    const int quarter = warp & 3;            // TMEM lane quarter this warp may touch
    const int half = (warp - 2) >> 2;        // which 64 keys of a tile (and which half of O's columns)
    const int row = quarter * 32 + lane;
    const int qrow = q0 + row;
    const bool row_ok = qrow < p.S;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const int bar_id = 1 + quarter;          // pairs this warp with the one that owns the other half of the same rows
    const unsigned* mrow = (p.mask != nullptr && row_ok) ? p.mask + b * p.mask_sb + static_cast<long long>(qrow) * p.mask_words : nullptr;
    float m_ref = -INFINITY, l_part = 0.f;
    bool ok = true;
    for (int j = 0; j < T; ++j) {
      const int buf = j & 1;
      const int key0 = j * FA_BN + half * 64;
      // keys of this thread's 64 columns that its row may see
      unsigned bits[2];
#pragma unroll
      for (int w = 0; w < 2; ++w) {
        unsigned bw = 0u;
        const int k0 = key0 + 32 * w;
        if (row_ok && k0 < p.S) {
          bw = 0xffffffffu;
          if (mrow != nullptr) bw = (k0 >> 5) < p.mask_words ? __ldg(mrow + (k0 >> 5)) : 0u;
          const int lim = qrow - k0;           // columns ≤ lim are causal
          if (lim < 0) bw = 0u;
          else if (lim < 31) bw &= (2u << lim) - 1u;
          const int rem = p.S - k0;
          if (rem < 32) bw &= (1u << rem) - 1u;
        }
        bits[w] = bw;
      }
      bool got = mbar_wait(&s_full[buf], (j >> 1) & 1, abort_flag, status, ST_TIMEOUT_TMEM_FULL);
      tc_fence_after();
      // Raw scores stay unscaled: the softmax scale is positive, so the maximum commutes with it and the scaling rides on the
      // exponent's fused multiply-add.  Masking is skipped for warps whose 32 rows see every key of the tile (the common case
      // below the diagonal without a bitmask), which removes a select per element.
      float t[64];
      {
        uint32_t r[32];
        tmem_ld_x32(tmem_base + lane_addr + buf * FA_BN + half * 64, r);
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < 32; ++c) t[c] = __uint_as_float(r[c]);
        tmem_ld_x32(tmem_base + lane_addr + buf * FA_BN + half * 64 + 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < 32; ++c) t[32 + c] = __uint_as_float(r[c]);
      }
      tc_fence_before();
      mbar_arrive(&s_free[buf]);
      if (!__all_sync(0xffffffffu, (bits[0] & bits[1]) == 0xffffffffu)) {
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          t[c] = ((bits[0] >> c) & 1u) ? t[c] : -INFINITY;
          t[32 + c] = ((bits[1] >> c) & 1u) ? t[32 + c] : -INFINITY;
        }
      }
      float lmax;
      {   // eight independent chains: the reduction is latency-bound otherwise (two warps per scheduler cannot hide it)
        float m8[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) m8[i] = t[i];
#pragma unroll
        for (int c = 8; c < 64; ++c) m8[c & 7] = fmaxf(m8[c & 7], t[c]);
        lmax = fmaxf(fmaxf(fmaxf(m8[0], m8[1]), fmaxf(m8[2], m8[3])), fmaxf(fmaxf(m8[4], m8[5]), fmaxf(m8[6], m8[7])));
      }
      lmax *= p.scale_log2;
      float* mx = xch + buf * 256;
      mx[half * 128 + row] = lmax;
      if (!named_bar_and(bar_id, 64, got)) {
        ok = false;
        break;
      }
      const float tile_max = fmaxf(lmax, mx[(half ^ 1) * 128 + row]);
      float alpha = 1.f;
      if (tile_max > m_ref + FA_RESCALE || (m_ref == -INFINITY && tile_max > -INFINITY)) {
        alpha = m_ref == -INFINITY ? 0.f : exp2f(m_ref - tile_max);
        m_ref = tile_max;
        l_part *= alpha;
      }
      // P's buffer and O belong to the previous tile's output MMA until it has completed
      got = j == 0 || mbar_wait(o_done, (j - 1) & 1, abort_flag, status, ST_TIMEOUT_TMEM_EMPTY);
      if (!named_bar_and(bar_id, 64, got)) {
        ok = false;
        break;
      }
      if (j > 0) {
        tc_fence_after();
        if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
          for (int c = 0; c < DVH / 32; ++c) {
            uint32_t o[32];
            const uint32_t ta = tmem_base + lane_addr + Cfg::O_COL + half * DVH + c * 32;
            tmem_ld_x32(ta, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_x32(ta, o);
          }
          tmem_wait_st();
        }
      }
      // P row → shared memory: block `half`, line `row`, eight 16-byte chunks at (chunk ^ (row & 7)).  exp2(−inf) = 0 covers
      // masked keys; a row that has seen no key yet uses 0 as its reference so that −inf − m stays −inf.
      const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;
      uint8_t* prow = ps + half * FA_BLK + row * 128;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        uint32_t w4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float p0 = exp2f(fmaf(t[8 * ch + 2 * i], p.scale_log2, neg_m));
          const float p1 = exp2f(fmaf(t[8 * ch + 2 * i + 1], p.scale_log2, neg_m));
          acc[2 * i] += p0;
          acc[2 * i + 1] += p1;
          w4[i] = pack_bf16x2(p0, p1);
        }
        *reinterpret_cast<uint4*>(prow + ((ch ^ (row & 7)) << 4)) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
      }
      l_part += ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(p_full);
    }
    // ------------------------------------------------------------ epilogue: O / l, lse
    bool got = ok && mbar_wait(o_done, (T - 1) & 1, abort_flag, status, ST_TIMEOUT_TMEM_FULL);
    float* sl = xch;   // row sums of the two halves (the maxima are no longer needed)
    if (got) sl[half * 128 + row] = l_part;
    if (named_bar_and(bar_id, 64, got)) {
      tc_fence_after();
      const float l_tot = l_part + sl[(half ^ 1) * 128 + row];
      const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
      __nv_bfloat16* orow = p.out + b * p.o_sb + static_cast<long long>(qrow) * p.o_ss + h * p.o_sh + half * DVH;
#pragma unroll
      for (int c = 0; c < DVH / 32; ++c) {
        uint32_t o[32];
        tmem_ld_x32(tmem_base + lane_addr + Cfg::O_COL + half * DVH + c * 32, o);
        tmem_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(o[8 * ch]) * inv, __uint_as_float(o[8 * ch + 1]) * inv);
            v.y = pack_bf16x2(__uint_as_float(o[8 * ch + 2]) * inv, __uint_as_float(o[8 * ch + 3]) * inv);
            v.z = pack_bf16x2(__uint_as_float(o[8 * ch + 4]) * inv, __uint_as_float(o[8 * ch + 5]) * inv);
            v.w = pack_bf16x2(__uint_as_float(o[8 * ch + 6]) * inv, __uint_as_float(o[8 * ch + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + ch * 8) = v;
          }
        }
      }
      if (half == 0 && row_ok)
        p.lse[(static_cast<long long>(b) * p.H + h) * p.S + qrow] =
            l_tot > 0.f ? (m_ref + log2f(l_tot)) * 0.6931471805599453f : INFINITY;
    }
  }

  // ---------------------------------------------------------------- teardown
  __syncwarp();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);   // bounded grace period for copies / MMAs still in flight
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace cmb

namespace cmb_host {

// 4-D map over a [B, S, H, D] tensor with unit inner stride: dims (D, S, H, B), box [64 columns × box_rows rows].
int make_tmap_bshd(CUtensorMap* out, const void* base, int D, long long S, int H, int Bn, long long s_row, long long s_head,
                   long long s_batch, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return 101;
  bind_context_once();
  if (reinterpret_cast<uintptr_t>(base) & 15) return 102;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(S), static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(Bn)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(s_row) * 2, static_cast<cuuint64_t>(H > 1 ? s_head : s_row) * 2,
                           static_cast<cuuint64_t>(Bn > 1 ? s_batch : s_row * S) * 2};
  for (int i = 0; i < 3; ++i)
    if (strides[i] == 0 || (strides[i] & 15)) return 105;
  cuuint32_t box[4] = {64, static_cast<cuuint32_t>(box_rows), 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1000 + static_cast<int>(r);
}

}  // namespace cmb_host

namespace {

struct FlashArgs {
  const void *q, *k, *v;
  int B, S, H, Hk, Dq, Dv;
  long long q_sb, q_ss, q_sh, k_sb, k_ss, k_sh, v_sb, v_ss, v_sh;
};

template <int DQB, int DVB>
int launch_flash_fwd(const FlashArgs& a, cmb::FlashParams& p, cudaStream_t stream) {
  using Cfg = cmb::FlashCfg<DQB, DVB>;
  CUtensorMap tmQ, tmK, tmV;
  int rc = cmb_host::make_tmap_bshd(&tmQ, a.q, a.Dq, a.S, a.H, a.B, a.q_ss, a.q_sh, a.q_sb, 128);
  if (rc) return rc;
  rc = cmb_host::make_tmap_bshd(&tmK, a.k, a.Dq, a.S, a.Hk, a.B, a.k_ss, a.k_sh, a.k_sb, 128);
  if (rc) return rc + 10000;
  rc = cmb_host::make_tmap_bshd(&tmV, a.v, a.Dv, a.S, a.Hk, a.B, a.v_ss, a.v_sh, a.v_sb, 128);
  if (rc) return rc + 20000;
  auto kern = cmb::flash_fwd_kernel<DQB, DVB>;
  static std::atomic<unsigned long long> attr_done{0};
  if (cmb_host::set_smem_limit_once_per_device(attr_done, reinterpret_cast<const void*>(kern), Cfg::SMEM_BYTES)) return 103;
  dim3 grid((a.S + cmb::FA_BM - 1) / cmb::FA_BM, a.H, a.B);
  kern<<<grid, cmb::FA_THREADS, Cfg::SMEM_BYTES, stream>>>(tmQ, tmK, tmV, p);
  return cudaGetLastError() == cudaSuccess ? 0 : 104;
}

}  // namespace

// Causal attention under an optional bitmask. q [B,S,H,Dq], k [B,S,Hk,Dq], v [B,S,Hk,Dv] bf16 with unit inner stride;
// ip = {B, S, H, Hk, Dq, Dv, mask_words}; lp = {q_sb, q_ss, q_sh, k_sb, k_ss, k_sh, v_sb, v_ss, v_sh, o_sb, o_ss, o_sh, mask_sb}
// (element / word strides). (Dq, Dv) ∈ {(64,64), (128,128), (192,128)}. Returns 0, 1 for an unsupported shape.
extern "C" int cmb_flash_fwd(const void* q, const void* k, const void* v, const unsigned* mask, void* out, float* lse,
                             const int* ip, const long long* lp, float scale, int* status, void* stream) {
  FlashArgs a{};
  a.q = q; a.k = k; a.v = v;
  a.B = ip[0]; a.S = ip[1]; a.H = ip[2]; a.Hk = ip[3]; a.Dq = ip[4]; a.Dv = ip[5];
  a.q_sb = lp[0]; a.q_ss = lp[1]; a.q_sh = lp[2]; a.k_sb = lp[3]; a.k_ss = lp[4]; a.k_sh = lp[5];
  a.v_sb = lp[6]; a.v_ss = lp[7]; a.v_sh = lp[8];
  if (a.B <= 0 || a.S <= 0 || a.H <= 0 || a.Hk <= 0 || a.H % a.Hk || a.B > 65535 || a.H > 65535 || !(scale > 0.f)) return 1;
  cmb::FlashParams p{};
  p.B = a.B; p.S = a.S; p.H = a.H; p.Hk = a.Hk;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.mask = mask; p.mask_words = ip[6]; p.mask_sb = lp[12];
  p.out = static_cast<__nv_bfloat16*>(out); p.o_sb = lp[9]; p.o_ss = lp[10]; p.o_sh = lp[11];
  p.lse = lse; p.status = status;
  if ((p.o_sb | p.o_ss | p.o_sh) & 7 || (reinterpret_cast<uintptr_t>(out) & 15)) return 1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (a.Dq == 192 && a.Dv == 128) return launch_flash_fwd<3, 2>(a, p, st);
  if (a.Dq == 128 && a.Dv == 128) return launch_flash_fwd<2, 2>(a, p, st);
  if (a.Dq == 64 && a.Dv == 64) return launch_flash_fwd<1, 1>(a, p, st);
  return 1;
}

// =====================================================================================================================
// Backward.  Two launches of one kernel template, neither of which materialises an S×S tensor or uses atomics:
//
//   mode DKV  CTA = 128 keys of one (batch, kv head); loops over the query heads of the group and over 64-query sub-tiles
//             from the diagonal down.  Rows are keys:   Sᵀ = K·Qᵀ,  dPᵀ = V·dOᵀ  →  Pᵀ, dSᵀ (bf16, shared memory)
//             →  dV += Pᵀ·dO,  dK += dSᵀ·Q  accumulate in TMEM over the whole loop (a GQA group is summed on chip).
//   mode DQ   CTA = 128 queries of one (batch, head); loops over 64-key sub-tiles up to the diagonal.  Rows are queries:
//             S = Q·Kᵀ,  dP = dO·Vᵀ  →  dS  →  dQ += dS·K  in TMEM.
//
// with P = exp(scale·S − lse) under mask ∧ causal and dS = P ∘ (dP − δ)·scale, δ = rowsum(dO ∘ O) from a pre-pass.
// The score products are recomputed in both modes (7 tile products instead of the minimal 5); in exchange every output
// tile has exactly one writer.  The streamed sub-tile is the B operand of the score products (K-major) and, read MN-major
// from the same shared-memory tile, of the gradient products.  Math: cppmega_mlx/nn/_tilelang/sparse_mla_path_c.py:2644-2814
// (per-query recompute, ds = p(dp − rowsum), fp32 atomic scatter of dKV there).
namespace cmb {

enum : int { BWD_DQ = 0, BWD_DKV = 1 };
constexpr int FB_SUB = 64;                 // streamed rows per step
constexpr int FB_TBLK = FB_SUB * 128;      // bytes of one streamed [64 rows × 64 bf16] block

struct FlashBwdParams {
  int B, S, H, Hk;
  float scale, scale_log2;
  const unsigned* mask;
  long long mask_sb;
  int mask_words;
  const float* lse;                 // [B, H, S] (natural log, +inf for empty rows)
  const float* delta;               // [B, H, S]
  __nv_bfloat16* out1;              // DQ: dQ [B,S,H,Dq];  DKV: dK [B,S,Hk,Dq]
  long long o1_sb, o1_ss, o1_sh;
  __nv_bfloat16* out2;              // DKV: dV [B,S,Hk,Dv]
  long long o2_sb, o2_ss, o2_sh;
  int* status;
};

template <int DQB, int DVB>
struct FlashBwdCfg {
  static constexpr int R1_BYTES = DQB * FA_BLK, R2_BYTES = DVB * FA_BLK;
  static constexpr int T1_BYTES = DQB * FB_TBLK, T2_BYTES = DVB * FB_TBLK;
  static constexpr int STAGE_BYTES = T1_BYTES + T2_BYTES;
  static constexpr int A_BYTES = FA_BLK;          // one [128 rows × 64 columns] bf16 A tile
  static constexpr int CTL_BYTES = 1024 + 8 * 32 * 16;
  static constexpr int SMEM_BYTES = R1_BYTES + R2_BYTES + 2 * STAGE_BYTES + 2 * A_BYTES + CTL_BYTES + 1024;
  static constexpr int X1_COL = 0, X2_COL = 64, O1_COL = 128, O2_COL = 128 + DQB * 64;
  static constexpr int TMEM_COLS = 512;
};

template <int MODE, int DQB, int DVB>
__global__ void __launch_bounds__(FA_THREADS, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmR1, const __grid_constant__ CUtensorMap tmR2,
                 const __grid_constant__ CUtensorMap tmT1, const __grid_constant__ CUtensorMap tmT2, const FlashBwdParams p) {
  using Cfg = FlashBwdCfg<DQB, DVB>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* r1s = smem;
  uint8_t* r2s = r1s + Cfg::R1_BYTES;
  uint8_t* ts = r2s + Cfg::R2_BYTES;                 // 2 stages of {T1, T2}
  uint8_t* pas = ts + 2 * Cfg::STAGE_BYTES;          // Pᵀ (DKV only)
  uint8_t* dss = pas + Cfg::A_BYTES;                 // dS / dSᵀ
  uint8_t* ctl = dss + Cfg::A_BYTES;
  uint64_t* r_full = reinterpret_cast<uint64_t*>(ctl);
  uint64_t* t_full = r_full + 1;     // [2]
  uint64_t* t_empty = t_full + 2;    // [2]
  uint64_t* x_full = t_empty + 2;
  uint64_t* x_free = x_full + 1;
  uint64_t* a_full = x_free + 1;
  uint64_t* a_free = a_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(a_free + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float4* aux = reinterpret_cast<float4*>(ctl + 1024);   // [8 warps][32 columns] {lse·log2e, δ, mask word, –}

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, b = blockIdx.z;
  const int g = p.H / p.Hk;
  const int row0 = tile * 128;                        // first resident row (query in DQ mode, key in DKV mode)
  const int nsub_all = (p.S + FB_SUB - 1) / FB_SUB;
  // DQ: key sub-tiles 0 .. last one touching the diagonal.  DKV: per head of the group, query sub-tiles from the diagonal on.
  const int sub_first = MODE == BWD_DQ ? 0 : 2 * tile;
  const int sub_count = MODE == BWD_DQ ? min(nsub_all, 2 * tile + 2) : nsub_all - 2 * tile;
  const int heads = MODE == BWD_DQ ? 1 : g;
  const int h_first = MODE == BWD_DQ ? static_cast<int>(blockIdx.y) : static_cast<int>(blockIdx.y) * g;
  const int hk = MODE == BWD_DQ ? static_cast<int>(blockIdx.y) / g : static_cast<int>(blockIdx.y);
  const int NT = heads * sub_count;
  int* status = p.status;

  if (threadIdx.x == 0) {
    mbar_init(r_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&t_full[i], 1);
      mbar_init(&t_empty[i], 1);
    }
    mbar_init(x_full, 1);
    mbar_init(x_free, 256);
    mbar_init(a_full, 256);
    mbar_init(a_free, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmR1);
    tma_prefetch_desc(&tmR2);
    tma_prefetch_desc(&tmT1);
    tma_prefetch_desc(&tmT2);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      const int hr = MODE == BWD_DQ ? h_first : hk;    // head index of the resident operands
      mbar_arrive_expect_tx(r_full, Cfg::R1_BYTES + Cfg::R2_BYTES);
#pragma unroll
      for (int kb = 0; kb < DQB; ++kb) tma_load_4d(r1s + kb * FA_BLK, &tmR1, r_full, kb * 64, row0, hr, b);
#pragma unroll
      for (int kb = 0; kb < DVB; ++kb) tma_load_4d(r2s + kb * FA_BLK, &tmR2, r_full, kb * 64, row0, hr, b);
      for (int n = 0; n < NT; ++n) {
        const int st = n & 1;
        const int ht = MODE == BWD_DQ ? hk : h_first + n / sub_count;   // head index of the streamed operands
        const int t0 = (sub_first + n % sub_count) * FB_SUB;
        if (!mbar_wait(&t_empty[st], ((n >> 1) & 1) ^ 1, abort_flag, status, ST_TIMEOUT_EMPTY)) break;
        uint8_t* t1 = ts + st * Cfg::STAGE_BYTES;
        uint8_t* t2 = t1 + Cfg::T1_BYTES;
        mbar_arrive_expect_tx(&t_full[st], Cfg::STAGE_BYTES);
#pragma unroll
        for (int kb = 0; kb < DQB; ++kb) tma_load_4d(t1 + kb * FB_TBLK, &tmT1, &t_full[st], kb * 64, t0, ht, b);
#pragma unroll
        for (int kb = 0; kb < DVB; ++kb) tma_load_4d(t2 + kb * FB_TBLK, &tmT2, &t_full[st], kb * 64, t0, ht, b);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (one thread)
    if (lane == 0) {
      constexpr uint32_t idesc_x = make_idesc(128, FB_SUB, 1, 1, 0, 0);
      constexpr uint32_t idesc_o1 = make_idesc(128, DQB * 64, 1, 1, 0, 1);
      constexpr uint32_t idesc_o2 = make_idesc(128, DVB * 64, 1, 1, 0, 1);
      const uint32_t r1a = smem_u32(r1s), r2a = smem_u32(r2s), tsa = smem_u32(ts), paa = smem_u32(pas), dsa = smem_u32(dss);
      bool ok = mbar_wait(r_full, 0, abort_flag, status, ST_TIMEOUT_FULL);
      auto issue_scores = [&](int n) {
        const int st = n & 1;
        if (!mbar_wait(&t_full[st], (n >> 1) & 1, abort_flag, status, ST_TIMEOUT_FULL)) return false;
        if (!mbar_wait(x_free, (n & 1) ^ 1, abort_flag, status, ST_TIMEOUT_TMEM_EMPTY)) return false;
        tc_fence_after();
        const uint32_t t1 = tsa + st * Cfg::STAGE_BYTES, t2 = t1 + Cfg::T1_BYTES;
#pragma unroll
        for (int kb = 0; kb < DQB; ++kb)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16(tmem_base + Cfg::X1_COL, make_smem_desc_sw128(r1a + kb * FA_BLK + k * 32, 16, 1024),
                     make_smem_desc_sw128(t1 + kb * FB_TBLK + k * 32, 16, 1024), idesc_x, (kb > 0 || k > 0) ? 1u : 0u);
#pragma unroll
        for (int kb = 0; kb < DVB; ++kb)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16(tmem_base + Cfg::X2_COL, make_smem_desc_sw128(r2a + kb * FA_BLK + k * 32, 16, 1024),
                     make_smem_desc_sw128(t2 + kb * FB_TBLK + k * 32, 16, 1024), idesc_x, (kb > 0 || k > 0) ? 1u : 0u);
        umma_commit(x_full);
        return true;
      };
      if (ok) ok = issue_scores(0);
      for (int n = 0; n < NT && ok; ++n) {
        if (n + 1 < NT && !issue_scores(n + 1)) break;
        if (!mbar_wait(a_full, n & 1, abort_flag, status, ST_TIMEOUT_TMEM_FULL)) break;
        tc_fence_after();
        const int st = n & 1;
        const uint32_t t1 = tsa + st * Cfg::STAGE_BYTES, t2 = t1 + Cfg::T1_BYTES;
#pragma unroll
        for (int k = 0; k < FB_SUB / 16; ++k) {
          if (MODE == BWD_DKV)   // dV += Pᵀ · dO
            umma_f16(tmem_base + Cfg::O2_COL, make_smem_desc_sw128(paa + k * 32, 16, 1024),
                     make_smem_desc_sw128(t2 + k * 2048, FB_TBLK, 1024), idesc_o2, (n > 0 || k > 0) ? 1u : 0u);
          // dK += dSᵀ · Q   or   dQ += dS · K
          umma_f16(tmem_base + Cfg::O1_COL, make_smem_desc_sw128(dsa + k * 32, 16, 1024),
                   make_smem_desc_sw128(t1 + k * 2048, FB_TBLK, 1024), idesc_o1, (n > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&t_empty[st]);
        umma_commit(a_free);
      }
    }
  } else {
    // ---------------------------------------------------------------- P / dS producers and epilogue (8 warps)
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;                  // which 32 of the 64 streamed columns
    const int row = quarter * 32 + lane;
    const int grow = row0 + row;                       // global index of this thread's row (query or key)
    const bool row_ok = grow < p.S;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    float4* my_aux = aux + (warp - 2) * 32;
    const float LOG2E = 1.4426950408889634f;
    float lse2_row = 0.f, delta_row = 0.f;
    const unsigned* mrow = nullptr;
    if (MODE == BWD_DQ) {
      const long long o = (static_cast<long long>(b) * p.H + h_first) * p.S + grow;
      lse2_row = row_ok ? p.lse[o] * LOG2E : INFINITY;
      delta_row = row_ok ? p.delta[o] : 0.f;
      if (p.mask != nullptr && row_ok) mrow = p.mask + b * p.mask_sb + static_cast<long long>(grow) * p.mask_words;
    }
    // Per-step side inputs are fetched one step ahead so that their global-memory latency hides behind the previous step:
    // DQ mode needs this row's mask word for the step's 32 keys; DKV mode needs, per query column, lse, δ and the mask word
    // of this warp's 32 keys (lane c fetches column c; the warp shares them through its private staging row).
    auto fetch = [&](int n, unsigned& word, float4& a) {
      word = 0u;
      a = make_float4(INFINITY, 0.f, __uint_as_float(0u), 0.f);
      if (n >= NT) return;
      const int c0n = (sub_first + n % sub_count) * FB_SUB + half * 32;
      if (MODE == BWD_DQ) {
        if (row_ok && c0n < p.S) {
          word = 0xffffffffu;
          if (mrow != nullptr) word = (c0n >> 5) < p.mask_words ? __ldg(mrow + (c0n >> 5)) : 0u;
        }
      } else {
        const int hq = h_first + n / sub_count;
        const int qc = c0n + lane;
        if (qc < p.S) {
          const long long o = (static_cast<long long>(b) * p.H + hq) * p.S + qc;
          a.x = __ldg(p.lse + o) * LOG2E;
          a.y = __ldg(p.delta + o);
          unsigned w = 0xffffffffu;
          if (p.mask != nullptr) {
            const int wi = (row0 + quarter * 32) >> 5;
            w = wi < p.mask_words ? __ldg(p.mask + b * p.mask_sb + static_cast<long long>(qc) * p.mask_words + wi) : 0u;
          }
          a.z = __uint_as_float(w);
        }
      }
    };
    unsigned word_next;
    float4 aux_next;
    fetch(0, word_next, aux_next);
    for (int n = 0; n < NT; ++n) {
      const int c0 = (sub_first + n % sub_count) * FB_SUB + half * 32;   // global index of this thread's first column
      unsigned bits = word_next;
      if (MODE == BWD_DQ) {
        if (row_ok && c0 < p.S) {
          const int lim = grow - c0;
          if (lim < 0) bits = 0u;
          else if (lim < 31) bits &= (2u << lim) - 1u;
          const int rem = p.S - c0;
          if (rem < 32) bits &= (1u << rem) - 1u;
        }
      } else {
        __syncwarp();            // everyone is done reading the previous step's row
        my_aux[lane] = aux_next;
        __syncwarp();
      }
      fetch(n + 1, word_next, aux_next);
      if (!mbar_wait(x_full, n & 1, abort_flag, status, ST_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after();
      uint32_t x1[32], x2[32];
      tmem_ld_x32(tmem_base + lane_addr + Cfg::X1_COL + half * 32, x1);
      tmem_ld_x32(tmem_base + lane_addr + Cfg::X2_COL + half * 32, x2);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(x_free);
      uint32_t pw[16], dw[16];
#pragma unroll
      for (int c = 0; c < 32; c += 2) {
        float pv[2], dv[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          bool on;
          float l2, dl;
          if (MODE == BWD_DQ) {
            on = (bits >> (c + e)) & 1u;
            l2 = lse2_row;
            dl = delta_row;
          } else {
            const float4 a = my_aux[c + e];
            on = row_ok && ((__float_as_uint(a.z) >> lane) & 1u) && grow <= c0 + c + e;
            l2 = a.x;
            dl = a.y;
          }
          // exp2(x·c − lse): an empty row has lse = +inf and yields 0; the softmax scale rides on the fused multiply-add
          const float pe = on ? exp2f(fmaf(__uint_as_float(x1[c + e]), p.scale_log2, -l2)) : 0.f;
          pv[e] = pe;
          dv[e] = (pe * p.scale) * (__uint_as_float(x2[c + e]) - dl);
        }
        pw[c >> 1] = pack_bf16x2(pv[0], pv[1]);
        dw[c >> 1] = pack_bf16x2(dv[0], dv[1]);
      }
      // the gradient MMAs of the previous step still read the A tiles until their commit arrives
      if (!mbar_wait(a_free, (n & 1) ^ 1, abort_flag, status, ST_TIMEOUT_TMEM_EMPTY)) break;
      uint8_t* prow = pas + row * 128;
      uint8_t* drow = dss + row * 128;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        const int sw = ((half * 4 + ch) ^ (row & 7)) << 4;
        if (MODE == BWD_DKV) *reinterpret_cast<uint4*>(prow + sw) = make_uint4(pw[4 * ch], pw[4 * ch + 1], pw[4 * ch + 2], pw[4 * ch + 3]);
        *reinterpret_cast<uint4*>(drow + sw) = make_uint4(dw[4 * ch], dw[4 * ch + 1], dw[4 * ch + 2], dw[4 * ch + 3]);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(a_full);
    }
    // ------------------------------------------------------------ epilogue: accumulators → bf16 rows
    if (mbar_wait(a_free, (NT - 1) & 1, abort_flag, status, ST_TIMEOUT_TMEM_FULL)) {
      tc_fence_after();
      const int ho = MODE == BWD_DQ ? h_first : hk;
      __nv_bfloat16* o1 = p.out1 + b * p.o1_sb + static_cast<long long>(grow) * p.o1_ss + ho * p.o1_sh + half * (DQB * 32);
#pragma unroll
      for (int c = 0; c < DQB; ++c) {
        uint32_t o[32];
        tmem_ld_x32(tmem_base + lane_addr + Cfg::O1_COL + half * (DQB * 32) + c * 32, o);
        tmem_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int ch = 0; ch < 4; ++ch)
            *reinterpret_cast<uint4*>(o1 + c * 32 + ch * 8) =
                make_uint4(pack_bf16x2(__uint_as_float(o[8 * ch]), __uint_as_float(o[8 * ch + 1])),
                           pack_bf16x2(__uint_as_float(o[8 * ch + 2]), __uint_as_float(o[8 * ch + 3])),
                           pack_bf16x2(__uint_as_float(o[8 * ch + 4]), __uint_as_float(o[8 * ch + 5])),
                           pack_bf16x2(__uint_as_float(o[8 * ch + 6]), __uint_as_float(o[8 * ch + 7])));
        }
      }
      if (MODE == BWD_DKV) {
        __nv_bfloat16* o2 = p.out2 + b * p.o2_sb + static_cast<long long>(grow) * p.o2_ss + ho * p.o2_sh + half * (DVB * 32);
#pragma unroll
        for (int c = 0; c < DVB; ++c) {
          uint32_t o[32];
          tmem_ld_x32(tmem_base + lane_addr + Cfg::O2_COL + half * (DVB * 32) + c * 32, o);
          tmem_wait_ld();
          if (row_ok) {
#pragma unroll
            for (int ch = 0; ch < 4; ++ch)
              *reinterpret_cast<uint4*>(o2 + c * 32 + ch * 8) =
                  make_uint4(pack_bf16x2(__uint_as_float(o[8 * ch]), __uint_as_float(o[8 * ch + 1])),
                             pack_bf16x2(__uint_as_float(o[8 * ch + 2]), __uint_as_float(o[8 * ch + 3])),
                             pack_bf16x2(__uint_as_float(o[8 * ch + 4]), __uint_as_float(o[8 * ch + 5])),
                             pack_bf16x2(__uint_as_float(o[8 * ch + 6]), __uint_as_float(o[8 * ch + 7])));
          }
        }
      }
    }
  }

  __syncwarp();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace cmb

namespace {

template <int MODE, int DQB, int DVB>
int launch_flash_bwd(const FlashArgs& a, const void* dO, long long do_sb, long long do_ss, long long do_sh, cmb::FlashBwdParams& p,
                     cudaStream_t stream) {
  using Cfg = cmb::FlashBwdCfg<DQB, DVB>;
  CUtensorMap tmR1, tmR2, tmT1, tmT2;
  int rc;
  const int rq = MODE == cmb::BWD_DQ ? 128 : cmb::FB_SUB;    // box rows of the query-side maps
  const int rk = MODE == cmb::BWD_DQ ? cmb::FB_SUB : 128;    // box rows of the key-side maps
  CUtensorMap tmQ, tmDO, tmK, tmV;
  rc = cmb_host::make_tmap_bshd(&tmQ, a.q, a.Dq, a.S, a.H, a.B, a.q_ss, a.q_sh, a.q_sb, rq);
  if (rc) return rc;
  rc = cmb_host::make_tmap_bshd(&tmDO, dO, a.Dv, a.S, a.H, a.B, do_ss, do_sh, do_sb, rq);
  if (rc) return rc + 10000;
  rc = cmb_host::make_tmap_bshd(&tmK, a.k, a.Dq, a.S, a.Hk, a.B, a.k_ss, a.k_sh, a.k_sb, rk);
  if (rc) return rc + 20000;
  rc = cmb_host::make_tmap_bshd(&tmV, a.v, a.Dv, a.S, a.Hk, a.B, a.v_ss, a.v_sh, a.v_sb, rk);
  if (rc) return rc + 30000;
  if (MODE == cmb::BWD_DQ) { tmR1 = tmQ; tmR2 = tmDO; tmT1 = tmK; tmT2 = tmV; }
  else { tmR1 = tmK; tmR2 = tmV; tmT1 = tmQ; tmT2 = tmDO; }
  auto kern = cmb::flash_bwd_kernel<MODE, DQB, DVB>;
  static std::atomic<unsigned long long> attr_done{0};
  if (cmb_host::set_smem_limit_once_per_device(attr_done, reinterpret_cast<const void*>(kern), Cfg::SMEM_BYTES)) return 103;
  dim3 grid((a.S + 127) / 128, MODE == cmb::BWD_DQ ? a.H : a.Hk, a.B);
  kern<<<grid, cmb::FA_THREADS, Cfg::SMEM_BYTES, stream>>>(tmR1, tmR2, tmT1, tmT2, p);
  return cudaGetLastError() == cudaSuccess ? 0 : 104;
}

template <int DQB, int DVB>
int flash_bwd_both(const FlashArgs& a, const void* dO, const long long* lp, cmb::FlashBwdParams p, void* dq, void* dk, void* dv,
                   cudaStream_t st) {
  cmb::FlashBwdParams pk = p;
  pk.out1 = static_cast<__nv_bfloat16*>(dk); pk.o1_sb = lp[15]; pk.o1_ss = lp[16]; pk.o1_sh = lp[17];
  pk.out2 = static_cast<__nv_bfloat16*>(dv); pk.o2_sb = lp[18]; pk.o2_ss = lp[19]; pk.o2_sh = lp[20];
  int rc = launch_flash_bwd<cmb::BWD_DKV, DQB, DVB>(a, dO, lp[9], lp[10], lp[11], pk, st);
  if (rc) return rc;
  cmb::FlashBwdParams pq = p;
  pq.out1 = static_cast<__nv_bfloat16*>(dq); pq.o1_sb = lp[12]; pq.o1_ss = lp[13]; pq.o1_sh = lp[14];
  rc = launch_flash_bwd<cmb::BWD_DQ, DQB, DVB>(a, dO, lp[9], lp[10], lp[11], pq, st);
  return rc ? rc + 50000 : 0;
}

}  // namespace

// Backward of cmb_flash_fwd. dO [B,S,H,Dv]; lse, delta [B,H,S] fp32 (delta = rowsum(dO ∘ O)); outputs dQ [B,S,H,Dq],
// dK [B,S,Hk,Dq], dV [B,S,Hk,Dv] bf16 (every element written). ip as in cmb_flash_fwd; lp = {q_sb,q_ss,q_sh, k_sb,k_ss,k_sh,
// v_sb,v_ss,v_sh, do_sb,do_ss,do_sh, dq_sb,dq_ss,dq_sh, dk_sb,dk_ss,dk_sh, dv_sb,dv_ss,dv_sh, mask_sb}.
extern "C" int cmb_flash_bwd(const void* q, const void* k, const void* v, const void* dO, const unsigned* mask, const float* lse,
                             const float* delta, void* dq, void* dk, void* dv, const int* ip, const long long* lp, float scale,
                             int* status, void* stream) {
  FlashArgs a{};
  a.q = q; a.k = k; a.v = v;
  a.B = ip[0]; a.S = ip[1]; a.H = ip[2]; a.Hk = ip[3]; a.Dq = ip[4]; a.Dv = ip[5];
  a.q_sb = lp[0]; a.q_ss = lp[1]; a.q_sh = lp[2]; a.k_sb = lp[3]; a.k_ss = lp[4]; a.k_sh = lp[5];
  a.v_sb = lp[6]; a.v_ss = lp[7]; a.v_sh = lp[8];
  if (a.B <= 0 || a.S <= 0 || a.H <= 0 || a.Hk <= 0 || a.H % a.Hk || a.B > 65535 || a.H > 65535 || !(scale > 0.f)) return 1;
  for (int i = 12; i < 21; ++i)
    if (lp[i] & 7) return 1;
  if ((reinterpret_cast<uintptr_t>(dq) | reinterpret_cast<uintptr_t>(dk) | reinterpret_cast<uintptr_t>(dv)) & 15) return 1;
  cmb::FlashBwdParams p{};
  p.B = a.B; p.S = a.S; p.H = a.H; p.Hk = a.Hk;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.mask = mask; p.mask_words = ip[6]; p.mask_sb = lp[21];
  p.lse = lse; p.delta = delta; p.status = status;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (a.Dq == 192 && a.Dv == 128) return flash_bwd_both<3, 2>(a, dO, lp, p, dq, dk, dv, st);
  if (a.Dq == 128 && a.Dv == 128) return flash_bwd_both<2, 2>(a, dO, lp, p, dq, dk, dv, st);
  if (a.Dq == 64 && a.Dv == 64) return flash_bwd_both<1, 1>(a, dO, lp, p, dq, dk, dv, st);
  return 1;
}
