// bf16 GEMM on tcgen05 tensor cores (sm_100a), fp32 accumulation in TMEM, optionally batched.
//
//   C[M,N] (+)= A · Bᵀ      A: M×K, B: N×K, each either K-major (K contiguous, the natural
//                           layout of activations and nn.Linear weights) or MN-major (the
//                           contraction index is the slow one: what dgrad/wgrad see without
//                           any transposed copies).
//   Batched: up to three batch dimensions (n2, n3, n4), each operand with its own element strides;
//   dimension 2 of A or B may be shared by `div` consecutive problems (heads of one group).
//
// Structure: persistent CTAs (one per SM), 320 threads in three roles —
//   warp 0     TMA producer: fills a 4..6-deep ring of {A tile, B tile} stages (128-byte swizzle)
//   warp 1     MMA issuer  : one thread issues tcgen05.mma (128×BN×16) into one of two TMEM
//                            accumulators; tcgen05.commit hands stages back / signals the epilogue
//   warps 2-9  epilogue    : two warp-groups, each owning half of the tile's columns; every warp
//                            reads its 32 TMEM lanes, applies the epilogue, stages a 32-row box in
//                            swizzled shared memory and issues a TMA store (or TMA reduce-add when
//                            accumulating).  Overlaps with the next tile's mainloop thanks to the
//                            double-buffered accumulator.
// Epilogues: plain; decay-mask `acc · exp(r[t] − c[s]) · [s ≤ t]` (the intra-chunk matrix of the
// Mamba3 scan); row-exp `acc · exp(r[t])` (the carried-state term of the same scan).  Every mbarrier wait is bounded (see sm100.cuh); a timeout is reported via `status`.
//
// Takes the role of the reference's dense `mx.matmul` call sites ("Path A",
// docs/production_kernel_routing.md:62-140); there is no GEMM kernel in the reference to compare to.
#include <atomic>
#include <cstdlib>
#include <mutex>

#include "sm100.cuh"

namespace cmb {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;  // 64 bf16 = one 128-byte swizzle line
constexpr int GEMM_EPI_WARPS = 8;
constexpr int GEMM_THREADS = 64 + 32 * GEMM_EPI_WARPS;
constexpr int GEMM_GROUP_M = 16;
constexpr int GEMM_CBOX_BYTES = 32 * 128;  // one epilogue warp's staging box: 32 rows × 128 bytes

enum : int {
  GEMM_OUT_F32 = 1,
  GEMM_ACCUMULATE = 2,
  GEMM_EPI_DECAY_MASK = 4,   // acc · exp(r[t] − c[s]) · [s ≤ t]
  GEMM_EPI_ROW_EXP = 8,      // acc · exp(r[t])
  GEMM_CAUSAL_SKIP = 16,     // tiles entirely above the diagonal (n0 ≥ m0 + BM) are not computed nor written
  GEMM_K_UPPER = 32,         // contraction restricted to k < m0 + BM   (keys up to the query tile)
  GEMM_K_LOWER = 64,         // contraction restricted to k ≥ m0        (queries from the key tile on)
  GEMM_EPI_SOFTMAX_STATS = 128,  // no C; per (row, tile half): running max / Σexp of masked scale·acc
  GEMM_EPI_EXP_MASK = 256,       // P = [mask] · exp(scale·acc − r[t])
  GEMM_EPI_DS = 512,             // dS = aux · (acc − r[t]) · scale   (aux has C's layout, bf16)
  GEMM_EPI_AXPBY = 1024,         // scale · acc + scale2 · aux        (aux has C's layout, bf16)
  GEMM_EPI_AMAX = 4096,          // max |C| over the written elements (NaNs ignored) is folded into *amax with an integer atomicMax:
                                 // the per-tensor FP8 scale of the product without a reduction pass over it
  GEMM_EPI_RELU2 = 8192,         // max(acc, 0)²: the squared-ReLU activation of an up projection without a pass over its output
  GEMM_EPI_SYM_MIRROR = 2048,    // with CAUSAL_SKIP on a symmetric product (bf16 C): every element whose transposed position lies
                                 // in a skipped tile is also stored there, so the full matrix exists after one launch
};

struct GemmParams {
  int M, N, K;
  int nb2, nb3, nb4;
  int a_div2, b_div2;
  int flags;
  const float* row_vec;
  const float* col_vec;
  long long sv2, sv3, sv4;  // element strides of the epilogue vectors over the batch dims
  const __nv_bfloat16* aux;  // DS epilogue: matrix with C's geometry
  long long ldc, sC2, sC3, sC4;
  const unsigned* mask;      // attention epilogues: bit s of row t allows key s; nullptr = causal only
  long long mask_sb;         // words between batches (dim 4)
  int mask_words;            // words per row
  float scale, scale2;
  float* stats;              // SOFTMAX_STATS output: float2 per (problem, row, tile_n, half)
  const int* tile_group;     // grouped (MoE) mode: B's dim-2 index for each 128-row tile of A / C; nullptr = batched rule
  const int* k_ranges;       // grouped wgrad: contraction range [k_begin, k_end) per dim-2 problem (multiples of 64)
  __nv_bfloat16* c_base;     // SYM_MIRROR: C as a plain pointer (the mirrored elements are stored with ordinary stores)
  float* amax;               // EPI_AMAX: one fp32 word (non-negative floats order like their bit patterns)
  const int* m_limit;        // optional device scalar: row tiles starting at or beyond *m_limit are neither computed nor written
                             // (the used part of a statically sized, token-sorted buffer is only known on the device)
  int group_m;               // row tiles per rasterisation group (consecutive tiles walk down a group's rows before the next column)
  int* status;
};

// PAIR = 1: two CTAs of a cluster share one 256×BN tile (tcgen05 cta_group::2).  Each stages its own 128 rows of A and half of
// B's rows, so a stage is 32 KB instead of 48 KB per CTA and the ring is six deep.
template <int BN, int PAIR = 0>
struct GemmCfg {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_ROWS = PAIR ? BN / 2 : BN;      // rows of B this CTA stages
  static constexpr int B_BYTES = B_ROWS * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = PAIR ? 6 : ((BN == 256) ? 4 : 6);
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int C_BYTES = GEMM_EPI_WARPS * GEMM_CBOX_BYTES;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + C_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
};

__device__ __forceinline__ void tma_load_5d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1, int c2,
                                            int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2),
      "r"(c3), "r"(c4)
      : "memory");
}
// The same load issued by a CTA of a pair: the transaction bytes are counted on `bar_cluster_addr`, an mbarrier that may live in
// the other CTA of the pair (the issuing CTA's barrier of the even CTA collects both halves of a stage).
__device__ __forceinline__ void tma_load_5d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int c0, int c1,
                                                 int c2, int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2),
      "r"(c3), "r"(c4)
      : "memory");
}
__device__ __forceinline__ void tma_store_5d(const CUtensorMap* m, const void* smem_src, int c0, int c1, int c2, int c3,
                                             int c4) {
  asm volatile("cp.async.bulk.tensor.5d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5, %6}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
               : "memory");
}
__device__ __forceinline__ void tma_reduce_add_5d(const CUtensorMap* m, const void* smem_src, int c0, int c1, int c2,
                                                  int c3, int c4) {
  asm volatile("cp.reduce.async.bulk.tensor.5d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5, %6}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
               : "memory");
}

struct TileCoord {
  int tm, tn, i2, i3, i4;
};

// With CAUSAL_SKIP only the tiles that touch the lower triangle are enumerated (row tm keeps its first causal_kept(tm) column
// tiles), so a persistent CTA's share of the index space is a share of the real work: striding over all tiles and skipping left
// the CTAs with up to 1.5× the mean number of kept tiles.
// `tile_m` is the row extent of a tile: 128, or 256 for a CTA pair.
__host__ __device__ __forceinline__ int causal_kept(int tm, int num_n, int bn, int tile_m = GEMM_BM) {
  const int k = (tm * tile_m + tile_m - 1) / bn + 1;
  return k < num_n ? k : num_n;
}
__host__ __device__ __forceinline__ int tiles_per_problem(int flags, int num_m, int num_n, int bn, int tile_m = GEMM_BM) {
  if (!(flags & GEMM_CAUSAL_SKIP)) return num_m * num_n;
  int n = 0;
  for (int tm = 0; tm < num_m; ++tm) n += causal_kept(tm, num_n, bn, tile_m);
  return n;
}

__device__ __forceinline__ TileCoord tile_coords(int t, int num_m, int num_n, int nb2, int nb3, int per_problem, bool causal, int bn,
                                                 int tile_m = GEMM_BM, int group_m = GEMM_GROUP_M) {
  TileCoord c;
  const int batch = t / per_problem;
  const int r0 = t - batch * per_problem;
  c.i2 = batch % nb2;
  const int q = batch / nb2;
  c.i3 = q % nb3;
  c.i4 = q / nb3;
  if (causal) {
    int acc = 0, tm = 0;
    for (; tm < num_m - 1; ++tm) {
      const int k = causal_kept(tm, num_n, bn, tile_m);
      if (r0 < acc + k) break;
      acc += k;
    }
    c.tm = tm;
    c.tn = r0 - acc;
    return c;
  }
  const int per_group = group_m * num_n;
  const int g = r0 / per_group;
  const int first_m = g * group_m;
  const int gsz = min(num_m - first_m, group_m);
  const int r = r0 - g * per_group;
  c.tm = first_m + r % gsz;
  c.tn = r / gsz;
  return c;
}

// `m0` is the first row of the whole tile (of the pair's 256 rows in the pair form), so both CTAs of a pair decide alike.
__device__ __forceinline__ bool tile_skipped(int flags, int m0, int n0, int m_limit, int tile_m = GEMM_BM) {
  return ((flags & GEMM_CAUSAL_SKIP) && n0 >= m0 + tile_m) || m0 >= m_limit;
}
__device__ __forceinline__ void k_range(int flags, int m0, int num_kb, const int* k_ranges, int i2, int& kb0, int& kb1) {
  kb0 = (flags & GEMM_K_LOWER) ? m0 / GEMM_BK : 0;
  kb1 = (flags & GEMM_K_UPPER) ? min(num_kb, (m0 + GEMM_BM + GEMM_BK - 1) / GEMM_BK) : num_kb;
  if (k_ranges != nullptr) {
    kb0 = max(kb0, k_ranges[2 * i2] / GEMM_BK);
    kb1 = min(kb1, (k_ranges[2 * i2 + 1] + GEMM_BK - 1) / GEMM_BK);
  }
}

template <int BN, bool A_MN, bool B_MN, int PAIR = 0>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const GemmParams p) {
  using Cfg = GemmCfg<BN, PAIR>;
  // PAIR: launched as clusters of two CTAs.  Both walk the same sequence of 256-row tiles; CTA `rank` owns rows
  // [rank·128, rank·128 + 128) of the tile and rows [rank·BN/2, …) of B's tile.  The even CTA's MMA thread issues for both.
  constexpr int TILE_M = GEMM_BM << PAIR;
  const int cta_rank = PAIR ? static_cast<int>(cluster_ctarank()) : 0;
  const int first_tile = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int tile_stride = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  const int m_off = cta_rank * GEMM_BM;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* csmem = smem + STAGES * Cfg::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(csmem + Cfg::C_BYTES);
  uint64_t* full_bar = bars;                     // [STAGES]
  uint64_t* empty_bar = bars + STAGES;           // [STAGES]
  uint64_t* tfull_bar = bars + 2 * STAGES;       // [2]
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (p.M + TILE_M - 1) / TILE_M;
  const int num_n = (p.N + BN - 1) / BN;
  const bool causal = (p.flags & GEMM_CAUSAL_SKIP) != 0;
  const int per_problem = tiles_per_problem(p.flags, num_m, num_n, BN, TILE_M);
  const int num_tiles = per_problem * p.nb2 * p.nb3 * p.nb4;
  const int num_kb = (p.K + GEMM_BK - 1) / GEMM_BK;
  int* status = p.status;
  const int m_limit = p.m_limit != nullptr ? *p.m_limit : 0x7fffffff;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], GEMM_EPI_WARPS << PAIR);   // PAIR: the epilogue warps of both CTAs release the even CTA's barrier
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(tmem_slot, Cfg::TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  if (PAIR)
    cluster_sync_all();   // the other CTA's barriers are initialised before anything signals them
  else
    __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = first_tile; t < num_tiles && ok; t += tile_stride) {
        const TileCoord tc = tile_coords(t, num_m, num_n, p.nb2, p.nb3, per_problem, causal, BN, TILE_M, p.group_m);
        const int m0 = tc.tm * TILE_M + m_off, n0 = tc.tn * BN + cta_rank * Cfg::B_ROWS;
        const int a2 = tc.i2 / p.a_div2;
        const int b2 = p.tile_group != nullptr ? p.tile_group[tc.tm] : tc.i2 / p.b_div2;
        if (tile_skipped(p.flags, tc.tm * TILE_M, tc.tn * BN, m_limit, TILE_M)) continue;
        int kb0, kb1;
        k_range(p.flags, m0, num_kb, p.k_ranges, tc.i2, kb0, kb1);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, status, ST_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          const int k0 = kb * GEMM_BK;
          if (PAIR) {
            // both CTAs' bytes are counted on the even CTA's barrier, which only its own producer arms
            const uint32_t lead_full = mapa_u32(smem_u32(&full_bar[stage]), 0);
            if (cta_rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * Cfg::STAGE_BYTES);
            if (A_MN) {
#pragma unroll
              for (int i = 0; i < GEMM_BM / 64; ++i)
                tma_load_5d_pair(sa + i * (GEMM_BK * 128), &tmA, lead_full, m0 + 64 * i, k0, a2, tc.i3, tc.i4);
            } else {
              tma_load_5d_pair(sa, &tmA, lead_full, k0, m0, a2, tc.i3, tc.i4);
            }
            if (B_MN) {
#pragma unroll
              for (int i = 0; i < Cfg::B_ROWS / 64; ++i)
                tma_load_5d_pair(sb + i * (GEMM_BK * 128), &tmB, lead_full, n0 + 64 * i, k0, b2, tc.i3, tc.i4);
            } else {
              tma_load_5d_pair(sb, &tmB, lead_full, k0, n0, b2, tc.i3, tc.i4);
            }
          } else {
            mbar_arrive_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
            if (A_MN) {
#pragma unroll
              for (int i = 0; i < GEMM_BM / 64; ++i)
                tma_load_5d(sa + i * (GEMM_BK * 128), &tmA, &full_bar[stage], m0 + 64 * i, k0, a2, tc.i3, tc.i4);
            } else {
              tma_load_5d(sa, &tmA, &full_bar[stage], k0, m0, a2, tc.i3, tc.i4);
            }
            if (B_MN) {
#pragma unroll
              for (int i = 0; i < BN / 64; ++i)
                tma_load_5d(sb + i * (GEMM_BK * 128), &tmB, &full_bar[stage], n0 + 64 * i, k0, b2, tc.i3, tc.i4);
            } else {
              tma_load_5d(sb, &tmB, &full_bar[stage], k0, n0, b2, tc.i3, tc.i4);
            }
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && cta_rank == 0) {
      constexpr uint32_t idesc = make_idesc(TILE_M, BN, 1, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int t = first_tile; t < num_tiles && ok; t += tile_stride) {
        const TileCoord tc = tile_coords(t, num_m, num_n, p.nb2, p.nb3, per_problem, causal, BN, TILE_M, p.group_m);
        const int m0 = tc.tm * TILE_M;
        if (tile_skipped(p.flags, m0, tc.tn * BN, m_limit, TILE_M)) continue;
        int kb0, kb1;
        k_range(p.flags, m0, num_kb, p.k_ranges, tc.i2, kb0, kb1);
        const int buf = local & 1;
        const uint32_t aphase = (local >> 1) & 1;
        ++local;
        if (!mbar_wait(&tempty_bar[buf], aphase ^ 1, abort_flag, status, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, status, ST_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint32_t sb = sa + Cfg::A_BYTES;
#pragma unroll
          for (int k = 0; k < GEMM_BK / 16; ++k) {
            const uint64_t adesc = A_MN ? make_smem_desc_sw128(sa + k * 2048, GEMM_BK * 128, 1024)
                                        : make_smem_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc_sw128(sb + k * 2048, GEMM_BK * 128, 1024)
                                        : make_smem_desc_sw128(sb + k * 32, 16, 1024);
            if (PAIR)
              umma_f16_pair(tmem_d, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
            else
              umma_f16(tmem_d, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          if (PAIR)
            umma_commit_pair(&empty_bar[stage], 3);   // the stage goes back to both CTAs' producers
          else
            umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) {
          if (PAIR)
            umma_commit_pair(&tfull_bar[buf], 3);
          else
            umma_commit(&tfull_bar[buf]);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (8 warps)
    const int ew = warp - 2;
    const int quarter = warp & 3;  // TMEM lane quarter this warp may read
    const int half = ew >> 2;      // which half of the tile's columns
    const bool out_f32 = (p.flags & GEMM_OUT_F32) != 0;
    const bool accum = (p.flags & GEMM_ACCUMULATE) != 0;
    const bool decay = (p.flags & GEMM_EPI_DECAY_MASK) != 0;
    const bool rowexp = (p.flags & GEMM_EPI_ROW_EXP) != 0;
    const bool e_stats = (p.flags & GEMM_EPI_SOFTMAX_STATS) != 0;
    const bool e_expm = (p.flags & GEMM_EPI_EXP_MASK) != 0;
    const bool e_ds = (p.flags & GEMM_EPI_DS) != 0;
    const bool attn = e_stats || e_expm || e_ds;
    const bool e_axpby = (p.flags & GEMM_EPI_AXPBY) != 0;
    const bool e_mirror = (p.flags & GEMM_EPI_SYM_MIRROR) != 0 && !out_f32;
    const bool e_amax = (p.flags & GEMM_EPI_AMAX) != 0 && p.amax != nullptr;
    const bool e_relu2 = (p.flags & GEMM_EPI_RELU2) != 0;
    uint8_t* cbox = csmem + ew * GEMM_CBOX_BYTES;
    int local = 0;
    const uint32_t lead_tempty = PAIR ? mapa_u32(smem_u32(&tempty_bar[0]), 0) : 0u;
    for (int t = first_tile; t < num_tiles; t += tile_stride) {
      const TileCoord tc = tile_coords(t, num_m, num_n, p.nb2, p.nb3, per_problem, causal, BN, TILE_M, p.group_m);
      const int tile_m0 = tc.tm * TILE_M + m_off;
      if (tile_skipped(p.flags, tc.tm * TILE_M, tc.tn * BN, m_limit, TILE_M)) continue;
      const int buf = local & 1;
      const uint32_t aphase = (local >> 1) & 1;
      ++local;
      if (!mbar_wait(&tfull_bar[buf], aphase, abort_flag, status, ST_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after();
      bool empty_k = false;
      if (p.k_ranges != nullptr) {  // a problem with no contraction steps leaves the accumulator unwritten: emit zeros
        int kb0, kb1;
        k_range(p.flags, tile_m0, num_kb, p.k_ranges, tc.i2, kb0, kb1);
        empty_k = kb0 >= kb1;
      }
      const int row0 = tile_m0 + quarter * 32;
      const int row = row0 + lane;
      const int ncol0 = tc.tn * BN + half * (BN / 2);
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN + half * (BN / 2);
      float rv = 0.f;
      const float* colv = nullptr;
      if (decay || rowexp || e_expm || e_ds) {
        const long long voff = tc.i2 * p.sv2 + tc.i3 * p.sv3 + tc.i4 * p.sv4;
        rv = row < p.M ? p.row_vec[voff + row] : 0.f;
        if (decay) colv = p.col_vec + voff;
        if (rowexp) rv = __expf(rv);
      }
      const unsigned* mrow = nullptr;
      if (attn && p.mask != nullptr && row < p.M)
        mrow = p.mask + tc.i4 * p.mask_sb + static_cast<long long>(row) * p.mask_words;
      const __nv_bfloat16* auxrow = nullptr;
      if ((e_ds || e_axpby) && row < p.M)
        auxrow = p.aux + tc.i2 * p.sC2 + tc.i3 * p.sC3 + tc.i4 * p.sC4 + static_cast<long long>(row) * p.ldc;
      const bool aux_aligned = auxrow != nullptr && (reinterpret_cast<uintptr_t>(auxrow) & 15) == 0;
      float run_m = -INFINITY, run_l = 0.f;
      float tile_amax = 0.f;
#pragma unroll 1
      for (int c = 0; c < (BN / 2) / 32; ++c) {
        uint32_t r[32];
        const int col0 = ncol0 + c * 32;
        // AXPBY: this row's 32 aux values as four 16-byte loads, issued before the accumulator read so the two latencies overlap
        uint4 ax[4];
        const bool ax_wide = e_axpby && auxrow != nullptr && aux_aligned && col0 + 32 <= p.N;
        if (ax_wide) {
#pragma unroll
          for (int q = 0; q < 4; ++q) ax[q] = *reinterpret_cast<const uint4*>(auxrow + col0 + 8 * q);
        }
        tmem_ld_x32(taddr + c * 32, r);
        tmem_wait_ld();
        if (empty_k) {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        if (attn) {
          // keys this row may see inside the 32-column chunk: mask word ∧ causal ∧ in range
          unsigned bits = 0u;
          if (row < p.M && col0 < p.N) {
            bits = mrow != nullptr ? mrow[col0 >> 5] : 0xffffffffu;
            const int lim = row - col0;  // columns j ≤ lim are causal
            if (lim < 0) bits = 0u;
            else if (lim < 31) bits &= (2u << lim) - 1u;
            const int rem = p.N - col0;
            if (rem < 32) bits &= (1u << rem) - 1u;
          }
          if (e_stats) {
            float cm = -INFINITY;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if ((bits >> j) & 1u) cm = fmaxf(cm, __uint_as_float(r[j]) * p.scale);
            if (cm > -INFINITY) {
              const float nm = fmaxf(run_m, cm);
              float acc = 0.f;
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if ((bits >> j) & 1u) acc += __expf(__uint_as_float(r[j]) * p.scale - nm);
              run_l = run_l * __expf(run_m - nm) + acc;
              run_m = nm;
            }
            continue;
          }
          if (e_expm) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float v = ((bits >> j) & 1u) ? __expf(__uint_as_float(r[j]) * p.scale - rv) : 0.f;
              r[j] = __float_as_uint(v);
            }
          } else {  // e_ds
            uint32_t pw[16];
            if (auxrow != nullptr && col0 + 32 <= p.N) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint4 v = *reinterpret_cast<const uint4*>(auxrow + col0 + 8 * q);
                pw[4 * q] = v.x; pw[4 * q + 1] = v.y; pw[4 * q + 2] = v.z; pw[4 * q + 3] = v.w;
              }
            } else {
#pragma unroll
              for (int q = 0; q < 16; ++q) {
                float lo = 0.f, hi = 0.f;
                if (auxrow != nullptr && col0 + 2 * q < p.N) lo = __bfloat162float(auxrow[col0 + 2 * q]);
                if (auxrow != nullptr && col0 + 2 * q + 1 < p.N) hi = __bfloat162float(auxrow[col0 + 2 * q + 1]);
                pw[q] = pack_bf16x2(lo, hi);
              }
            }
#pragma unroll
            for (int q = 0; q < 16; ++q) {
              const float2 pp = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pw[q]));
              const float d0 = ((bits >> (2 * q)) & 1u) ? pp.x * (__uint_as_float(r[2 * q]) - rv) * p.scale : 0.f;
              const float d1 = ((bits >> (2 * q + 1)) & 1u) ? pp.y * (__uint_as_float(r[2 * q + 1]) - rv) * p.scale : 0.f;
              r[2 * q] = __float_as_uint(d0);
              r[2 * q + 1] = __float_as_uint(d1);
            }
          }
        }
        if (ax_wide) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            float f[8];
            unpack8_bf16(ax[q], f);
#pragma unroll
            for (int i = 0; i < 8; ++i) r[8 * q + i] = __float_as_uint(p.scale * __uint_as_float(r[8 * q + i]) + p.scale2 * f[i]);
          }
        } else if (e_axpby) {
#pragma unroll
          for (int q = 0; q < 16; ++q) {
            float lo = 0.f, hi = 0.f;
            if (auxrow != nullptr && col0 + 2 * q + 1 < p.N) {
              const float2 pp = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(auxrow + col0 + 2 * q));
              lo = pp.x;
              hi = pp.y;
            } else if (auxrow != nullptr && col0 + 2 * q < p.N) {
              lo = __bfloat162float(auxrow[col0 + 2 * q]);
            }
            r[2 * q] = __float_as_uint(p.scale * __uint_as_float(r[2 * q]) + p.scale2 * lo);
            r[2 * q + 1] = __float_as_uint(p.scale * __uint_as_float(r[2 * q + 1]) + p.scale2 * hi);
          }
        }
        if (decay) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int s = col0 + j;
            float v = 0.f;
            if (s <= row && s < p.N) v = __uint_as_float(r[j]) * __expf(rv - colv[s]);
            r[j] = __float_as_uint(v);
          }
        }
        if (rowexp) {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * rv);
        }
        if (e_relu2) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float v = fmaxf(__uint_as_float(r[j]), 0.f);
            r[j] = __float_as_uint(v * v);
          }
        }
        if (e_mirror && row < p.M && (row / BN) * BN >= (col0 / TILE_M) * TILE_M + TILE_M) {
          // (col, row) lies in a tile the causal skip left out (its tile would start at column (row / BN)·BN ≥ its first row +
          // the tile height): this thread's 32 values go there as column `row`; for a fixed j the warp writes 32 consecutive elements.
          __nv_bfloat16* cm = p.c_base + tc.i2 * p.sC2 + tc.i3 * p.sC3 + tc.i4 * p.sC4 + row;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) cm[static_cast<long long>(col0 + j) * p.ldc] = __float2bfloat16(__uint_as_float(r[j]));
        }
        if (e_amax && row < p.M) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float a = fabsf(__uint_as_float(r[j]));
            if (col0 + j < p.N && a == a) tile_amax = fmaxf(tile_amax, a);
          }
        }
        // Stage into the swizzled box: row `lane`, 16-byte chunk ch lands at chunk (ch ^ (lane & 7)).
        const bool new_box = out_f32 || (c & 1) == 0;
        if (new_box) {
          if (lane == 0) tma_store_wait_read<0>();
          __syncwarp();
        }
        uint8_t* rowp = cbox + lane * 128;
        if (out_f32) {
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) {
            const uint4 v = make_uint4(r[4 * ch], r[4 * ch + 1], r[4 * ch + 2], r[4 * ch + 3]);
            *reinterpret_cast<uint4*>(rowp + ((ch ^ (lane & 7)) << 4)) = v;
          }
        } else {
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
        }
        const bool box_done = out_f32 || (c & 1) == 1;
        if (box_done) {
          fence_proxy_async_smem();
          __syncwarp();
          const int bcol0 = out_f32 ? col0 : col0 - 32;
          if (lane == 0 && row0 < p.M && bcol0 < p.N) {
            if (accum)
              tma_reduce_add_5d(&tmC, cbox, bcol0, row0, tc.i2, tc.i3, tc.i4);
            else
              tma_store_5d(&tmC, cbox, bcol0, row0, tc.i2, tc.i3, tc.i4);
            tma_store_commit();
          }
        }
      }
      if (e_amax) {
        tile_amax = warp_max(tile_amax);
        if (lane == 0 && tile_amax > 0.f) atomicMax(reinterpret_cast<unsigned int*>(p.amax), __float_as_uint(tile_amax));
      }
      if (e_stats && row < p.M) {
        const long long prob = (static_cast<long long>(tc.i4) * p.nb3 + tc.i3) * p.nb2 + tc.i2;
        float2* dst = reinterpret_cast<float2*>(p.stats) + (prob * p.M + row) * (2 * num_n) + tc.tn * 2 + half;
        *dst = make_float2(run_m, run_l);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR)
          mbar_arrive_cluster(lead_tempty + buf * 8);
        else
          mbar_arrive(&tempty_bar[buf]);
      }
    }
    if (lane == 0) tma_store_wait<0>();  // all global writes done before the staging memory goes away
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  if (*abort_flag) {
    // Give TMA copies / MMAs that may still be in flight a bounded time to land before the
    // shared memory and TMEM they target are released.
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  tc_fence_before();
  if (PAIR)
    cluster_sync_all();   // neither CTA leaves (or frees TMEM) while the other may still signal its barriers or read its tiles
  else
    __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    if (PAIR)
      tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
    else
      tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace cmb

// =============================================================================== host
namespace cmb_host {

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

void bind_context_once() {
  // The driver-API encoder needs a current context; a thread whose first CUDA call is this one (an autograd
  // worker, say) has none until a runtime call binds the primary context.
  static thread_local bool bound = false;
  if (!bound) {
    cudaFree(nullptr);
    bound = true;
  }
}

static CUtensorMapDataType dtype_of(int elem_bytes) {
  return elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                         : (elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8);
}
static CUtensorMapSwizzle swizzle_of(int bytes) {
  return bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
         : bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
         : bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B
                       : CU_TENSOR_MAP_SWIZZLE_NONE;
}

int make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint64_t ld,
                 uint32_t box_rows, uint32_t box_cols, int swizzle_bytes) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return 101;
  bind_context_once();
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || ((ld * elem_bytes) & 15) != 0) return 102;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dtype_of(elem_bytes), 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_of(swizzle_bytes), CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1000 + static_cast<int>(r);
}

// 5-D map: (cols, rows, n2, n3, n4); strides in elements for rows and the three batch dims.
static int make_tmap_5d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint64_t ld,
                        const uint64_t nb[3], const int64_t sb[3], uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return 101;
  bind_context_once();
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || ((ld * elem_bytes) & 15) != 0) return 102;
  cuuint64_t dims[5] = {cols, rows, nb[0], nb[1], nb[2]};
  cuuint64_t strides[4];
  strides[0] = ld * static_cast<uint64_t>(elem_bytes);
  for (int i = 0; i < 3; ++i) {
    uint64_t s = static_cast<uint64_t>(sb[i]) * elem_bytes;
    if (nb[i] > 1 && s == 0) return 108;       // a zero stride cannot broadcast an operand: use a_div2 / b_div2
    if (nb[i] <= 1) s = strides[0];            // unused batch dim: any legal stride
    if (s & 15) return 105;
    strides[i + 1] = s;
  }
  cuuint32_t box[5] = {box_cols, box_rows, 1, 1, 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(out, dtype_of(elem_bytes), 5, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1000 + static_cast<int>(r);
}

static int sm_count() { return sm_count_current_device(); }

struct GemmArgs {
  const void* A;
  const void* B;
  void* C;
  int M, N, K;
  int64_t lda, ldb, ldc;
  int flags;
  uint64_t nb[3];
  int64_t sA[3], sB[3], sC[3];
  int a_div2, b_div2;
  const float* row_vec;
  const float* col_vec;
  int64_t sv[3];
  const void* aux;
  const unsigned* mask;
  int64_t mask_sb;
  int mask_words;
  float scale, scale2;
  float* stats;
  const int* tile_group;
  const int* k_ranges;
  const int* m_limit;
  float* amax;
  int b_groups;  // grouped mode: number of dim-2 slices of B (independent of the problem batch count)
  int* status;
  int max_ctas;
  cudaStream_t stream;
};

// Launches that may run as CTA pairs: dense products with the element-wise epilogues, with or without lower-triangle tile
// skipping and the symmetric mirror; nothing whose contraction range or operand depends on the 128-row tile (attention
// epilogues, per-tile groups, row limits), and at least one full 256-row tile.
static bool pair_eligible(const GemmArgs& g) {
  constexpr int no = cmb::GEMM_K_UPPER | cmb::GEMM_K_LOWER | cmb::GEMM_EPI_SOFTMAX_STATS | cmb::GEMM_EPI_EXP_MASK | cmb::GEMM_EPI_DS;
  return (g.flags & no) == 0 && g.tile_group == nullptr && g.k_ranges == nullptr && g.m_limit == nullptr && g.M >= 256;
}

// 0 = off, 1 = on for eligible launches (the default: 4–13 % faster on the model's projection shapes).  The environment
// variable CPPMEGA_GEMM_PAIR sets the initial value;
// cmb_gemm_set_pair_mode changes it for the process.
static std::atomic<int>& pair_mode_ref() {
  static std::atomic<int> mode{[] {
    const char* e = std::getenv("CPPMEGA_GEMM_PAIR");
    return e != nullptr ? (std::atoi(e) != 0 ? 1 : 0) : 1;
  }()};
  return mode;
}
static int pair_mode() { return pair_mode_ref().load(std::memory_order_relaxed); }

// Row tiles per rasterisation group; CPPMEGA_GEMM_GROUP_M overrides the default.  Measured on the model's projection shapes, 4, 8
// and 16 are within ±2 % of one another in either form and 32 is 2–7 % slower, so both forms keep 16.
static int group_m_setting(int /*pair*/) {
  static const int env = [] {
    const char* e = std::getenv("CPPMEGA_GEMM_GROUP_M");
    return e != nullptr ? std::atoi(e) : 0;
  }();
  return env > 0 ? env : cmb::GEMM_GROUP_M;
}

template <int BN, bool A_MN, bool B_MN, int PAIR = 0>
static int launch_gemm(const GemmArgs& g) {
  using Cfg = cmb::GemmCfg<BN, PAIR>;
  CUtensorMap tmA, tmB, tmC;
  int rc;
  uint64_t nbA[3] = {g.nb[0] / g.a_div2, g.nb[1], g.nb[2]};
  uint64_t nbB[3] = {g.tile_group != nullptr ? static_cast<uint64_t>(g.b_groups) : g.nb[0] / g.b_div2, g.nb[1], g.nb[2]};
  // K-major operand stored [rows=M|N, cols=K]; MN-major operand stored [rows=K, cols=M|N].
  if (A_MN)
    rc = make_tmap_5d(&tmA, g.A, 2, g.K, g.M, g.lda, nbA, g.sA, cmb::GEMM_BK, 64);
  else
    rc = make_tmap_5d(&tmA, g.A, 2, g.M, g.K, g.lda, nbA, g.sA, cmb::GEMM_BM, cmb::GEMM_BK);
  if (rc) return rc;
  if (B_MN)
    rc = make_tmap_5d(&tmB, g.B, 2, g.K, g.N, g.ldb, nbB, g.sB, cmb::GEMM_BK, 64);
  else
    rc = make_tmap_5d(&tmB, g.B, 2, g.N, g.K, g.ldb, nbB, g.sB, Cfg::B_ROWS, cmb::GEMM_BK);
  if (rc) return rc + 10000;
  const bool f32 = (g.flags & cmb::GEMM_OUT_F32) != 0;
  if (g.flags & cmb::GEMM_EPI_SOFTMAX_STATS) {
    tmC = tmA;  // no matrix output in this mode; the map is never used
  } else {
    rc = make_tmap_5d(&tmC, g.C, f32 ? 4 : 2, g.M, g.N, g.ldc, g.nb, g.sC, 32, f32 ? 32 : 64);
    if (rc) return rc + 20000;
  }
  auto kern = cmb::gemm_bf16_kernel<BN, A_MN, B_MN, PAIR>;
  static std::atomic<unsigned long long> attr_done{0};
  if (set_smem_limit_once_per_device(attr_done, reinterpret_cast<const void*>(kern), Cfg::SMEM_BYTES)) return 103;
  constexpr int tile_m = cmb::GEMM_BM << PAIR;
  const long long num_tiles = static_cast<long long>(cmb::tiles_per_problem(g.flags, (g.M + tile_m - 1) / tile_m, (g.N + BN - 1) / BN, BN, tile_m)) *
                              g.nb[0] * g.nb[1] * g.nb[2];
  if (num_tiles > 0x7fffffffLL) return 106;
  int grid = sm_count();
  if (g.max_ctas > 0 && g.max_ctas < grid) grid = g.max_ctas;
  if (PAIR) {
    grid /= 2;                                  // pairs
    if (grid < 1) grid = 1;
  }
  if (num_tiles < grid) grid = static_cast<int>(num_tiles);
  cmb::GemmParams p;
  p.M = g.M; p.N = g.N; p.K = g.K;
  p.nb2 = static_cast<int>(g.nb[0]); p.nb3 = static_cast<int>(g.nb[1]); p.nb4 = static_cast<int>(g.nb[2]);
  p.a_div2 = g.a_div2; p.b_div2 = g.b_div2;
  p.flags = g.flags;
  p.row_vec = g.row_vec; p.col_vec = g.col_vec;
  p.sv2 = g.sv[0]; p.sv3 = g.sv[1]; p.sv4 = g.sv[2];
  p.aux = static_cast<const __nv_bfloat16*>(g.aux);
  p.ldc = g.ldc; p.sC2 = g.sC[0]; p.sC3 = g.sC[1]; p.sC4 = g.sC[2];
  p.mask = g.mask; p.mask_sb = g.mask_sb; p.mask_words = g.mask_words;
  p.scale = g.scale; p.scale2 = g.scale2; p.stats = g.stats;
  p.tile_group = g.tile_group; p.k_ranges = g.k_ranges;
  p.c_base = static_cast<__nv_bfloat16*>(g.C);
  p.m_limit = g.m_limit;
  p.amax = g.amax;
  p.group_m = group_m_setting(PAIR);
  p.status = g.status;
  if (PAIR) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * grid);
    cfg.blockDim = dim3(cmb::GEMM_THREADS);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cfg.stream = g.stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmC, p) == cudaSuccess ? 0 : 104;
  }
  kern<<<grid, cmb::GEMM_THREADS, Cfg::SMEM_BYTES, g.stream>>>(tmA, tmB, tmC, p);
  return cudaGetLastError() == cudaSuccess ? 0 : 104;
}

static int dispatch(const GemmArgs& g, int a_mn, int b_mn) {
  if (g.M <= 0 || g.N <= 0 || g.K <= 0 || g.nb[0] * g.nb[1] * g.nb[2] == 0) return 0;
  if (g.a_div2 <= 0 || g.b_div2 <= 0 || g.nb[0] % g.a_div2 || g.nb[0] % g.b_div2) return 107;
  const bool big = g.N > 128;
#define CMB_GEMM_CASE(BN_, AM_, BM_) return launch_gemm<BN_, AM_, BM_>(g)
  if (big && pair_mode() == 1 && pair_eligible(g)) {
    if (!a_mn && !b_mn) return launch_gemm<256, false, false, 1>(g);
    if (!a_mn && b_mn) return launch_gemm<256, false, true, 1>(g);
    if (a_mn && !b_mn) return launch_gemm<256, true, false, 1>(g);
    return launch_gemm<256, true, true, 1>(g);
  }
  if (big) {
    if (!a_mn && !b_mn) CMB_GEMM_CASE(256, false, false);
    if (!a_mn && b_mn) CMB_GEMM_CASE(256, false, true);
    if (a_mn && !b_mn) CMB_GEMM_CASE(256, true, false);
    CMB_GEMM_CASE(256, true, true);
  } else {
    if (!a_mn && !b_mn) CMB_GEMM_CASE(128, false, false);
    if (!a_mn && b_mn) CMB_GEMM_CASE(128, false, true);
    if (a_mn && !b_mn) CMB_GEMM_CASE(128, true, false);
    CMB_GEMM_CASE(128, true, true);
  }
#undef CMB_GEMM_CASE
}

}  // namespace cmb_host

// Process-wide switch for the CTA-pair (cta_group::2) form of eligible launches; returns the previous value.
extern "C" int cmb_gemm_set_pair_mode(int mode) { return cmb_host::pair_mode_ref().exchange(mode != 0 ? 1 : 0); }

// C ABI. A is M×K (K-major, row pitch lda) or, with a_mn_major, stored K×M (row pitch lda).
// B is N×K (K-major) or, with b_mn_major, stored K×N. C is M×N row-major (pitch ldc), bf16 unless
// flags&1 (fp32); flags&2 accumulates into C. All pointers 16-byte aligned, every pitch a multiple of 16 bytes.
extern "C" int cmb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                             int a_mn_major, int b_mn_major, int flags, int* status, int max_ctas, void* stream) {
  cmb_host::GemmArgs g{};
  g.A = A; g.B = B; g.C = C; g.M = M; g.N = N; g.K = K;
  g.lda = lda; g.ldb = ldb; g.ldc = ldc;
  g.flags = flags & 3;
  for (int i = 0; i < 3; ++i) { g.nb[i] = 1; g.sA[i] = g.sB[i] = g.sC[i] = 0; g.sv[i] = 0; }
  g.a_div2 = g.b_div2 = 1;
  g.status = status; g.max_ctas = max_ctas; g.stream = static_cast<cudaStream_t>(stream);
  return cmb_host::dispatch(g, a_mn_major, b_mn_major);
}

// Batched form. `ip` = {M, N, K, a_mn, b_mn, flags, a_div2, b_div2, max_ctas, mask_words, b_groups, number of `pp` entries}; `lp` = {lda, ldb, ldc, nb2,
// nb3, nb4, sA2, sA3, sA4, sB2, sB3, sB4, sC2, sC3, sC4, sv2, sv3, sv4, mask_sb} (element counts / strides).
// `pp` = {row_vec, col_vec, aux, mask, stats, tile_group, k_ranges, m_limit, amax} device pointers (any may be null). Flags select the
// epilogue, see the enum at the top of this file. Grouped (MoE) use: `tile_group[i]` names B's dim-2 slice for the i-th
// 128-row tile of A/C (A and C plain 2-D, B stacked per expert); `k_ranges[2e], k_ranges[2e+1]` bound the contraction
// of dim-2 problem e (wgrad over one expert's rows of the token-sorted buffers).
extern "C" int cmb_gemm_bf16_batched(const void* A, const void* B, void* C, const int* ip, const long long* lp,
                                     const void* const* pp, float scale, float scale2, int* status, void* stream) {
  cmb_host::GemmArgs g{};
  g.A = A; g.B = B; g.C = C; g.M = ip[0]; g.N = ip[1]; g.K = ip[2];
  g.flags = ip[5]; g.a_div2 = ip[6]; g.b_div2 = ip[7]; g.max_ctas = ip[8]; g.mask_words = ip[9];
  g.lda = lp[0]; g.ldb = lp[1]; g.ldc = lp[2];
  for (int i = 0; i < 3; ++i) {
    g.nb[i] = static_cast<uint64_t>(lp[3 + i]);
    g.sA[i] = lp[6 + i]; g.sB[i] = lp[9 + i]; g.sC[i] = lp[12 + i]; g.sv[i] = lp[15 + i];
  }
  g.mask_sb = lp[18];
  g.row_vec = static_cast<const float*>(pp[0]); g.col_vec = static_cast<const float*>(pp[1]);
  g.aux = pp[2]; g.mask = static_cast<const unsigned*>(pp[3]); g.stats = static_cast<float*>(const_cast<void*>(pp[4]));
  g.tile_group = static_cast<const int*>(pp[5]); g.k_ranges = static_cast<const int*>(pp[6]);
  g.m_limit = ip[11] >= 8 ? static_cast<const int*>(pp[7]) : nullptr;   // ip[11]: how many entries `pp` holds (older callers pass 7)
  g.amax = ip[11] >= 9 ? static_cast<float*>(const_cast<void*>(pp[8])) : nullptr;
  if ((g.flags & cmb::GEMM_EPI_AMAX) && g.amax == nullptr) return 108;
  g.b_groups = ip[10];
  if (g.tile_group != nullptr && g.b_groups <= 0) return 109;
  g.scale = scale;
  g.scale2 = scale2;
  g.status = status; g.stream = static_cast<cudaStream_t>(stream);
  const int f = g.flags;
  if ((f & cmb::GEMM_EPI_DECAY_MASK) && (g.row_vec == nullptr || g.col_vec == nullptr)) return 108;
  if ((f & (cmb::GEMM_EPI_ROW_EXP | cmb::GEMM_EPI_EXP_MASK | cmb::GEMM_EPI_DS)) && g.row_vec == nullptr) return 108;
  if ((f & (cmb::GEMM_EPI_DS | cmb::GEMM_EPI_AXPBY)) && g.aux == nullptr) return 108;
  if ((f & cmb::GEMM_EPI_SOFTMAX_STATS) && g.stats == nullptr) return 108;
  return cmb_host::dispatch(g, ip[3], ip[4]);
}
