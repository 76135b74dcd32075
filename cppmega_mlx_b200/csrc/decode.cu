// Flash-decoding on tcgen05 for one new query per sequence: split over the key list, keys fetched through a page table
// (or from a contiguous cache), scores and outputs on the tensor cores with the *keys* as the MMA M dimension so that a
// handful of heads (N = 16) wastes no tensor work:
//
//   GEMM1   Sᵀ[64 keys, 16 heads]  = K_tile[64, Dk] · Qᵀ                 (A = key rows, K-major, M = 64)
//   softmax (online, lazy re-referencing of the running max), P → shared memory as bf16
//   GEMM2   Oᵀ[Dv, 16 heads]     += V_tileᵀ[Dv, 64 keys] · Pᵀ           (A = the same rows read MN-major, M = 128)
//
// For latent MLA (Dk = 576, Dv = 512) K and V are the same 1152-byte cache row, so every byte of the cache crosses HBM
// once per head group and is used by both GEMMs from one shared-memory tile.  A per-sequence key list (`topk`, −1 padded)
// restricts attention to the indexer's selection (sparse-MLA decode).  Semantics follow the dense oracle
// (cppmega_mlx/nn/sparse_mla.py:125-210 for the sparse form; cppmega_mlx/inference/serving.py:47-215 describes the paged
// pools): masked softmax over valid keys, zeros when no key is valid.
//
// Roles in a 320-thread CTA: warps 0-3 softmax / TMEM read-back, warps 4-5 and 8-9 cp.async gather (pairs alternate tiles; 8 lanes per 128-byte line,
// hand-swizzled into the 128B-swizzle layout the MMA descriptors expect; dense key ranges use TMA boxes instead), warp 6 issues the
// score MMAs and warp 7 the output MMAs.  Tiles of 64 keys are
// double-buffered.  Every mbarrier wait is bounded (sm100.cuh); an abandoned wait raises the CTA's abort flag, everything
// drains, TMEM is freed and the status word reports the site.
#include <cstring>

#include "sm100.cuh"

namespace cmb {

constexpr int DEC_TILE = 64;       // keys per tile
constexpr int DEC_N = 16;          // heads per CTA (MMA N)
constexpr int DEC_BLK = 8192;      // bytes of one [64 keys × 64 bf16] block
constexpr int DEC_THREADS = 320;   // warps 0-3 softmax, 4-5 and 8-9 gather, 6 score MMAs, 7 output MMAs
constexpr float DEC_RESCALE_THRESHOLD = 8.f;  // log2 units a tile max may exceed the reference before O is rescaled

struct DecodeParams {
  const __nv_bfloat16* q;        // [B, H, Dk], strides q_sb, q_sh (elements)
  long long q_sb, q_sh;
  const __nv_bfloat16* k;        // row (b|page, pos) at k + page*k_page + (pos % page_size)*k_row (+ b*k_batch if no table)
  const __nv_bfloat16* v;        // same for values (unused when K and V share a row)
  long long k_page, k_row, k_batch, k_head;   // k_head: offset between kv heads
  long long v_page, v_row, v_batch, v_head;
  const int* table;              // [B, table_w] page ids, or nullptr for a contiguous cache
  int table_w, page_size;
  int n_pages;                   // pages in the pool (0 = unknown): page ids from the table are checked against it
  const int* lengths;            // [B]
  const int* topk;               // [B, topk_n] key positions (−1 = unused) or nullptr
  int topk_n;
  int B, H, kv_heads, splits;
  float scale_log2;              // softmax scale · log2(e)
  float* ws_o;                   // [B, H, splits, Dv] un-normalised partial outputs
  float* ws_m;                   // [B, H, splits] reference max (log2 domain)
  float* ws_l;                   // [B, H, splits] partial denominators
  int* status;
  int tma;                       // 1: tiles are fetched with TMA boxes (dense key ranges); 0: per-row cp.async gather
  int box_rows;                  // rows per TMA box (min(64, page_size))
  long long* trace;              // optional: per-tile clock samples of CTA (0,0,0), TRACE_SLOTS per tile (nullptr = off)
};

constexpr int TRACE_SLOTS = 16;
// Record the SM clock at pipeline point `slot` of tile `t` (only CTA 0; one elected thread per role calls it).
__device__ __forceinline__ void trace_mark(const DecodeParams& p, int t, int slot) {
  if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && t < 64) p.trace[t * TRACE_SLOTS + slot] = clock64();
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ int float_order(float x) {
  const int i = __float_as_int(x);
  return i >= 0 ? i : i ^ 0x7fffffff;
}
__device__ __forceinline__ float order_float(int i) { return __int_as_float(i >= 0 ? i : i ^ 0x7fffffff); }

template <int DKB, int DVB, bool SHARED>
struct DecCfg {
  static constexpr int BUF_BYTES = (SHARED ? DKB : DKB + DVB) * DEC_BLK;
  static constexpr int Q_BYTES = DKB * DEC_N * 128;
  static constexpr int P_BYTES = DEC_N * 128;
  static constexpr int SMEM_BYTES = 2 * BUF_BYTES + Q_BYTES + P_BYTES + 1024 /*alignment slack*/ + 1024 /*control*/;
  static constexpr int MB = DVB / 2;                      // 128-row output blocks
  static constexpr int TMEM_COLS = (2 * DEC_N + MB * DEC_N) <= 64 ? 64 : 128;
};

template <int DKB, int DVB, bool SHARED>
__global__ void __launch_bounds__(DEC_THREADS, 1)
paged_decode_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const DecodeParams p) {
  using Cfg = DecCfg<DKB, DVB, SHARED>;
  constexpr int MB = Cfg::MB;
  constexpr int DV = DVB * 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* bufs = smem;                                   // 2 tiles
  uint8_t* qs = bufs + 2 * Cfg::BUF_BYTES;                // Q, K-major blocks of [16 heads × 64]
  uint8_t* ps = qs + Cfg::Q_BYTES;                        // P, [16 heads × 64 keys]
  uint8_t* ctl = ps + Cfg::P_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctl);  // [2]
  uint64_t* empty_bar = full_bar + 2;                     // [2]
  uint64_t* sfull_bar = empty_bar + 2;                    // [2]
  uint64_t* sfree_bar = sfull_bar + 2;                    // [2]
  uint64_t* pfull_bar = sfree_bar + 2;
  uint64_t* odone_bar = pfull_bar + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(odone_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* valid = reinterpret_cast<uint8_t*>(tmem_slot + 2);       // [2][64]
  float* wmax = reinterpret_cast<float*>(valid + 2 * DEC_TILE);     // [4][16]
  float* wsum = wmax + 4 * DEC_N;                                   // [4][16]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, b = blockIdx.y, zi = blockIdx.z;
  const int g = p.H / p.kv_heads;
  const int gchunks = (g + DEC_N - 1) / DEC_N;
  const int kvh = zi / gchunks, gc = zi % gchunks;
  const int h0 = kvh * g + gc * DEC_N;
  const int nh = min(DEC_N, g - gc * DEC_N);
  const int length = p.lengths[b];
  const int total = p.topk != nullptr ? p.topk_n : length;
  const int tiles_total = (total + DEC_TILE - 1) / DEC_TILE;
  const int tiles_per = (tiles_total + p.splits - 1) / p.splits;
  const int t_begin = split * tiles_per;
  const int T = max(0, min(tiles_total, t_begin + tiles_per) - t_begin);
  const long long ws_row = (static_cast<long long>(b) * p.H + h0) * p.splits + split;   // + h * splits

  if (T == 0) {  // nothing to attend to in this split: neutral partial
    for (int i = threadIdx.x; i < nh * DV; i += blockDim.x) {
      const int h = i / DV, d = i % DV;
      p.ws_o[(ws_row + static_cast<long long>(h) * p.splits) * DV + d] = 0.f;
    }
    if (threadIdx.x < nh) {
      p.ws_m[ws_row + static_cast<long long>(threadIdx.x) * p.splits] = -INFINITY;
      p.ws_l[ws_row + static_cast<long long>(threadIdx.x) * p.splits] = 0.f;
    }
    return;
  }

  // ---------------------------------------------------------------- setup
  if (threadIdx.x == 0) {
    mbar_init(&full_bar[0], p.tma ? 1 : 64);
    mbar_init(&full_bar[1], p.tma ? 1 : 64);
    mbar_init(&empty_bar[0], 1);
    mbar_init(&empty_bar[1], 1);
    mbar_init(&sfull_bar[0], 1);
    mbar_init(&sfull_bar[1], 1);
    mbar_init(&sfree_bar[0], 128);
    mbar_init(&sfree_bar[1], 128);
    mbar_init(pfull_bar, 128);
    mbar_init(odone_bar, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 6) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  // Q → shared memory, K-major 128B-swizzled blocks of [16 rows × 64 cols]; rows past `nh` are zero.
  for (int i = threadIdx.x; i < DKB * DEC_N * 8; i += blockDim.x) {
    const int c = i & 7, h = (i >> 3) % DEC_N, kb = i / (8 * DEC_N);
    uint4 val = make_uint4(0, 0, 0, 0);
    if (h < nh)
      val = *reinterpret_cast<const uint4*>(p.q + b * p.q_sb + (h0 + h) * p.q_sh + kb * 64 + c * 8);
    *reinterpret_cast<uint4*>(qs + kb * (DEC_N * 128) + h * 128 + ((c ^ (h & 7)) << 4)) = val;
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base;                 // 2 × 16 columns
  const uint32_t tmem_o = tmem_base + 2 * DEC_N;     // MB × 16 columns

  const bool gather_warp = warp == 4 || warp == 5 || warp >= 8;
  if (p.tma && gather_warp) {
    // ---------------------------------------------------------------- TMA producer (dense key ranges)
    // A 64-key tile is 64/box_rows boxes of [box_rows keys × 64 columns] per 128-byte column block, fetched straight into
    // the 128B-swizzled layout; completion is counted in bytes on the tile's mbarrier, so the producer never waits for data.
    if (warp == 4) {
      if (lane == 0) {
        tma_prefetch_desc(&tmK);
        if (!SHARED) tma_prefetch_desc(&tmV);
      }
      const int R = p.box_rows;
      const int last_page = p.table != nullptr ? (length - 1) / p.page_size : 0;
      for (int t = 0; t < T; ++t) {
        const int buf = t & 1;
        const int pos0 = (t_begin + t) * DEC_TILE;
        int ok = lane == 0 ? static_cast<int>(mbar_wait(&empty_bar[buf], ((t >> 1) & 1) ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);   // one lane waits; the whole warp takes the same exit
        if (!ok) break;
        valid[buf * DEC_TILE + lane] = pos0 + lane < length ? 1 : 0;
        valid[buf * DEC_TILE + 32 + lane] = pos0 + 32 + lane < length ? 1 : 0;
        __syncwarp();
        if (lane == 0) {
          trace_mark(p, t, 1);
          uint8_t* kb_s = bufs + buf * Cfg::BUF_BYTES;
          uint8_t* vb_s = kb_s + DKB * DEC_BLK;
          mbar_arrive_expect_tx(&full_bar[buf], Cfg::BUF_BYTES);
          for (int r0 = 0; r0 < DEC_TILE; r0 += R) {
            const int pos = pos0 + r0;
            int c2, c3;
            if (p.table != nullptr) {   // keys past the sequence re-read its last page (finite rows, masked by the softmax)
              c3 = p.table[static_cast<long long>(b) * p.table_w + min(pos / p.page_size, last_page)];
              c2 = pos % p.page_size;
            } else {
              c3 = b;
              c2 = pos;                 // rows past the cache extent are zero-filled by the TMA unit
            }
#pragma unroll
            for (int kb = 0; kb < DKB; ++kb) tma_load_4d(kb_s + kb * DEC_BLK + r0 * 128, &tmK, &full_bar[buf], kb * 64, kvh, c2, c3);
            if (!SHARED) {
#pragma unroll
              for (int kb = 0; kb < DVB; ++kb) tma_load_4d(vb_s + kb * DEC_BLK + r0 * 128, &tmV, &full_bar[buf], kb * 64, kvh, c2, c3);
            }
          }
          trace_mark(p, t, 2);
        }
      }
    }
  } else if (gather_warp) {
    // ---------------------------------------------------------------- gather
    // Two pairs of gather warps alternate tiles (warps 4,5: even tiles; warps 8,9: odd tiles), each warp fetching half of
    // the tile's rows.  A pair waits only for its own buffer to be released and for its own copies to land, so tile t+1 is
    // in flight while tile t is being consumed and no warp ever waits on work that needs another pair's arrival first.
    const int lw = warp >= 8 ? 1 : 0;
    const int half = warp & 1;
    const int sub = lane >> 3, c = lane & 7;
    const __nv_bfloat16* kbase = p.k + kvh * p.k_head + (p.table == nullptr ? b * p.k_batch : 0);
    const __nv_bfloat16* vbase = SHARED ? nullptr : p.v + kvh * p.v_head + (p.table == nullptr ? b * p.v_batch : 0);
    for (int t = lw; t < T; t += 2) {
      const int buf = t & 1;
      uint8_t* kb_s = bufs + buf * Cfg::BUF_BYTES;
      uint8_t* vb_s = kb_s + DKB * DEC_BLK;
      // Phase 1: all index / page-table reads of this lane's 16 rows are issued before anything depends on them (they
      // are dependent global loads; serialising them row by row would cost a memory latency per row).
      constexpr int RPL = DEC_TILE / 8;   // rows per lane group (half a tile per warp)
      int pos[RPL];
#pragma unroll
      for (int it = 0; it < RPL; ++it) {
        const int ki = (t_begin + t) * DEC_TILE + half * 32 + it * 4 + sub;
        pos[it] = -1;
        if (ki < total) pos[it] = p.topk != nullptr ? __ldg(p.topk + static_cast<long long>(b) * p.topk_n + ki) : ki;
        if (pos[it] >= length || (p.table != nullptr && pos[it] / p.page_size >= p.table_w)) pos[it] = -1;
      }
      int page[RPL];
#pragma unroll
      for (int it = 0; it < RPL; ++it)
        page[it] = (p.table != nullptr && pos[it] >= 0) ? __ldg(p.table + static_cast<long long>(b) * p.table_w + pos[it] / p.page_size) : 0;
#pragma unroll
      for (int it = 0; it < RPL; ++it) {
        // a page id outside the pool: the row is dropped like a key past the sequence, and the first one is reported
        if (p.n_pages > 0 && pos[it] >= 0 && (page[it] < 0 || page[it] >= p.n_pages)) {
          if (p.status != nullptr && atomicCAS(p.status, 0, ST_BAD_ARGUMENT) == 0) {
            p.status[1] = b;
            p.status[2] = page[it];
            p.status[3] = p.n_pages;
          }
          pos[it] = -1;
        }
      }
      if (lane == 0) trace_mark(p, t, 0);
      // Phase 2: the copies, once the buffer has been released (the index reads above overlap that wait).
      if (!mbar_wait(&empty_bar[buf], ((t >> 1) & 1) ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) break;
      if (lane == 0) trace_mark(p, t, 1);
#pragma unroll
      for (int it = 0; it < RPL; ++it) {
        const int row = half * 32 + it * 4 + sub;
        const bool ok_row = pos[it] >= 0;
        long long koff = 0, voff = 0;
        if (ok_row) {
          if (p.table != nullptr) {
            const int in = pos[it] % p.page_size;
            koff = page[it] * p.k_page + in * p.k_row;
            voff = page[it] * p.v_page + in * p.v_row;
          } else {
            koff = pos[it] * p.k_row;
            voff = pos[it] * p.v_row;
          }
        }
        if (c == 0) valid[buf * DEC_TILE + row] = ok_row ? 1 : 0;
        const uint32_t nbytes = ok_row ? 16u : 0u;
        const uint32_t dst_row = row * 128 + ((c ^ (row & 7)) << 4);
        const __nv_bfloat16* ksrc = kbase + koff + c * 8;
#pragma unroll
        for (int kb = 0; kb < DKB; ++kb) cp_async16(smem_u32(kb_s + kb * DEC_BLK + dst_row), ksrc + kb * 64, nbytes);
        if (!SHARED) {
          const __nv_bfloat16* vsrc = vbase + voff + c * 8;
#pragma unroll
          for (int kb = 0; kb < DVB; ++kb) cp_async16(smem_u32(vb_s + kb * DEC_BLK + dst_row), vsrc + kb * 64, nbytes);
        }
      }
      cp_async_commit();
      if (lane == 0) trace_mark(p, t, 2);
      cp_async_wait<0>();
      fence_proxy_async_smem();
      mbar_arrive(&full_bar[buf]);
      if (lane == 0) trace_mark(p, t, 3);
    }
    cp_async_wait<0>();
  } else if (warp == 6) {
    // ---------------------------------------------------------------- score MMAs (one thread)
    // The two GEMMs are issued by two different threads (this one and warp 7's): each only waits for what its own GEMM
    // needs, so the output MMAs of tile t are never queued behind the load of tile t+1 and a tile buffer is released as
    // early as the data flow allows.  They touch disjoint TMEM columns and never the same shared-memory tile at once.
    if (lane == 0) {
      constexpr uint32_t idesc1 = make_idesc(DEC_TILE, DEC_N, 1, 1, 0, 0);
      const uint64_t bdesc0 = make_smem_desc_sw128(smem_u32(qs), 16, 1024);
      for (int t = 0; t < T; ++t) {
        const int buf = t & 1;
        if (!mbar_wait(&full_bar[buf], (t >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_FULL)) break;
        trace_mark(p, t, 4);
        if (!mbar_wait(&sfree_bar[buf], ((t >> 1) & 1) ^ 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        trace_mark(p, t, 5);
        const uint64_t adesc0 = make_smem_desc_sw128(smem_u32(bufs + buf * Cfg::BUF_BYTES), 16, 1024);
#pragma unroll
        for (int kb = 0; kb < DKB; ++kb) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            // offsets are added to the descriptors' 16-byte-unit address field (all buffers sit below 256 KB: no carry)
            umma_f16(tmem_s + buf * DEC_N, adesc0 + ((kb * DEC_BLK + k * 32) >> 4), bdesc0 + ((kb * (DEC_N * 128) + k * 32) >> 4),
                     idesc1, (kb > 0 || k > 0) ? 1u : 0u);
          }
        }
        umma_commit(&sfull_bar[buf]);
        trace_mark(p, t, 6);
      }
    }
  } else if (warp == 7) {
    // ---------------------------------------------------------------- output MMAs (one thread)
    if (lane == 0) {
      constexpr uint32_t idesc2 = make_idesc(128, DEC_N, 1, 1, 1, 0);
      const uint64_t bdesc0 = make_smem_desc_sw128(smem_u32(ps), 16, 1024);
      for (int t = 0; t < T; ++t) {
        if (!mbar_wait(pfull_bar, t & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) break;
        tc_fence_after();
        trace_mark(p, t, 7);
        const uint32_t vb_s = smem_u32(bufs + (t & 1) * Cfg::BUF_BYTES + (SHARED ? 0 : DKB * DEC_BLK));
        const uint64_t adesc0 = make_smem_desc_sw128(vb_s, DEC_BLK, 1024);
#pragma unroll
        for (int j = 0; j < MB; ++j) {
#pragma unroll
          for (int k = 0; k < DEC_TILE / 16; ++k)
            umma_f16(tmem_o + j * DEC_N, adesc0 + (((2 * j) * DEC_BLK + k * 2048) >> 4), bdesc0 + ((k * 32) >> 4), idesc2,
                     (t > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&empty_bar[t & 1]);
        umma_commit(odone_bar);
        trace_mark(p, t, 8);
      }
    }
  } else if (warp < 4) {
    // ---------------------------------------------------------------- softmax / read-back (128 threads)
    const int tid = threadIdx.x;                       // TMEM lane
    const bool key_lane = lane < 16;                   // M = 64 accumulators sit in lanes 0-15 of every lane quarter
    const int key = warp * 16 + lane;                  // key within the tile (meaningful when key_lane)
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    float m_ref[DEC_N], l_part[DEC_N];
#pragma unroll
    for (int h = 0; h < DEC_N; ++h) {
      m_ref[h] = -INFINITY;
      l_part[h] = 0.f;
    }
    bool ok = true;
    for (int t = 0; t < T && ok; ++t) {
      const int buf = t & 1;
      // Exit decisions are taken at the two barriers below so that all 128 threads leave the loop together.
      bool got = mbar_wait(&sfull_bar[buf], (t >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL);
      tc_fence_after();
      if (tid == 0) trace_mark(p, t, 9);
      uint32_t sr[16];
      tmem_ld_x16(tmem_s + buf * DEC_N + lane_addr, sr);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(&sfree_bar[buf]);
      const bool kvalid = key_lane && valid[buf * DEC_TILE + key] != 0;
      float s[DEC_N];
#pragma unroll
      for (int h = 0; h < DEC_N; ++h) {
        s[h] = kvalid ? __uint_as_float(sr[h]) * p.scale_log2 : -INFINITY;
        const float wm = order_float(__reduce_max_sync(0xffffffffu, float_order(s[h])));
        if (lane == h) wmax[warp * DEC_N + h] = wm;
      }
      if (!named_bar_and(1, 128, got)) {
        ok = false;
        break;
      }
      if (tid == 0) trace_mark(p, t, 10);
      float alpha[DEC_N];
      bool rescale = false;
#pragma unroll
      for (int h = 0; h < DEC_N; ++h) {
        const float tm = fmaxf(fmaxf(wmax[h], wmax[DEC_N + h]), fmaxf(wmax[2 * DEC_N + h], wmax[3 * DEC_N + h]));
        alpha[h] = 1.f;
        if (tm > m_ref[h] + DEC_RESCALE_THRESHOLD || (m_ref[h] == -INFINITY && tm > -INFINITY)) {
          alpha[h] = m_ref[h] == -INFINITY ? 0.f : exp2f(m_ref[h] - tm);
          if (m_ref[h] != -INFINITY) rescale = true;
          m_ref[h] = tm;
          l_part[h] *= alpha[h];
        }
      }
      got = t == 0 || mbar_wait(odone_bar, (t - 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY);
      if (!named_bar_and(2, 128, got)) {  // also: wmax may be overwritten by the next tile only after everyone has read it
        ok = false;
        break;
      }
      if (tid == 0) trace_mark(p, t, 11);
      if (t > 0) {
        tc_fence_after();
        if (rescale) {  // uniform over the 128 threads: every thread derived it from the same shared values
#pragma unroll
          for (int j = 0; j < MB; ++j) {
            uint32_t o[16];
            tmem_ld_x16(tmem_o + j * DEC_N + lane_addr, o);
            tmem_wait_ld();
#pragma unroll
            for (int h = 0; h < DEC_N; ++h) o[h] = __float_as_uint(__uint_as_float(o[h]) * alpha[h]);
            asm volatile(
                "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, "
                "%14, %15, %16};" ::"r"(tmem_o + j * DEC_N + lane_addr),
                "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]), "r"(o[8]),
                "r"(o[9]), "r"(o[10]), "r"(o[11]), "r"(o[12]), "r"(o[13]), "r"(o[14]), "r"(o[15])
                : "memory");
          }
          tmem_wait_st();
        }
      }
      if (key_lane) {
        const int chunk = key >> 3, within = (key & 7) * 2;
#pragma unroll
        for (int h = 0; h < DEC_N; ++h) {
          const float pv = s[h] == -INFINITY ? 0.f : exp2f(s[h] - m_ref[h]);
          const __nv_bfloat16 pb = __float2bfloat16(pv);
          l_part[h] += __bfloat162float(pb);     // the denominator sums exactly what the tensor cores multiply
          *reinterpret_cast<__nv_bfloat16*>(ps + h * 128 + ((chunk ^ (h & 7)) << 4) + within) = pb;
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(pfull_bar);
      if (tid == 0) trace_mark(p, t, 12);
    }
    // ------------------------------------------------------------ partial results
    if (ok) ok = mbar_wait(odone_bar, (T - 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL);
    ok = named_bar_and(1, 128, ok);
    if (ok) {
      tc_fence_after();
#pragma unroll
      for (int h = 0; h < DEC_N; ++h) {
        const float ws = warp_sum(key_lane ? l_part[h] : 0.f);
        if (lane == h) wsum[warp * DEC_N + h] = ws;
      }
      named_bar_sync(1, 128);
      if (tid < nh) {
        const long long r = ws_row + static_cast<long long>(tid) * p.splits;
        p.ws_l[r] = wsum[tid] + wsum[DEC_N + tid] + wsum[2 * DEC_N + tid] + wsum[3 * DEC_N + tid];
        float mine = -INFINITY;   // m_ref is identical in every thread; select without dynamic register indexing
#pragma unroll
        for (int h = 0; h < DEC_N; ++h)
          if (h == tid) mine = m_ref[h];
        p.ws_m[r] = mine;
      }
#pragma unroll
      for (int j = 0; j < MB; ++j) {
        uint32_t o[16];
        tmem_ld_x16(tmem_o + j * DEC_N + lane_addr, o);
        tmem_wait_ld();
#pragma unroll
        for (int h = 0; h < DEC_N; ++h)
          if (h < nh) p.ws_o[(ws_row + static_cast<long long>(h) * p.splits) * DV + j * 128 + tid] = __uint_as_float(o[h]);
      }
    }
  }
  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 6) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// out[b,h,:] = Σ_s o_s · 2^(m_s − M) / Σ_s l_s · 2^(m_s − M); zeros when no split saw a valid key. One block per (b,h).
__global__ void decode_combine_kernel(const float* __restrict__ ws_o, const float* __restrict__ ws_m,
                                      const float* __restrict__ ws_l, __nv_bfloat16* __restrict__ out, float* __restrict__ lse,
                                      int splits, int DV) {
  const long long bh = blockIdx.x;
  const float* m = ws_m + bh * splits;
  const float* l = ws_l + bh * splits;
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, m[s]);
  float denom = 0.f;
  for (int s = 0; s < splits; ++s) denom += m[s] == -INFINITY ? 0.f : l[s] * exp2f(m[s] - M);
  const float inv = denom > 0.f ? 1.f / denom : 0.f;
  for (int d = threadIdx.x; d < DV; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s)
      if (m[s] != -INFINITY) acc += ws_o[(bh * splits + s) * DV + d] * exp2f(m[s] - M);
    out[bh * DV + d] = __float2bfloat16(acc * inv);
  }
  if (lse != nullptr && threadIdx.x == 0) lse[bh] = denom > 0.f ? (M + log2f(denom)) * 0.6931471805599453f : -INFINITY;
}

}  // namespace cmb

namespace {

long long* g_decode_trace = nullptr;

// 4-D map over a cache: (columns, kv heads, rows per page | cache length, pages | batch); strides in elements.
int make_tmap_cache(CUtensorMap* out, const void* base, int cols, int kv_heads, long long ext2, long long ext3, long long s_head,
                    long long s_row, long long s_outer, int box_rows) {
  cmb_host::EncodeTiledFn fn = cmb_host::encode_tiled_fn();
  if (fn == nullptr) return 101;
  cmb_host::bind_context_once();
  if (reinterpret_cast<uintptr_t>(base) & 15) return 102;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(kv_heads), static_cast<cuuint64_t>(ext2),
                        static_cast<cuuint64_t>(ext3)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>((kv_heads > 1 ? s_head : s_row) * 2), static_cast<cuuint64_t>(s_row * 2),
                           static_cast<cuuint64_t>((ext3 > 1 ? s_outer : s_row * ext2) * 2)};
  for (int i = 0; i < 3; ++i)
    if (strides[i] == 0 || (strides[i] & 15)) return 105;
  cuuint32_t box[4] = {64, 1, static_cast<cuuint32_t>(box_rows), 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1000 + static_cast<int>(r);
}

template <int DKB, int DVB, bool SHARED>
int launch_decode(cmb::DecodeParams& p, long long ext2, long long ext3, cudaStream_t stream) {
  using Cfg = cmb::DecCfg<DKB, DVB, SHARED>;
  auto kern = cmb::paged_decode_kernel<DKB, DVB, SHARED>;
  static std::atomic<unsigned long long> attr_done{0};
  if (cmb_host::set_smem_limit_once_per_device(attr_done, reinterpret_cast<const void*>(kern), Cfg::SMEM_BYTES)) return 103;
  // Dense key ranges whose 64-key tiles decompose into whole boxes inside one page go through TMA.
  const bool paged = p.table != nullptr;
  const int ps = p.page_size;
  p.tma = p.topk == nullptr && ext2 > 0 && ext3 > 0 &&
          (!paged || (ps % 8 == 0 && (ps >= cmb::DEC_TILE ? ps % cmb::DEC_TILE == 0 : cmb::DEC_TILE % ps == 0)));
  p.box_rows = paged && ps < cmb::DEC_TILE ? ps : cmb::DEC_TILE;
  CUtensorMap tmK, tmV;
  memset(&tmK, 0, sizeof(tmK));
  memset(&tmV, 0, sizeof(tmV));
  if (p.tma) {
    int rc = make_tmap_cache(&tmK, p.k, DKB * 64, p.kv_heads, ext2, ext3, p.k_head, p.k_row, paged ? p.k_page : p.k_batch, p.box_rows);
    if (rc == 0 && !SHARED)
      rc = make_tmap_cache(&tmV, p.v, DVB * 64, p.kv_heads, ext2, ext3, p.v_head, p.v_row, paged ? p.v_page : p.v_batch, p.box_rows);
    if (rc != 0) p.tma = 0;   // fall back to the per-row gather (e.g. strides the tensor-map encoder refuses)
  }
  const int g = p.H / p.kv_heads;
  const int gchunks = (g + cmb::DEC_N - 1) / cmb::DEC_N;
  dim3 grid(p.splits, p.B, p.kv_heads * gchunks);
  // The second pair of gather warps only exists in per-row mode; without it two CTAs of the small variants fit an SM's registers.
  kern<<<grid, p.tma ? 256 : cmb::DEC_THREADS, Cfg::SMEM_BYTES, stream>>>(tmK, tmV, p);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // namespace

// One decode step of attention for B sequences. q [B,H,Dk] bf16 (strides in elements), out [B,H,Dv] bf16 contiguous.
// ip = {B, H, kv_heads, Dk, Dv, shared_kv, table_w, page_size, topk_n, splits, ext2, ext3} (ext2 = rows per page or the
// contiguous cache's length, ext3 = pages in the pool or batch rows: the extents of the cache tensor, 0 = unknown); lp = {q_sb, q_sh, k_page, k_row, k_batch,
// k_head, v_page, v_row, v_batch, v_head} (elements). table / topk / v / lse may be null. Workspaces: ws_o
// [B,H,splits,Dv], ws_m and ws_l [B,H,splits] fp32. Returns 0, or 1 for an unsupported shape.
extern "C" int cmb_paged_decode(const void* q, const void* k, const void* v, const int* table, const int* lengths,
                                const int* topk, void* out, float* lse, float* ws_o, float* ws_m, float* ws_l,
                                const int* ip, const long long* lp, float scale, int* status, void* stream) {
  cmb::DecodeParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k = static_cast<const __nv_bfloat16*>(k);
  p.v = static_cast<const __nv_bfloat16*>(v);
  p.table = table;
  p.lengths = lengths;
  p.topk = topk;
  p.B = ip[0], p.H = ip[1], p.kv_heads = ip[2];
  const int Dk = ip[3], Dv = ip[4], shared = ip[5];
  p.table_w = ip[6], p.page_size = ip[7] > 0 ? ip[7] : 1, p.topk_n = ip[8], p.splits = ip[9];
  p.n_pages = table != nullptr ? ip[11] : 0;
  p.q_sb = lp[0], p.q_sh = lp[1];
  p.k_page = lp[2], p.k_row = lp[3], p.k_batch = lp[4], p.k_head = lp[5];
  p.v_page = lp[6], p.v_row = lp[7], p.v_batch = lp[8], p.v_head = lp[9];
  p.scale_log2 = scale * 1.4426950408889634f;
  p.ws_o = ws_o, p.ws_m = ws_m, p.ws_l = ws_l, p.status = status;
  p.trace = g_decode_trace;
  if (p.B <= 0 || p.H <= 0 || p.kv_heads <= 0 || p.H % p.kv_heads || p.splits <= 0 || p.splits > 65535) return 1;
  if ((p.q_sb | p.q_sh | p.k_page | p.k_row | p.k_batch | p.k_head | p.v_page | p.v_row | p.v_batch | p.v_head) & 7) return 1;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15) return 1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc = 1;
  const long long e2 = ip[10], e3 = ip[11];
  if (shared && Dk == 576 && Dv == 512) rc = launch_decode<9, 8, true>(p, e2, e3, st);
  else if (!shared && v != nullptr && Dk == 128 && Dv == 128) rc = launch_decode<2, 2, false>(p, e2, e3, st);
  else if (!shared && v != nullptr && Dk == 192 && Dv == 128) rc = launch_decode<3, 2, false>(p, e2, e3, st);
  else if (!shared && v != nullptr && Dk == 64 && Dv == 128) rc = launch_decode<1, 2, false>(p, e2, e3, st);
  else if (!shared && v != nullptr && Dk == 256 && Dv == 256) rc = launch_decode<4, 4, false>(p, e2, e3, st);
  if (rc) return rc;
  cmb::decode_combine_kernel<<<static_cast<unsigned>(p.B) * p.H, 128, 0, st>>>(ws_o, ws_m, ws_l, static_cast<__nv_bfloat16*>(out),
                                                                              lse, p.splits, Dv);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// Diagnostic: subsequent launches of the decode kernel record SM-clock samples of CTA 0 into `buf`
// (int64[64 tiles][16 slots]: 0 indices ready, 1 buffer released, 2 copies issued, 3 copies landed, 4 MMA saw the tile,
// 5 score buffer free, 6 score MMAs issued, 7 P ready, 8 output MMAs issued, 9 scores ready, 10 max exchanged,
// 11 previous output done, 12 P written). Pass null to switch it off.
extern "C" void cmb_paged_decode_set_trace(long long* buf) { g_decode_trace = buf; }
