// bf16 GEMM on tcgen05 tensor cores (sm_100a), fp32 accumulation in TMEM.
//
//   C[M,N] (+)= A · Bᵀ      A: M×K, B: N×K, each either K-major (K contiguous, the natural
//                           layout of activations and nn.Linear weights) or MN-major (the
//                           contraction index is the slow one: what dgrad/wgrad see without
//                           any transposed copies).
//
// Structure: persistent CTAs (one per SM), 192 threads in three roles —
//   warp 0    TMA producer: fills a 4..6-deep ring of {A tile, B tile} stages (128-byte swizzle)
//   warp 1    MMA issuer  : one elected thread issues tcgen05.mma (128×BN×16) into one of two
//                           TMEM accumulators; tcgen05.commit hands stages back / signals the epilogue
//   warps 2-5 epilogue    : tcgen05.ld the finished accumulator, convert, store; overlaps with the
//                           mainloop of the next tile thanks to the double-buffered accumulator.
// Every mbarrier wait is bounded (see sm100.cuh); a timeout is reported through `status`.
//
// Takes the role of the reference's dense `mx.matmul` call sites ("Path A",
// docs/production_kernel_routing.md:62-140); there is no GEMM kernel in the reference to compare to.
#include <mutex>
#include <unordered_map>

#include "sm100.cuh"

namespace cmb {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;  // 64 bf16 = one 128-byte swizzle line
constexpr int GEMM_THREADS = 192;
constexpr int GEMM_GROUP_M = 16;

enum : int { GEMM_OUT_F32 = 1, GEMM_ACCUMULATE = 2 };

template <int BN>
struct GemmCfg {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
};

__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int& tm, int& tn) {
  const int per_group = GEMM_GROUP_M * num_n;
  const int g = t / per_group;
  const int first_m = g * GEMM_GROUP_M;
  const int gsz = min(num_m - first_m, GEMM_GROUP_M);
  const int r = t - g * per_group;
  tm = first_m + r % gsz;
  tn = r / gsz;
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, void* __restrict__ Cv,
                 int M, int N, int K, int ldc, int flags, int* __restrict__ status) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
  uint64_t* full_bar = bars;                 // [STAGES]
  uint64_t* empty_bar = bars + STAGES;       // [STAGES]
  uint64_t* tfull_bar = bars + 2 * STAGES;   // [2]
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (M + GEMM_BM - 1) / GEMM_BM;
  const int num_n = (N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (K + GEMM_BK - 1) / GEMM_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
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
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int tm, tn;
        tile_coords(t, num_m, num_n, tm, tn);
        const int m0 = tm * GEMM_BM, n0 = tn * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, status, ST_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
          const int k0 = kb * GEMM_BK;
          if (A_MN) {
#pragma unroll
            for (int i = 0; i < GEMM_BM / 64; ++i) tma_load_2d(sa + i * (GEMM_BK * 128), &tmA, &full_bar[stage], m0 + 64 * i, k0);
          } else {
            tma_load_2d(sa, &tmA, &full_bar[stage], k0, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i) tma_load_2d(sb + i * (GEMM_BK * 128), &tmB, &full_bar[stage], n0 + 64 * i, k0);
          } else {
            tma_load_2d(sb, &tmB, &full_bar[stage], k0, n0);
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
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(GEMM_BM, BN, 1, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++local) {
        const int buf = local & 1;
        const uint32_t aphase = (local >> 1) & 1;
        if (!mbar_wait(&tempty_bar[buf], aphase ^ 1, abort_flag, status, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
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
            umma_f16(tmem_d, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(&tfull_bar[buf]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (4 warps)
    const int quarter = warp & 3;  // TMEM lanes this warp may read
    const bool out_f32 = (flags & GEMM_OUT_F32) != 0;
    const bool accum = (flags & GEMM_ACCUMULATE) != 0;
    int local = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++local) {
      const int buf = local & 1;
      const uint32_t aphase = (local >> 1) & 1;
      if (!mbar_wait(&tfull_bar[buf], aphase, abort_flag, status, ST_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after();
      int tm, tn;
      tile_coords(t, num_m, num_n, tm, tn);
      const int row = tm * GEMM_BM + quarter * 32 + lane;
      const int n0 = tn * BN;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_x32(taddr + c * 32, r);
        tmem_wait_ld();
        const int col0 = n0 + c * 32;
        if (row < M && col0 < N) {
          if (out_f32) {
            float* dst = reinterpret_cast<float*>(Cv) + static_cast<size_t>(row) * ldc + col0;
            if (col0 + 32 <= N && (ldc & 3) == 0) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float4 v = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                       __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                if (accum) {
                  const float4 o = *reinterpret_cast<const float4*>(dst + 4 * j);
                  v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                }
                *reinterpret_cast<float4*>(dst + 4 * j) = v;
              }
            } else {
              for (int j = 0; j < 32 && col0 + j < N; ++j) {
                float v = __uint_as_float(r[j]);
                if (accum) v += dst[j];
                dst[j] = v;
              }
            }
          } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(Cv) + static_cast<size_t>(row) * ldc + col0;
            if (col0 + 32 <= N && (ldc & 7) == 0) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float f[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[8 * j + e]);
                if (accum) {
                  const uint4 o = *reinterpret_cast<const uint4*>(dst + 8 * j);
                  const __nv_bfloat162* ob = reinterpret_cast<const __nv_bfloat162*>(&o);
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float2 of = __bfloat1622float2(ob[e]);
                    f[2 * e] += of.x;
                    f[2 * e + 1] += of.y;
                  }
                }
                uint4 v;
                v.x = pack_bf16x2(f[0], f[1]);
                v.y = pack_bf16x2(f[2], f[3]);
                v.z = pack_bf16x2(f[4], f[5]);
                v.w = pack_bf16x2(f[6], f[7]);
                *reinterpret_cast<uint4*>(dst + 8 * j) = v;
              }
            } else {
              for (int j = 0; j < 32 && col0 + j < N; ++j) {
                float v = __uint_as_float(r[j]);
                if (accum) v += __bfloat162float(dst[j]);
                dst[j] = __float2bfloat16(v);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  if (*abort_flag) {
    // Give TMA copies / MMAs that may still be in flight a bounded time to land before the
    // shared memory and TMEM they target are released.
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

int make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint64_t ld,
                 uint32_t box_rows, uint32_t box_cols, int swizzle_bytes) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return 101;
  // The driver-API encoder needs a current context; a thread whose first CUDA call is this one (an autograd
  // worker, say) has none until a runtime call binds the primary context.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(nullptr);
    ctx_bound = true;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || ((ld * elem_bytes) & 15) != 0) return 102;
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                           : (elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8);
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapSwizzle sw = swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                          : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                          : swizzle_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B
                                                : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1000 + static_cast<int>(r);
}

static int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

template <int BN, bool A_MN, bool B_MN>
static int launch_gemm(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int flags,
                       int* status, int max_ctas, cudaStream_t stream) {
  using Cfg = cmb::GemmCfg<BN>;
  CUtensorMap tmA, tmB;
  int rc;
  // K-major operand stored [rows=M|N, cols=K]; MN-major operand stored [rows=K, cols=M|N].
  if (A_MN)
    rc = make_tmap_2d(&tmA, A, 2, K, M, lda, cmb::GEMM_BK, 64, 128);
  else
    rc = make_tmap_2d(&tmA, A, 2, M, K, lda, cmb::GEMM_BM, cmb::GEMM_BK, 128);
  if (rc) return rc;
  if (B_MN)
    rc = make_tmap_2d(&tmB, B, 2, K, N, ldb, cmb::GEMM_BK, 64, 128);
  else
    rc = make_tmap_2d(&tmB, B, 2, N, K, ldb, BN, cmb::GEMM_BK, 128);
  if (rc) return rc + 10;
  auto kern = cmb::gemm_bf16_kernel<BN, A_MN, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess) return 103;
    attr_set = true;
  }
  const int num_tiles = ((M + cmb::GEMM_BM - 1) / cmb::GEMM_BM) * ((N + BN - 1) / BN);
  int grid = sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (num_tiles < grid) grid = num_tiles;
  kern<<<grid, cmb::GEMM_THREADS, Cfg::SMEM_BYTES, stream>>>(tmA, tmB, C, M, N, K, ldc, flags, status);
  return cudaGetLastError() == cudaSuccess ? 0 : 104;
}

}  // namespace cmb_host

// C ABI. A is M×K (K-major, row pitch lda) or, with a_mn_major, stored K×M (row pitch lda).
// B is N×K (K-major) or, with b_mn_major, stored K×N. C is M×N row-major (pitch ldc), bf16 unless
// flags&1 (fp32); flags&2 accumulates into C. All pointers 16-byte aligned, pitches multiples of 8.
extern "C" int cmb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                             int a_mn_major, int b_mn_major, int flags, int* status, int max_ctas, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool big = N > 128;
#define CMB_GEMM_CASE(BN_, AM_, BM_) \
  return cmb_host::launch_gemm<BN_, AM_, BM_>(A, B, C, M, N, K, lda, ldb, ldc, flags, status, max_ctas, s)
  if (big) {
    if (!a_mn_major && !b_mn_major) CMB_GEMM_CASE(256, false, false);
    if (!a_mn_major && b_mn_major) CMB_GEMM_CASE(256, false, true);
    if (a_mn_major && !b_mn_major) CMB_GEMM_CASE(256, true, false);
    CMB_GEMM_CASE(256, true, true);
  } else {
    if (!a_mn_major && !b_mn_major) CMB_GEMM_CASE(128, false, false);
    if (!a_mn_major && b_mn_major) CMB_GEMM_CASE(128, false, true);
    if (a_mn_major && !b_mn_major) CMB_GEMM_CASE(128, true, false);
    CMB_GEMM_CASE(128, true, true);
  }
#undef CMB_GEMM_CASE
}
