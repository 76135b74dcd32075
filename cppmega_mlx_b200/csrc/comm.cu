// Kernels that talk to peer GPUs through symmetric memory over NVLink / NVSwitch.  Every rank maps every peer's
// buffers, so `bufs[r]` below is rank r's copy of the same logical buffer.  Two forms of the ZeRO-1 kernels exist: plain
// peer loads and stores (one per rank), and — when the buffers are bound to an NVSwitch multicast object and the caller asks
// for it — `multimem.ld_reduce` (the switch adds the W ranks' gradients, one load per 16 bytes) and `multimem.st` (one store
// reaches every rank's parameter buffer).
//
//  * cmb_comm_barrier        epoch-flag barrier: release-store my epoch into every peer's pad, acquire-poll my pad.
//                            The poll is bounded; on expiry a status word is set and the kernel returns.
//  * cmb_zero1_adamw_ranges ZeRO-1 for AdamW-owned tensors in ONE kernel over a table of ranges: sum the W peers' bf16
//                            gradients of each owned range (the reduce-scatter), bf16→fp32, AdamW on local fp32 moments,
//                            and push the new bf16 parameters into every rank's parameter buffer (the all-gather).
//  * cmb_zero1_muon_reduce_ranges  same gradient reduction fused with Muon's momentum stage: writes the bf16 Newton–Schulz
//                            input and per-block partial sums of its squared norm (added in fixed order by
//                            cmb_zero1_sumsq_finalize).
//  * cmb_zero1_push_update   p ← p − coef·u for an owned tensor, stored to every rank (all-gather side of Muon).
//
// These replace the reference's per-leaf all_sum for gradients and its all_sum-of-zero-padded-shards "gather"
// (cppmega_mlx/training/distributed_optimizer.py:302-324, :326-391).
#include "sm100.cuh"

namespace cmb {

constexpr int COMM_MAX_RANKS = 16;

struct PeerPtrs {
  void* p[COMM_MAX_RANKS];
  void* mc;   // multicast address of the same buffer (one access reaches every rank's copy), or nullptr
};

__device__ __forceinline__ void st_release_sys(int* addr, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// pads[r] = rank r's int32[COMM_MAX_RANKS] flag block. Thread t signals peer t and waits for peer t.
__global__ void comm_barrier_kernel(PeerPtrs pads, int rank, int world, int epoch, long long spin_limit, int* status) {
  const int t = threadIdx.x;
  if (t < world) {
    __threadfence_system();
    st_release_sys(static_cast<int*>(pads.p[t]) + rank, epoch);
    const int* mine = static_cast<const int*>(pads.p[rank]) + t;
    bool ok = false;
    for (long long i = 0; i < spin_limit; ++i) {
      if (ld_acquire_sys(mine) >= epoch) {
        ok = true;
        break;
      }
      __nanosleep(64);
    }
    if (!ok && status != nullptr && atomicCAS(status, 0, ST_TIMEOUT_PEER_FLAG) == 0) {
      status[1] = rank;
      status[2] = t;
      status[3] = epoch;
    }
    __threadfence_system();
  }
}

__device__ __forceinline__ void unpack8(const uint4& q, float (&f)[8]) {
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(b[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  v.x = pack_bf16x2(f[0], f[1]);
  v.y = pack_bf16x2(f[2], f[3]);
  v.z = pack_bf16x2(f[4], f[5]);
  v.w = pack_bf16x2(f[6], f[7]);
  return v;
}

// Sum over all ranks of 8 consecutive bf16 values at a multicast address (fp32 accumulation in the switch, bf16 result).
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
// 16 bytes to every rank's copy.
__device__ __forceinline__ void multimem_st_16(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
// 16 bytes at element offset `e` to every rank: one multicast store, or one store per peer.
__device__ __forceinline__ void store_all_16(const PeerPtrs& bufs, int world, long long e, const uint4& v) {
  if (bufs.mc != nullptr) {
    multimem_st_16(static_cast<__nv_bfloat16*>(bufs.mc) + e, v);
  } else {
    for (int r = 0; r < world; ++r) *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(bufs.p[r]) + e) = v;
  }
}

// Sum of the W ranks' gradients for 8 consecutive elements starting at flat offset `e` (16-byte aligned).
__device__ __forceinline__ void reduce8(const PeerPtrs& grads, int world, long long e, float inv_world, float (&g)[8]) {
  if (grads.mc != nullptr) {
    unpack8(multimem_ld_reduce_bf16x8(static_cast<const __nv_bfloat16*>(grads.mc) + e), g);
#pragma unroll
    for (int i = 0; i < 8; ++i) g[i] *= inv_world;
    return;
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) g[i] = 0.f;
  for (int r = 0; r < world; ++r) {
    const uint4 q = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(grads.p[r]) + e);
    float f[8];
    unpack8(q, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) g[i] += f[i];
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) g[i] *= inv_world;
}

// Eight consecutive fp32 state values as two 16-byte accesses (state tensors are 32-byte aligned at multiples of 8 elements).
__device__ __forceinline__ void ld8f(const float* p, float (&x)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}
__device__ __forceinline__ void st8f(float* p, const float (&x)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(x[4], x[5], x[6], x[7]);
}

__global__ void __launch_bounds__(256) zero1_push_update_kernel(PeerPtrs params, int rank, int world, long long off,
                                                                 long long n, const __nv_bfloat16* __restrict__ u,
                                                                 float coef) {
  const long long nvec = n >> 3;
  const __nv_bfloat16* myp = static_cast<const __nv_bfloat16*>(params.p[rank]);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e = off + 8 * i;
    float p[8], d[8];
    unpack8(*reinterpret_cast<const uint4*>(myp + e), p);
    unpack8(*reinterpret_cast<const uint4*>(u + 8 * i), d);
#pragma unroll
    for (int k = 0; k < 8; ++k) p[k] -= coef * d[k];
    store_all_16(params, world, e, pack8(p));
  }
}

// ---------------------------------------------------------------------------------------------- bucketed, overlappable forms
// A bucket is a set of tensors whose gradients become final together (one layer).  As soon as a rank's backward pass has
// produced them it raises its flag for the bucket in every peer's flag block; the owner's kernel for that bucket waits
// (bounded) until all W flags show the current step, then reduces the peers' gradients of the ranges it owns, updates and —
// for AdamW ranges — pushes the new parameters to every rank, all while the backward pass of the earlier layers is still
// running on the main stream.  No rank reads a bucket's weights again in the same backward pass once its flag is up, so the
// early parameter push is safe.  `ranges` is a device table; a launch covers all ranges of one bucket.
constexpr int Z1_PARTS = 148 * 4;      // the grid cap of the range kernels (comm_grid)
struct Z1Range {
  long long off;          // element offset inside the flat buffers (multiple of 8)
  long long n;            // elements
  float* s0;              // AdamW m / Muon momentum
  float* s1;              // AdamW v
  __nv_bfloat16* u;       // Muon: Newton–Schulz input (reduce) / orthogonalised update (push)
  float* sumsq;           // Muon: this tensor's row of Z1_PARTS per-block partial sums of u² (block b writes slot b)
  float coef;             // push: shape factor of the learning rate
  int pad;
};

// All threads of the block return the same verdict. flags = my flag block + bucket·COMM_MAX_RANKS.
__device__ __forceinline__ bool wait_bucket_flags(const int* flags, int world, int epoch, long long spin_limit, int* status, int rank, int bucket) {
  bool ok = true;
  if (flags != nullptr && threadIdx.x < world) {
    ok = false;
    for (long long i = 0; i < spin_limit; ++i) {
      if (ld_acquire_sys(flags + threadIdx.x) >= epoch) {
        ok = true;
        break;
      }
      __nanosleep(128);
    }
    if (!ok && status != nullptr && atomicCAS(status, 0, ST_TIMEOUT_PEER_FLAG) == 0) {
      status[1] = rank;
      status[2] = threadIdx.x;
      status[3] = (bucket << 20) | (epoch & 0xfffff);
    }
    __threadfence_system();
  }
  return __syncthreads_and(ok);
}

__global__ void zero1_bucket_signal_kernel(PeerPtrs pads, int rank, int world, int bucket, int epoch) {
  const int t = threadIdx.x;
  if (t < world) {
    __threadfence_system();       // this rank's gradient stores of the bucket (ordered before this launch on the stream) are visible first
    st_release_sys(static_cast<int*>(pads.p[t]) + bucket * COMM_MAX_RANKS + rank, epoch);
  }
}

__global__ void __launch_bounds__(256) zero1_adamw_ranges_kernel(PeerPtrs grads, PeerPtrs params, int rank, int world, const Z1Range* __restrict__ ranges,
                                                                  int nranges, float lr, float b1, float b2, float eps, float wd, float c1, float c2,
                                                                  float inv_world, const int* flags, int bucket, int epoch, long long spin_limit,
                                                                  int* status) {
  if (!wait_bucket_flags(flags, world, epoch, spin_limit, status, rank, bucket)) return;
  const __nv_bfloat16* myp = static_cast<const __nv_bfloat16*>(params.p[rank]);
  for (int ri = 0; ri < nranges; ++ri) {
    const Z1Range rg = ranges[ri];
    const long long nvec = rg.n >> 3;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec; i += static_cast<long long>(gridDim.x) * blockDim.x) {
      const long long e = rg.off + 8 * i;
      float g[8], p[8], mm[8], vv[8];
      reduce8(grads, world, e, inv_world, g);
      unpack8(*reinterpret_cast<const uint4*>(myp + e), p);
      ld8f(rg.s0 + 8 * i, mm);
      ld8f(rg.s1 + 8 * i, vv);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        mm[k] = b1 * mm[k] + (1.f - b1) * g[k];
        vv[k] = b2 * vv[k] + (1.f - b2) * g[k] * g[k];
        p[k] = p[k] * (1.f - lr * wd) - lr * c1 * mm[k] / (sqrtf(vv[k]) * c2 + eps);
      }
      st8f(rg.s0 + 8 * i, mm);
      st8f(rg.s1 + 8 * i, vv);
      store_all_16(params, world, e, pack8(p));
    }
    for (long long j = (nvec << 3) + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; j < rg.n; j += static_cast<long long>(gridDim.x) * blockDim.x) {
      float g = 0.f;
      for (int r = 0; r < world; ++r) g += __bfloat162float(static_cast<const __nv_bfloat16*>(grads.p[r])[rg.off + j]);
      g *= inv_world;
      const float mi = b1 * rg.s0[j] + (1.f - b1) * g;
      const float vi = b2 * rg.s1[j] + (1.f - b2) * g * g;
      rg.s0[j] = mi;
      rg.s1[j] = vi;
      const __nv_bfloat16 o = __float2bfloat16(__bfloat162float(myp[rg.off + j]) * (1.f - lr * wd) - lr * c1 * mi / (sqrtf(vi) * c2 + eps));
      for (int r = 0; r < world; ++r) static_cast<__nv_bfloat16*>(params.p[r])[rg.off + j] = o;
    }
  }
}

__global__ void __launch_bounds__(256) zero1_muon_reduce_ranges_kernel(PeerPtrs grads, PeerPtrs params, int rank, int world,
                                                                        const Z1Range* __restrict__ ranges, int nranges, float mu, float wd, int nesterov,
                                                                        float inv_world, const int* flags, int bucket, int epoch, long long spin_limit,
                                                                        int* status) {
  __shared__ float red[8];
  if (!wait_bucket_flags(flags, world, epoch, spin_limit, status, rank, bucket)) return;
  const __nv_bfloat16* myp = static_cast<const __nv_bfloat16*>(params.p[rank]);
  for (int ri = 0; ri < nranges; ++ri) {
    const Z1Range rg = ranges[ri];
    const long long nvec = rg.n >> 3;
    float acc = 0.f;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec; i += static_cast<long long>(gridDim.x) * blockDim.x) {
      const long long e = rg.off + 8 * i;
      float g[8], p[8], o[8], vv[8];
      reduce8(grads, world, e, inv_world, g);
      unpack8(*reinterpret_cast<const uint4*>(myp + e), p);
      ld8f(rg.s0 + 8 * i, vv);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float gi = g[k] + wd * p[k];
        vv[k] = mu * vv[k] + (1.f - mu) * gi;
        o[k] = nesterov ? gi * (1.f - mu) + vv[k] * mu : vv[k];
        acc += o[k] * o[k];
      }
      st8f(rg.s0 + 8 * i, vv);
      *reinterpret_cast<uint4*>(rg.u + 8 * i) = pack8(o);
    }
    acc = warp_sum(acc);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int w = 0; w < 8; ++w) t += red[w];
      rg.sumsq[blockIdx.x] = t;      // no atomics: the finalize kernel adds the row in a fixed order, so a step is reproducible bit for bit
    }
  }
}

// sumsq[t] = Σ_b partials[t][b] in a fixed order, and the row is cleared for the next step.  One block per tensor.
__global__ void __launch_bounds__(256) zero1_sumsq_finalize_kernel(float* __restrict__ partials, float* __restrict__ sumsq) {
  __shared__ float red[8];
  float* row = partials + static_cast<long long>(blockIdx.x) * Z1_PARTS;
  float acc = 0.f;
  for (int i = threadIdx.x; i < Z1_PARTS; i += 256) {
    acc += row[i];
    row[i] = 0.f;
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += red[w];
    sumsq[blockIdx.x] = t;
  }
}

__global__ void __launch_bounds__(256) zero1_push_ranges_kernel(PeerPtrs params, int rank, int world, const Z1Range* __restrict__ ranges, int nranges,
                                                                 float lr) {
  const __nv_bfloat16* myp = static_cast<const __nv_bfloat16*>(params.p[rank]);
  for (int ri = 0; ri < nranges; ++ri) {
    const Z1Range rg = ranges[ri];
    const long long nvec = rg.n >> 3;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec; i += static_cast<long long>(gridDim.x) * blockDim.x) {
      const long long e = rg.off + 8 * i;
      float p[8], d[8];
      unpack8(*reinterpret_cast<const uint4*>(myp + e), p);
      unpack8(*reinterpret_cast<const uint4*>(rg.u + 8 * i), d);
#pragma unroll
      for (int k = 0; k < 8; ++k) p[k] -= lr * rg.coef * d[k];
      store_all_16(params, world, e, pack8(p));
    }
  }
}

// ---------------------------------------------------------------------------------------------- stand-alone all-reduce
// Sum of every rank's copy of a symmetric buffer, left in every rank's copy.  The caller brackets the launch with the epoch
// barrier (all inputs written before, all outputs visible after).  Rank r reduces the r-th slice of 16-byte vectors and
// publishes it to everyone (a reduce-scatter and an all-gather in one pass):
//   multimem form — one `multimem.ld_reduce` (the switch adds the W copies) and one `multimem.st` (the switch replicates) per
//                   vector: this GPU receives one vector and sends one, whatever W is;
//   peer form     — W loads (fixed rank order: bitwise reproducible) and W stores per vector.
// `dtype`: 0 = fp32 (4 elements per vector), 1 = bf16 (8 per vector, fp32 accumulation).
template <int DTYPE>
__global__ void __launch_bounds__(256) allreduce_kernel(PeerPtrs bufs, int rank, int world, long long nvec) {
  const long long per = (nvec + world - 1) / world;
  const long long lo = rank * per, hi = min(nvec, lo + per);
  for (long long i = lo + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < hi; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    uint4 out;
    if (bufs.mc != nullptr) {
      const char* a = static_cast<const char*>(bufs.mc) + i * 16;
      if (DTYPE == 1) {
        out = multimem_ld_reduce_bf16x8(a);
      } else {
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(out.x), "=r"(out.y), "=r"(out.z), "=r"(out.w)
                     : "l"(a)
                     : "memory");
      }
      multimem_st_16(static_cast<char*>(bufs.mc) + i * 16, out);
    } else {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < world; ++r) {
        const uint4 q = *(static_cast<const uint4*>(bufs.p[r]) + i);
        if (DTYPE == 1) {
          float f[8];
          unpack8(q, f);
#pragma unroll
          for (int k = 0; k < 8; ++k) acc[k] += f[k];
        } else {
          acc[0] += __uint_as_float(q.x); acc[1] += __uint_as_float(q.y); acc[2] += __uint_as_float(q.z); acc[3] += __uint_as_float(q.w);
        }
      }
      out = DTYPE == 1 ? pack8(acc) : make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]), __float_as_uint(acc[3]));
      for (int r = 0; r < world; ++r) *(static_cast<uint4*>(bufs.p[r]) + i) = out;
    }
  }
}

static inline int comm_grid(long long nvec) {
  long long b = (nvec + 255) / 256;
  const long long cap = Z1_PARTS;
  return static_cast<int>(b < 1 ? 1 : (b > cap ? cap : b));
}
// `ptrs` holds the W peer addresses; with `use_mc` it holds one more entry, the multicast address (0 = none).
static inline bool fill(PeerPtrs& out, const long long* ptrs, int world, int use_mc = 0) {
  if (world < 1 || world > COMM_MAX_RANKS) return false;
  for (int r = 0; r < COMM_MAX_RANKS; ++r) out.p[r] = r < world ? reinterpret_cast<void*>(ptrs[r]) : nullptr;
  out.mc = use_mc ? reinterpret_cast<void*>(ptrs[world]) : nullptr;
  return true;
}

}  // namespace cmb

extern "C" int cmb_comm_barrier(const long long* pad_ptrs, int rank, int world, int epoch, long long spin_limit,
                                int* status, void* stream) {
  cmb::PeerPtrs pads;
  if (!cmb::fill(pads, pad_ptrs, world)) return 1;
  cmb::comm_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(pads, rank, world, epoch, spin_limit, status);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}



extern "C" int cmb_zero1_push_update(const long long* param_ptrs, int rank, int world, long long off, long long n,
                                     const void* u, float coef, void* stream) {
  cmb::PeerPtrs p;
  if (!cmb::fill(p, param_ptrs, world) || (off & 7) || (n & 7)) return 1;
  if (n <= 0) return 0;
  cmb::zero1_push_update_kernel<<<cmb::comm_grid(n / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      p, rank, world, off, n, static_cast<const __nv_bfloat16*>(u), coef);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// ---- bucketed forms. With `use_mc` the pointer arrays of the gradient and parameter buffers carry one more entry, the buffer's
// multicast address, and the vector paths use `multimem` (the scalar tails keep plain peer accesses).  `ranges`: device array of {off, n (int64), s0, s1, u, sumsq (pointers), coef (fp32), pad} (56 bytes → 56, 8-byte aligned);
// `flag_ptrs[r]`: rank r's int32[nbuckets · 16] flag block; a negative `bucket` skips the flag wait (the caller has synchronised already).
extern "C" int cmb_zero1_bucket_signal(const long long* flag_ptrs, int rank, int world, int bucket, int epoch, void* stream) {
  cmb::PeerPtrs pads;
  if (!cmb::fill(pads, flag_ptrs, world) || bucket < 0) return 1;
  cmb::zero1_bucket_signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(pads, rank, world, bucket, epoch);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

extern "C" int cmb_zero1_adamw_ranges(const long long* grad_ptrs, const long long* param_ptrs, const long long* flag_ptrs, int rank, int world,
                                      const void* ranges, int nranges, long long total_elems, const float* f, int bucket, int epoch,
                                      long long spin_limit, int* status, int max_blocks, int use_mc, void* stream) {
  cmb::PeerPtrs g, p, fl;
  if (!cmb::fill(g, grad_ptrs, world, use_mc) || !cmb::fill(p, param_ptrs, world, use_mc)) return 1;
  if (nranges <= 0) return 0;
  const int* flags = nullptr;
  if (bucket >= 0) {
    if (!cmb::fill(fl, flag_ptrs, world)) return 1;
    flags = static_cast<const int*>(fl.p[rank]) + bucket * cmb::COMM_MAX_RANKS;
  }
  int grid = cmb::comm_grid((total_elems + 7) / 8);
  if (max_blocks > 0 && grid > max_blocks) grid = max_blocks;
  cmb::zero1_adamw_ranges_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      g, p, rank, world, static_cast<const cmb::Z1Range*>(ranges), nranges, f[0], f[1], f[2], f[3], f[4], f[5], f[6], 1.f / world, flags, bucket, epoch,
      spin_limit, status);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

extern "C" int cmb_zero1_muon_reduce_ranges(const long long* grad_ptrs, const long long* param_ptrs, const long long* flag_ptrs, int rank, int world,
                                            const void* ranges, int nranges, long long total_elems, float mu, float wd, int nesterov, int bucket,
                                            int epoch, long long spin_limit, int* status, int max_blocks, int use_mc, void* stream) {
  cmb::PeerPtrs g, p, fl;
  if (!cmb::fill(g, grad_ptrs, world, use_mc) || !cmb::fill(p, param_ptrs, world)) return 1;
  if (nranges <= 0) return 0;
  const int* flags = nullptr;
  if (bucket >= 0) {
    if (!cmb::fill(fl, flag_ptrs, world)) return 1;
    flags = static_cast<const int*>(fl.p[rank]) + bucket * cmb::COMM_MAX_RANKS;
  }
  int grid = cmb::comm_grid(total_elems / 8);
  if (max_blocks > 0 && grid > max_blocks) grid = max_blocks;
  cmb::zero1_muon_reduce_ranges_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      g, p, rank, world, static_cast<const cmb::Z1Range*>(ranges), nranges, mu, wd, nesterov, 1.f / world, flags, bucket, epoch, spin_limit, status);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

extern "C" int cmb_zero1_sumsq_finalize(float* partials, float* sumsq, int ntensors, void* stream) {
  if (ntensors <= 0) return 0;
  cmb::zero1_sumsq_finalize_kernel<<<ntensors, 256, 0, static_cast<cudaStream_t>(stream)>>>(partials, sumsq);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

extern "C" int cmb_zero1_push_ranges(const long long* param_ptrs, int rank, int world, const void* ranges, int nranges, long long total_elems,
                                     float lr, int use_mc, void* stream) {
  cmb::PeerPtrs p;
  if (!cmb::fill(p, param_ptrs, world, use_mc)) return 1;
  if (nranges <= 0) return 0;
  cmb::zero1_push_ranges_kernel<<<cmb::comm_grid(total_elems / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      p, rank, world, static_cast<const cmb::Z1Range*>(ranges), nranges, lr);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// In-place all-reduce (sum) of a symmetric buffer of `nbytes` bytes (a multiple of 16); see allreduce_kernel.  `buf_ptrs` holds the W
// peer addresses followed, with `use_mc`, by the multicast address.  Bracket with cmb_comm_barrier on the same stream.
extern "C" int cmb_symm_allreduce(const long long* buf_ptrs, int rank, int world, long long nbytes, int dtype, int use_mc, void* stream) {
  cmb::PeerPtrs b;
  if (!cmb::fill(b, buf_ptrs, world, use_mc) || (nbytes & 15) || (dtype != 0 && dtype != 1)) return 1;
  if (nbytes <= 0) return 0;
  const long long nvec = nbytes / 16;
  const int grid = cmb::comm_grid((nvec + world - 1) / world);
  auto st = static_cast<cudaStream_t>(stream);
  if (dtype == 1)
    cmb::allreduce_kernel<1><<<grid, 256, 0, st>>>(b, rank, world, nvec);
  else
    cmb::allreduce_kernel<0><<<grid, 256, 0, st>>>(b, rank, world, nvec);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
