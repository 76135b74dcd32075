// Tensor-parallel and expert-parallel helpers over symmetric memory (plain peer loads / stores over NVLink, sm_100a).
//
//  * cmb_sum_slots      out[i] = Σ_s slots[s·n + i] (+ residual[i]): the local half of GEMM → reduce-scatter.  The GEMM's
//                       epilogue has already TMA-stored every rank's partial tile for my rows into my slot buffer over NVLink.
//  * cmb_ep_dispatch    expert-parallel dispatch: gather token rows by index and store each one straight into the receive
//                       buffer of the rank that owns its expert, at the slot computed from the exchanged counts (the buffer
//                       is already in the padded expert-sorted layout the grouped GEMM consumes).
//  * cmb_ep_combine     the way back: for every token, load its k expert outputs from the peers' output buffers, weight them
//                       with the gate and add them up (no atomics: one warp owns one token).
//  * cmb_ep_combine_bwd backward of combine with respect to the gate weights: dw[t,j] = ⟨dout[t], y_peer[slot(t,j)]⟩.
// Every expert-parallel kernel takes the receive buffers' row capacity: a slot of −1 means "dropped by the routing plan" and
// is skipped silently; any other slot outside [0, rows) is a caller error that is reported through the status block and
// skipped, so no store or load ever leaves a peer's buffer.
//
// The reference has neither tensor nor expert parallelism (config fields only, cppmega_mlx/config/model.py:56-91).
#include "sm100.cuh"

namespace cmb {

constexpr int TE_MAX_RANKS = 16;
struct TePeers {
  void* p[TE_MAX_RANKS];
};

__global__ void __launch_bounds__(256) sum_slots_kernel(const __nv_bfloat16* __restrict__ slots, int nslots, long long n,
                                                         const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ out) {
  const long long nvec = n >> 3;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    for (int s = 0; s < nslots; ++s) {
      const uint4 q = *reinterpret_cast<const uint4*>(slots + s * n + 8 * i);
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(b[k]);
        acc[2 * k] += f.x;
        acc[2 * k + 1] += f.y;
      }
    }
    if (residual != nullptr) {
      const uint4 q = *reinterpret_cast<const uint4*>(residual + 8 * i);
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(b[k]);
        acc[2 * k] += f.x;
        acc[2 * k + 1] += f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + 8 * i) = o;
  }
}

// A slot outside [0, rows) or a rank outside [0, world) is never dereferenced: the first offender is recorded in the
// status block (code ST_BAD_ARGUMENT, then assignment index, slot, rank) and the access is skipped.
__device__ __forceinline__ void te_report(int* status, long long a, long long slot, int rank, int lane) {
  if (status != nullptr && lane == 0 && atomicCAS(status, 0, ST_BAD_ARGUMENT) == 0) {
    status[1] = static_cast<int>(a);
    status[2] = static_cast<int>(slot < 0x7fffffffLL ? slot : 0x7fffffffLL);
    status[3] = rank;
  }
}

// One warp per assignment a: row tok[a] of x (scaled by scale[a] if given) → peer dest_rank[a], row dest_slot[a] of its buffer.
__global__ void __launch_bounds__(256) ep_dispatch_kernel(const __nv_bfloat16* __restrict__ x, const long long* __restrict__ tok,
                                                           const int* __restrict__ dest_rank, const long long* __restrict__ dest_slot,
                                                           const float* __restrict__ scale, TePeers bufs, long long assignments, int d,
                                                           long long rows, int world, int* status) {
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long a = warp; a < assignments; a += nwarps) {
    const long long slot = dest_slot[a];
    const int dr = dest_rank[a];
    if (slot < 0) continue;                       // dropped by the routing plan (no capacity at the destination)
    if (slot >= rows || dr < 0 || dr >= world) {  // never address memory outside a receive buffer: record and skip
      te_report(status, a, slot, dr, lane);
      continue;
    }
    const __nv_bfloat16* src = x + tok[a] * d;
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(bufs.p[dr]) + slot * d;
    const float sc = scale != nullptr ? scale[a] : 1.f;
    for (int c = lane * 8; c < d; c += 256) {
      uint4 q = *reinterpret_cast<const uint4*>(src + c);
      if (scale != nullptr) {
        __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = __bfloat1622float2(b[k]);
          b[k] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
        }
      }
      *reinterpret_cast<uint4*>(dst + c) = q;
    }
  }
}

// One warp per token t: out[t] = Σ_j w[t,j] · ybuf[rank(t,j)][slot(t,j)]  (assignment index = t·k + j; a negative slot is skipped).
// `rows_out` (optional, [tokens·k, d]) also receives every gathered row unweighted (zeros for a skipped slot): what the backward
// pass of the weighted sum needs, written in the same pass instead of by a separate gather.
__global__ void __launch_bounds__(256) ep_combine_kernel(TePeers ybufs, const int* __restrict__ src_rank, const long long* __restrict__ src_slot,
                                                          const float* __restrict__ w, __nv_bfloat16* __restrict__ out, long long tokens, int k,
                                                          int d, long long rows, int world, int* status, __nv_bfloat16* __restrict__ rows_out) {
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long t = warp; t < tokens; t += nwarps) {
    for (int c = lane * 8; c < d; c += 256) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      for (int j = 0; j < k; ++j) {
        const long long a = t * k + j;
        const long long slot = src_slot[a];
        const int sr = src_rank[a];
        const bool bad = slot >= 0 && (slot >= rows || sr < 0 || sr >= world);
        if (slot < 0 || bad) {
          if (bad && c == lane * 8) te_report(status, a, slot, sr, lane);
          if (rows_out != nullptr) *reinterpret_cast<uint4*>(rows_out + a * d + c) = make_uint4(0u, 0u, 0u, 0u);
          continue;
        }
        const float wj = w != nullptr ? w[a] : 1.f;
        const uint4 q = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(ybufs.p[sr]) + slot * d + c);
        if (rows_out != nullptr) *reinterpret_cast<uint4*>(rows_out + a * d + c) = q;
        const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(b[i]);
          acc[2 * i] = fmaf(wj, f.x, acc[2 * i]);
          acc[2 * i + 1] = fmaf(wj, f.y, acc[2 * i + 1]);
        }
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(out + t * d + c) = o;
    }
  }
}

// One warp per assignment a = t·k + j: dw[a] = ⟨g[t], ybuf[rank(a)][slot(a)]⟩.
__global__ void __launch_bounds__(256) ep_combine_bwd_kernel(TePeers ybufs, const int* __restrict__ src_rank, const long long* __restrict__ src_slot,
                                                              const __nv_bfloat16* __restrict__ g, float* __restrict__ dw, long long assignments,
                                                              int k, int d, long long rows, int world, int* status) {
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long a = warp; a < assignments; a += nwarps) {
    const long long slot = src_slot[a];
    const int sr = src_rank[a];
    float acc = 0.f;
    if (slot >= 0 && (slot >= rows || sr < 0 || sr >= world)) {
      te_report(status, a, slot, sr, lane);
    } else if (slot >= 0) {
      const __nv_bfloat16* y = static_cast<const __nv_bfloat16*>(ybufs.p[sr]) + slot * d;
      const __nv_bfloat16* gr = g + (a / k) * d;
      for (int c = lane * 8; c < d; c += 256) {
        const uint4 qy = *reinterpret_cast<const uint4*>(y + c);
        const uint4 qg = *reinterpret_cast<const uint4*>(gr + c);
        const __nv_bfloat162* by = reinterpret_cast<const __nv_bfloat162*>(&qy);
        const __nv_bfloat162* bg = reinterpret_cast<const __nv_bfloat162*>(&qg);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 fy = __bfloat1622float2(by[i]), fg = __bfloat1622float2(bg[i]);
          acc = fmaf(fy.x, fg.x, acc);
          acc = fmaf(fy.y, fg.y, acc);
        }
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) dw[a] = acc;
  }
}

// Private copy of a receive buffer: rows that hold an assignment are copied, padding rows inside the used part become zero, rows at
// or beyond *used_end (unused capacity; nothing downstream reads them) are left alone.  One warp per row.
__global__ void __launch_bounds__(256) ep_take_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                                       const unsigned char* __restrict__ valid, const int* __restrict__ used_end, long long rows,
                                                       int d) {
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const long long limit = used_end != nullptr ? min(static_cast<long long>(*used_end), rows) : rows;
  for (long long r = warp; r < limit; r += nwarps) {
    const bool v = valid[r] != 0;
    for (int c = lane * 8; c < d; c += 256)
      *reinterpret_cast<uint4*>(dst + r * d + c) = v ? *reinterpret_cast<const uint4*>(src + r * d + c) : make_uint4(0u, 0u, 0u, 0u);
  }
}

static bool te_fill(TePeers& out, const long long* ptrs, int world) {
  if (world <= 0 || world > TE_MAX_RANKS) return false;
  for (int r = 0; r < TE_MAX_RANKS; ++r) out.p[r] = r < world ? reinterpret_cast<void*>(ptrs[r]) : nullptr;
  return true;
}
static unsigned te_grid(long long work_items, int per_block) {
  long long g = (work_items + per_block - 1) / per_block;
  if (g < 1) g = 1;
  if (g > 148 * 8) g = 148 * 8;
  return static_cast<unsigned>(g);
}

}  // namespace cmb

extern "C" int cmb_sum_slots(const void* slots, int nslots, long long n, const void* residual, void* out, void* stream) {
  if (n <= 0) return 0;
  if (n & 7) return 1;
  cmb::sum_slots_kernel<<<cmb::te_grid(n / 8, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(slots), nslots, n, static_cast<const __nv_bfloat16*>(residual), static_cast<__nv_bfloat16*>(out));
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

extern "C" int cmb_ep_dispatch(const void* x, const long long* tok, const int* dest_rank, const long long* dest_slot, const float* scale,
                               const long long* buf_ptrs, int world, long long assignments, int d, long long rows, int* status,
                               void* stream) {
  cmb::TePeers bufs;
  if (!cmb::te_fill(bufs, buf_ptrs, world) || (d & 7) || rows < 0) return 1;
  if (assignments <= 0) return 0;
  cmb::ep_dispatch_kernel<<<cmb::te_grid(assignments, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), tok, dest_rank, dest_slot, scale, bufs, assignments, d, rows, world, status);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

extern "C" int cmb_ep_combine(const long long* ybuf_ptrs, int world, const int* src_rank, const long long* src_slot, const float* w, void* out,
                              long long tokens, int k, int d, long long rows, int* status, void* stream) {
  cmb::TePeers bufs;
  if (!cmb::te_fill(bufs, ybuf_ptrs, world) || (d & 7) || rows < 0) return 1;
  if (tokens <= 0) return 0;
  cmb::ep_combine_kernel<<<cmb::te_grid(tokens, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      bufs, src_rank, src_slot, w, static_cast<__nv_bfloat16*>(out), tokens, k, d, rows, world, status, nullptr);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

extern "C" int cmb_ep_take(const void* src, void* dst, const void* valid, const int* used_end, long long rows, int d, void* stream) {
  if (rows <= 0) return 0;
  if (d & 7) return 1;
  cmb::ep_take_kernel<<<cmb::te_grid(rows, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(src), static_cast<__nv_bfloat16*>(dst), static_cast<const unsigned char*>(valid), used_end, rows, d);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// The weighted combine that also keeps the gathered rows (training forward).
extern "C" int cmb_ep_combine_rows(const long long* ybuf_ptrs, int world, const int* src_rank, const long long* src_slot, const float* w, void* out,
                                   void* rows_out, long long tokens, int k, int d, long long rows, int* status, void* stream) {
  cmb::TePeers bufs;
  if (!cmb::te_fill(bufs, ybuf_ptrs, world) || (d & 7) || rows < 0) return 1;
  if (tokens <= 0) return 0;
  cmb::ep_combine_kernel<<<cmb::te_grid(tokens, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      bufs, src_rank, src_slot, w, static_cast<__nv_bfloat16*>(out), tokens, k, d, rows, world, status, static_cast<__nv_bfloat16*>(rows_out));
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

extern "C" int cmb_ep_combine_bwd(const long long* ybuf_ptrs, int world, const int* src_rank, const long long* src_slot, const void* g, float* dw,
                                  long long assignments, int k, int d, long long rows, int* status, void* stream) {
  cmb::TePeers bufs;
  if (!cmb::te_fill(bufs, ybuf_ptrs, world) || (d & 7) || rows < 0) return 1;
  if (assignments <= 0) return 0;
  cmb::ep_combine_bwd_kernel<<<cmb::te_grid(assignments, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      bufs, src_rank, src_slot, static_cast<const __nv_bfloat16*>(g), dw, assignments, k, d, rows, world, status);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
