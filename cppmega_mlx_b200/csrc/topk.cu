// Row-wise top-k index selection (the DSA selector): for each row, the column indices of the k largest
// scores inside [start, end), `-1` padded when fewer than k columns are valid; order unspecified.
//
// One CTA per row, exact radix select on order-preserving 32-bit keys: four 8-bit passes (MSB first) with a
// 256-bin shared-memory histogram narrow down the k-th largest key, a final pass emits every index whose key
// is above it plus as many ties as are still needed.  The row (≤ 32 KB for 8192 columns) stays in L2 between
// passes.  Oracle: ops.topk_select_reference (semantics of cppmega_mlx/nn/_tilelang/topk_selector.py:227-331;
// the two-stage 256-bin radix select the reference describes for CUDA: docs/tilelang_ports/topk_selector.md:33-45).
#include "sm100.cuh"

namespace cmb {

__device__ __forceinline__ unsigned order_key(float f) {
  const unsigned u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__global__ void __launch_bounds__(256) topk_select_kernel(const float* __restrict__ scores, const int* __restrict__ starts,
                                                          const int* __restrict__ ends, int* __restrict__ out, int n,
                                                          int k) {
  __shared__ int hist[256];
  __shared__ unsigned s_prefix;
  __shared__ int s_remaining, s_count, s_ties;
  const long long row = blockIdx.x;
  const float* sr = scores + row * n;
  int* orow = out + row * k;
  int lo = starts != nullptr ? starts[row] : 0;
  int hi = ends != nullptr ? ends[row] : n;
  lo = max(lo, 0);
  hi = min(hi, n);
  const int valid = max(hi - lo, 0);
  if (valid <= k) {
    for (int i = threadIdx.x; i < k; i += 256) orow[i] = i < valid ? lo + i : -1;
    return;
  }
  if (threadIdx.x == 0) {
    s_prefix = 0u;
    s_remaining = k;
    s_count = 0;
    s_ties = 0;
  }
  unsigned mask = 0u;
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    hist[threadIdx.x] = 0;
    __syncthreads();
    const unsigned prefix = s_prefix;
    for (int i = lo + threadIdx.x; i < hi; i += 256) {
      const unsigned key = order_key(sr[i]);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int cum = 0, rem = s_remaining, chosen = 0;
      for (int b = 255; b >= 0; --b) {
        const int h = hist[b];
        if (cum + h >= rem) {
          chosen = b;
          rem -= cum;
          break;
        }
        cum += h;
      }
      s_remaining = rem;
      s_prefix = prefix | (static_cast<unsigned>(chosen) << shift);
    }
    mask |= 255u << shift;
    __syncthreads();
  }
  const unsigned thr = s_prefix;
  const int ties_needed = s_remaining;
  for (int i = lo + threadIdx.x; i < hi; i += 256) {
    const unsigned key = order_key(sr[i]);
    if (key > thr) {
      orow[atomicAdd(&s_count, 1)] = i;
    } else if (key == thr) {
      if (atomicAdd(&s_ties, 1) < ties_needed) orow[atomicAdd(&s_count, 1)] = i;
    }
  }
}

}  // namespace cmb

extern "C" int cmb_topk_select(const float* scores, const int* starts, const int* ends, int* out, long long rows, int n,
                               int k, void* stream) {
  if (rows <= 0 || k <= 0) return 0;
  if (rows > 0x7fffffffLL) return 1;
  cmb::topk_select_kernel<<<static_cast<unsigned>(rows), 256, 0, static_cast<cudaStream_t>(stream)>>>(scores, starts, ends,
                                                                                                    out, n, k);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
