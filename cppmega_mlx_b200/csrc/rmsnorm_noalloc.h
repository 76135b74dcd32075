// RMSNorm backward that allocates nothing. This entry point has no counterpart in the reference project.
//
// Who it is for: code that drives this library from a place where device memory cannot be requested —
// a plugin running inside another runtime's memory pool with no allocator handed to it, a real-time or
// safety-reviewed loop whose rules forbid cudaMalloc after start-up, a host that has already given all
// device memory away to a serving engine. Such callers own their input and output buffers and nothing
// else. The ordinary cmb_rmsnorm_bwd needs an extra caller-provided buffer for per-block partial sums of
// the weight gradient; this variant keeps those partials in a fixed array inside the library image.
//
//   int cmb_rmsnorm_bwd_noalloc(gy, x, w, rstd, gx, gw, rows, cols, stream)
//     gy, x  : bf16 [rows, cols]   upstream gradient and the forward input
//     w      : bf16 [cols]         norm weight
//     rstd   : fp32 [rows]         1/rms saved by the forward
//     gx     : bf16 [rows, cols]   out: gradient w.r.t. x
//     gw     : fp32 [cols]         out: gradient w.r.t. w (fully reduced)
//     returns 0, or  -1 null pointer · -2 bad shape (cols must be a positive multiple of 8, rows > 0)
//                    -3 cols above the limit · -4 no usable current device · -5 scratch lookup failed
//                    -6 launch failed
//
// Limit: cols <= 8192 (any number of rows). The scratch is 148 x 8192 floats (4.6 MiB) and is held on
// every GPU that loads the library, for the life of the process.
//
// Set-up: the first call on a given GPU looks up the scratch array's device address (one cheap runtime
// query, no allocation) and caches it. Make that first call with the GPU current and outside of any
// stream capture; later calls on that GPU do no set-up at all.
//
// Sharing: all calls on a GPU use the same scratch. Calls issued to one stream are ordered and safe.
// Two calls that can run at the same time on one GPU (different streams, different threads) would
// overwrite each other's partial sums — serialise them. The scratch keeps whatever the last call left
// there; each call overwrites every word it later reads, so stale contents are never observed.
//
// The function itself calls no cudaMalloc / cudaFree and no library routine that allocates.
#pragma once
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
int cmb_rmsnorm_bwd_noalloc(const void* gy, const void* x, const void* w, const void* rstd, void* gx, float* gw,
                            int64_t rows, int cols, void* stream);
#ifdef __cplusplus
}
#endif
