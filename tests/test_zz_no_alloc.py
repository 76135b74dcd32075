"""The allocation-free RMSNorm backward, called the way its intended users call it: straight through the
exported C symbol with raw pointers, no Python wrapper in between.

Those users are embedders that own their buffers but may not ask the driver for more (plugins inside a
foreign memory pool, loops that must not allocate after start-up), so the test hands the function nothing
but pre-made inputs and outputs and checks the result against the ordinary entry point, twice in a row —
the second call runs on scratch that still holds the first call's partial sums.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ordinary(lib, gy, x, w, rstd):
    rows, cols = x.shape
    gx = torch.empty_like(x)
    nblk = min(rows, 148)
    part = torch.empty(nblk, cols, dtype=torch.float32, device=x.device)
    rc = lib.cmb_rmsnorm_bwd(ctypes.c_void_p(gy.data_ptr()), ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()),
                             ctypes.c_void_p(rstd.data_ptr()), ctypes.c_void_p(gx.data_ptr()),
                             ctypes.c_void_p(part.data_ptr()), ctypes.c_int64(rows), ctypes.c_int(cols), ctypes.c_int(nblk),
                             ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    return gx, part.sum(0)


def test_noalloc_rmsnorm_bwd_matches_ordinary_entry_point_twice():
    from cppmega_mlx_b200.ops import _backend as B
    lib = B.load_library()
    fn = lib.cmb_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # Shapes cover both kernels the entry point can pick: one warp per row (cols <= 2048 with at least 4 rows) and one block
    # per row (wider rows, or fewer than 4 rows), the widest accepted row, and fewer rows than partial-sum slots.  Later shapes
    # are smaller than earlier ones, so stale partial sums of an earlier call are still in the scratch when they run.
    for rows, cols in [(1000, 2048), (300, 4096), (5, 8192), (77, 512), (3, 512), (2, 512)]:
        x = torch.randn(rows, cols, device=dev).bfloat16()
        gy = torch.randn(rows, cols, device=dev).bfloat16()
        w = (torch.rand(cols, device=dev) + 0.5).bfloat16()
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5)
        ref_gx, ref_gw = _ordinary(lib, gy, x, w, rstd)
        # fp32 PyTorch statement of the same backward (rstd given): the oracle that does not share a kernel with either entry point
        g32, x32, w32 = gy.float(), x.float(), w.float()
        dot = (g32 * w32 * x32).sum(-1, keepdim=True)
        o_gx = g32 * w32 * rstd[:, None] - x32 * dot * rstd[:, None] ** 3 / cols
        o_gw = (g32 * x32 * rstd[:, None]).sum(0)
        for _ in range(2):                                   # two calls in a row on the same scratch
            gx = torch.empty_like(x)
            gw = torch.empty(cols, dtype=torch.float32, device=dev)
            rc = fn(ctypes.c_void_p(gy.data_ptr()), ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()),
                    ctypes.c_void_p(rstd.data_ptr()), ctypes.c_void_p(gx.data_ptr()), ctypes.c_void_p(gw.data_ptr()),
                    ctypes.c_int64(rows), ctypes.c_int(cols), stream)
            assert rc == 0
            torch.cuda.synchronize()
            assert torch.equal(gx, ref_gx), (rows, cols)
            assert (gw - ref_gw).abs().max() <= 1e-3 * ref_gw.abs().max() + 1e-4, (rows, cols)
            assert (gx.float() - o_gx).abs().max() <= 2e-2 * o_gx.abs().max() + 1e-3, (rows, cols)
            assert (gw - o_gw).abs().max() <= 2e-3 * o_gw.abs().max() + 1e-3, (rows, cols)
    args = lambda r, c: (ctypes.c_void_p(gy.data_ptr()), ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()),
                         ctypes.c_void_p(rstd.data_ptr()), ctypes.c_void_p(gx.data_ptr()), ctypes.c_void_p(gw.data_ptr()),
                         ctypes.c_int64(r), ctypes.c_int(c), stream)
    # refusals, each without touching anything: width past the limit, a null pointer, a width that is not a multiple of 8, no rows
    assert fn(*args(4, 8192 + 8)) == -3
    assert fn(None, *args(4, 512)[1:]) == -1
    assert fn(*args(4, 510)) == -2
    assert fn(*args(0, 512)) == -2
