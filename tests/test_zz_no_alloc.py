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
    for rows, cols in [(1000, 2048), (77, 512)]:  # second shape is smaller: stale partials of the first stay in scratch
        x = torch.randn(rows, cols, device=dev).bfloat16()
        gy = torch.randn(rows, cols, device=dev).bfloat16()
        w = (torch.rand(cols, device=dev) + 0.5).bfloat16()
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5)
        gx = torch.empty_like(x)
        gw = torch.empty(cols, dtype=torch.float32, device=dev)
        rc = fn(ctypes.c_void_p(gy.data_ptr()), ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()),
                ctypes.c_void_p(rstd.data_ptr()), ctypes.c_void_p(gx.data_ptr()), ctypes.c_void_p(gw.data_ptr()),
                ctypes.c_int64(rows), ctypes.c_int(cols), stream)
        assert rc == 0
        ref_gx, ref_gw = _ordinary(lib, gy, x, w, rstd)
        torch.cuda.synchronize()
        assert torch.equal(gx, ref_gx)
        assert (gw - ref_gw).abs().max() <= 1e-3 * ref_gw.abs().max() + 1e-4
    # sizes past the limit are refused without touching anything
    assert fn(ctypes.c_void_p(gy.data_ptr()), ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()),
              ctypes.c_void_p(rstd.data_ptr()), ctypes.c_void_p(gx.data_ptr()), ctypes.c_void_p(gw.data_ptr()),
              ctypes.c_int64(4), ctypes.c_int(8192 + 8), stream) == -3
