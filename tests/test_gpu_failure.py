"""Failure detection on the device without a fault: a bounded wait that runs out reports through the status word."""
import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_peer_flag_wait_runs_out_and_reports_status():
    """A barrier over two flag blocks where nothing ever writes the second rank's flag: the waiting thread gives up after its
    spin limit (≈ a millisecond here), records (code, rank, peer, epoch) and the kernel returns normally; the context stays
    usable."""
    from cppmega_mlx_b200.ops import _backend as B
    lib = B.load_library()
    dev = torch.device("cuda", 0)
    pads = [torch.zeros(64, dtype=torch.int32, device=dev) for _ in range(2)]      # both "ranks'" flag blocks live here
    ptrs = (ctypes.c_longlong * 2)(pads[0].data_ptr(), pads[1].data_ptr())
    status = torch.zeros(16, dtype=torch.int32, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    t0 = time.perf_counter()
    rc = lib.cmb_comm_barrier(ptrs, 0, 2, 7, ctypes.c_longlong(10_000), ctypes.c_void_p(status.data_ptr()), stream)
    torch.cuda.synchronize()
    assert rc == 0 and time.perf_counter() - t0 < 5.0
    st = status.tolist()
    assert st[0] == 5 and st[1:4] == [0, 1, 7]            # ST_TIMEOUT_PEER_FLAG, waiting rank 0, silent peer 1, epoch 7
    assert int(pads[0][0]) == 7 and int(pads[1][0]) == 7   # rank 0 did publish its own arrival to both blocks
    # once the peer's flag is there the same barrier passes and leaves the status word alone
    pads[0][1] = 7
    status.zero_()
    rc = lib.cmb_comm_barrier(ptrs, 0, 2, 7, ctypes.c_longlong(10_000), ctypes.c_void_p(status.data_ptr()), stream)
    torch.cuda.synchronize()
    assert rc == 0 and status.tolist()[0] == 0
    assert float((torch.ones(4, device=dev) * 2).sum()) == 8.0   # the context is alive
