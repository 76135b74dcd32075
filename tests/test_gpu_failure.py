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


def test_ep_dispatch_skips_slots_outside_the_receive_buffer_and_reports_them():
    """Expert-parallel dispatch with a receive buffer of 4 rows and assignments whose slots are −1 (dropped by the plan), in
    range, and beyond the capacity: rows in range arrive, the −1 slot is skipped silently, the out-of-range slot is skipped and
    named in the status block, nothing past the 4 rows is touched, and the gather on the way back returns zeros for both."""
    from cppmega_mlx_b200.ops import _backend as B
    lib = B.load_library()
    dev = torch.device("cuda", 0)
    d, rows = 64, 4
    guard = torch.full(((rows + 8) * d,), 7.0, dtype=torch.bfloat16, device=dev)        # 4 real rows followed by a guard area
    ptrs = (ctypes.c_longlong * 1)(guard.data_ptr())
    x = torch.randn(5, d, device=dev).bfloat16()
    tok = torch.arange(5, device=dev, dtype=torch.int64)
    dest = torch.zeros(5, dtype=torch.int32, device=dev)
    slot = torch.tensor([2, -1, 0, 9, 3], dtype=torch.int64, device=dev)                  # 9 ≥ rows: must not be written
    status = torch.zeros(16, dtype=torch.int32, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = lib.cmb_ep_dispatch(vp(x), vp(tok), vp(dest), vp(slot), None, ptrs, 1, ctypes.c_longlong(5), d, ctypes.c_longlong(rows),
                             vp(status), stream)
    torch.cuda.synchronize()
    assert rc == 0
    buf = guard.view(rows + 8, d)
    assert torch.equal(buf[2], x[0]) and torch.equal(buf[0], x[2]) and torch.equal(buf[3], x[4])
    assert bool((buf[1] == 7).all()) and bool((buf[rows:] == 7).all())                  # untouched: no store left the buffer
    st = status.tolist()
    assert st[0] == 6 and st[1:4] == [3, 9, 0]                                           # ST_BAD_ARGUMENT: assignment 3, slot 9, rank 0
    status.zero_()
    out = torch.full((5, d), 3.0, dtype=torch.bfloat16, device=dev)
    rc = lib.cmb_ep_combine(ptrs, 1, vp(dest), vp(slot), None, vp(out), ctypes.c_longlong(5), 1, d, ctypes.c_longlong(rows), vp(status), stream)
    torch.cuda.synchronize()
    assert rc == 0
    assert torch.equal(out[0], x[0]) and torch.equal(out[2], x[2]) and torch.equal(out[4], x[4])
    assert bool((out[1] == 0).all()) and bool((out[3] == 0).all())
    assert status.tolist()[0] == 6 and status.tolist()[2] == 9
    assert float((torch.ones(4, device=dev) * 2).sum()) == 8.0                           # the context is alive


def test_cross_entropy_target_outside_the_vocabulary_is_skipped_and_reported():
    """A target id ≥ V (or negative) in a valid row: nothing is read at that index, the row contributes no loss and no gradient, and
    the status block names (code, row, target, V).  The other rows are unaffected."""
    from cppmega_mlx_b200 import ops
    from cppmega_mlx_b200.ops import _backend as B
    torch.manual_seed(0)
    V, D, rows = 512, 64, 40
    h = (torch.randn(rows, D, device="cuda") * 0.5).bfloat16().requires_grad_()
    w = (torch.randn(V, D, device="cuda") * 0.1).bfloat16().requires_grad_()
    t = torch.randint(0, V, (rows,), device="cuda")
    bad = t.clone()
    bad[7] = V + 123
    B.check_status()
    loss_bad = ops.linear_cross_entropy(h, w, bad)
    loss_bad.backward()
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="status words") as e:
        B.check_status()
    assert f"[6, 7, {V + 123}, {V}" in str(e.value)           # ST_BAD_ARGUMENT, row 7, the target, the vocabulary size
    assert bool(torch.isfinite(loss_bad)) and bool(torch.isfinite(h.grad).all())
    assert float(h.grad[7].abs().max()) == 0.0                 # the bad row has no gradient
    B.check_status()                                           # reading the status cleared it
    assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0
