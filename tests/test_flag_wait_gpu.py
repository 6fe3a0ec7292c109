"""Failure detection on the device without a fault: the flag barrier of the peer-memory expert-parallel step gives up
after the context's wait limit when a rank never arrives, records the timeout in the status word and returns; the host
reads CTB_TIMEOUT and the context keeps working.  One GPU: both ranks' flag arrays live in this device's memory and
rank 1 simply never runs, so the wait runs out by itself (nothing traps, nothing spins for ever)."""
import ctypes as C
import time

import numpy as np
import pytest

from oracle import inputs, ref

pytestmark = pytest.mark.gpu


def test_barrier_wait_runs_out_and_the_context_stays_usable(cuda):
    import torch
    lib = cuda._lib
    ctx = lib.context(0)
    dummy = torch.zeros(64, device="cuda", dtype=torch.float16)       # stands in for the row buffers (not touched)
    flags = [torch.zeros(2, device="cuda", dtype=torch.int32) for _ in range(2)]
    epoch = torch.zeros(1, device="cuda", dtype=torch.int32)
    tab = lib.EpBuffers()
    tab.world, tab.rank = 2, 0
    for q in range(2):
        tab.recv_rows[q] = tab.recv_ids[q] = tab.recv_gates[q] = tab.slot_out[q] = dummy.data_ptr()
        tab.flags[q] = flags[q].data_ptr()
    tab.epoch = epoch.data_ptr()
    assert lib.lib.ctb_set_flag_wait_limit(ctx, 0) == lib.BAD_ARG                      # below one microsecond
    lib.check(lib.lib.ctb_set_flag_wait_limit(ctx, 50_000_000))                        # 50 ms
    try:
        t0 = time.perf_counter()
        lib.check(lib.lib.ctb_moe_ep_barrier(ctx, None, C.byref(tab)))                 # rank 1 never arrives
        st = lib.lib.ctb_check_device_status(ctx, None)
        waited = time.perf_counter() - t0
        assert st == lib.TIMEOUT and "bounded wait" in lib.last_error()
        assert 0.04 <= waited < 1.5                                                    # the limit, not the 2 s default
        assert flags[1][0].item() == 1 and flags[0][0].item() == 1                     # rank 0 did announce itself
        assert lib.lib.ctb_check_device_status(ctx, None) == lib.OK                    # the word was cleared
        # rank 1 arrives late: the next barrier (epoch 2) passes
        flags[0][1] = 2
        lib.check(lib.lib.ctb_moe_ep_barrier(ctx, None, C.byref(tab)))
        assert lib.lib.ctb_check_device_status(ctx, None) == lib.OK
    finally:
        lib.check(lib.lib.ctb_set_flag_wait_limit(ctx, 2_000_000_000))
    # the context still computes
    x = inputs.softmax(M=32, N=512)["input"]
    xd = torch.from_numpy(x).cuda()
    out = torch.empty_like(xd)
    cuda.softmax.softmax_tma_kernel(out, xd, 512)
    assert ref.max_abs_over_max(out.cpu().numpy(), ref.softmax(x)) <= 1e-5
