"""Bounded waits: a flag that nobody sets makes the wait give up with a status code; nothing traps or hangs."""

import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_peer_flag_wait_runs_out_and_reports():
    from nki_library_b200 import _lib
    flags = torch.zeros(4 * 8, dtype=torch.int32, device="cuda")
    epoch = torch.ones(1, dtype=torch.int32, device="cuda")   # waiting for step 1
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    # two "ranks" that both live in this buffer; this process only plays rank 0, so word [slot][1] is never posted
    table = (ctypes.c_void_p * 8)()
    table[0] = flags.data_ptr()
    table[1] = flags.data_ptr()
    t0 = time.time()
    _lib.call("b200moe_ep_signal_wait", table, 0, 2, 1, _lib.ptr(epoch), _lib.ptr(status), _lib.stream_ptr())
    torch.cuda.synchronize()
    waited = time.time() - t0
    assert int(status.item()) == 13            # 12 + slot
    assert 0.5 < waited < 15.0
    assert int(flags.view(4, 8)[1, 0].item()) == 1   # our own post went out
    # the context is still usable and a complete barrier passes at once
    flags.view(4, 8)[1, 1] = 1
    status.zero_()
    _lib.call("b200moe_ep_signal_wait", table, 0, 2, 1, _lib.ptr(epoch), _lib.ptr(status), _lib.stream_ptr())
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.ones(4, device="cuda").sum().item() == 4.0


def test_receive_buffer_overflow_is_reported():
    """More rows routed to a rank than its receive buffer holds -> status 21, no out-of-bounds store."""
    from nki_library_b200 import _lib
    world, E, B = 1, 4, 128
    counts_all = torch.tensor([300, 10, 0, 5], dtype=torch.int32, device="cuda")  # needs 3 + 1 + 0 + 1 = 5 blocks
    cap = 3
    b2e = torch.zeros(cap, dtype=torch.int32, device="cuda")
    cond = torch.zeros(cap + 2, dtype=torch.int32, device="cuda")
    valid = torch.zeros(cap * B, dtype=torch.int32, device="cuda")
    flags = torch.zeros(cap * B // 128, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    _lib.call("b200moe_ep_plan", _lib.ptr(counts_all), 0, world, E, B, cap, _lib.ptr(b2e), _lib.ptr(cond),
              _lib.ptr(valid), _lib.ptr(flags), _lib.ptr(status), _lib.stream_ptr())
    torch.cuda.synchronize()
    assert int(status.item()) == 21
    assert cond.tolist() == [1, 1, 1, 0, 0] and b2e.tolist() == [0, 0, 0]
    assert int((valid >= 0).sum().item()) == 300
