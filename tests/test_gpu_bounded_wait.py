"""A device-side wait that can never be satisfied runs into its time limit, the kernel records the reason in the
library's status word and returns; the host turns that into an exception and the CUDA context stays usable.  This is
how a peer that never shows up is detected on the device (host-side detection: heartbeats and process-group timeouts)."""
import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_flag_wait_times_out_with_status_and_context_survives():
    from arctic_platform_b200.ops import _lib
    dev = torch.device("cuda")
    flags = torch.zeros(64, device=dev, dtype=torch.int32)
    wait = _lib.declare("apb_epoch_wait", [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p])
    # a "group" of two ranks whose flag arrays are both this buffer: slot 1 belongs to a rank that does not exist,
    # so nothing ever announces epoch 5 there
    table = (ctypes.c_void_p * 2)(flags.data_ptr(), flags.data_ptr())
    _lib.status_clear()
    t0 = time.perf_counter()
    _lib.check(wait(table, 0, 2, 5, _lib.stream_ptr()), "apb_epoch_wait")
    with pytest.raises(_lib.CollectiveTimeout, match="105") as err:
        _lib.check_status("waiting for a rank that never arrives")
    # the record names the missing peer and the epochs: slot 1 still holds 0, epoch 5 was expected
    assert (err.value.code, err.value.peer, err.value.expected_epoch, err.value.seen_epoch) == (105, 1, 5, 0)
    assert isinstance(err.value, _lib.KernelError)
    elapsed = time.perf_counter() - t0
    assert 0.5 < elapsed < 10.0                      # the limit is one second, not forever
    assert int(flags[0]) == 5 and int(flags[1]) == 0
    # the context is intact: the status word is clear again and kernels of the library still run
    assert _lib.status_read() == 0
    from arctic_platform_b200.ops import gemm
    a = torch.randn(128, 64, device=dev).bfloat16()
    b = torch.randn(64, 64, device=dev).bfloat16()
    out = gemm.matmul_nt(a, b)
    _lib.check_status("after the timeout")
    assert (out.float() - a.float() @ b.float().t()).abs().max() < 0.5
    # a wait that IS satisfied returns at once and leaves the status clear
    flags[1] = 6
    t0 = time.perf_counter()
    _lib.check(wait(table, 0, 2, 6, _lib.stream_ptr()), "apb_epoch_wait")
    _lib.check_status("satisfied wait")
    assert time.perf_counter() - t0 < 0.5
