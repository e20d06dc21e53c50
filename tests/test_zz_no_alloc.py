"""Allocation-free lm-head log-prob entry point, called through its exported C symbol.

Some users of the library cannot allocate device memory when they need log-probs (no allocator of their
own, or a phase in which cudaMalloc is off limits), so ``apb_lmhead_logprob_fwd_noalloc`` keeps its
reduction scratch in a fixed array inside the library.  The test checks it against the ordinary entry
point (which takes the scratch from the caller) on two consecutive calls with different inputs -- the
second call sees the first call's leftovers in the shared scratch -- and checks that a problem larger than
the fixed array is refused.  This file sorts last so that a failure here cannot hide other tests.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _symbols():
    from arctic_platform_b200.ops import _lib
    lib = _lib.cuda_lib()
    c = ctypes
    noalloc = lib.apb_lmhead_logprob_fwd_noalloc
    noalloc.restype = c.c_int
    noalloc.argtypes = [c.c_void_p] * 7 + [c.c_int] * 3 + [c.c_longlong] * 2 + [c.c_float, c.c_void_p]
    plain = lib.apb_lmhead_logprob_fwd
    plain.restype = c.c_int
    plain.argtypes = [c.c_void_p] * 8 + [c.c_int] * 3 + [c.c_longlong] * 2 + [c.c_float, c.c_void_p]
    return _lib, noalloc, plain


def test_noalloc_matches_regular_entry_point_twice_and_rejects_oversize():
    _lib, noalloc, plain = _symbols()
    dev = torch.device("cuda", torch.cuda.current_device())
    stream = _lib.stream_ptr()          # also binds the library's runtime to this device
    for call, (M, H, V, scale) in enumerate([(200, 256, 32000, 1.0), (333, 512, 50304, 0.7)]):
        g = torch.Generator(device="cuda").manual_seed(100 + call)
        hidden = torch.randn(M, H, device=dev, generator=g).bfloat16()
        weight = (torch.randn(V, H, device=dev, generator=g) * 0.05).bfloat16()
        labels = torch.randint(0, V, (M,), device=dev, generator=g, dtype=torch.int32)
        out_a = [torch.empty(M, device=dev, dtype=torch.float32) for _ in range(3)]
        out_b = [torch.empty(M, device=dev, dtype=torch.float32) for _ in range(3)]
        scratch = torch.empty((M, (V + 127) // 128, 4), device=dev, dtype=torch.float32)
        rc = plain(hidden.data_ptr(), weight.data_ptr(), labels.data_ptr(), None, scratch.data_ptr(),
                   out_a[0].data_ptr(), out_a[1].data_ptr(), out_a[2].data_ptr(), M, V, H, hidden.stride(0),
                   weight.stride(0), scale, stream)
        assert rc == 0
        rc = noalloc(hidden.data_ptr(), weight.data_ptr(), labels.data_ptr(), None, out_b[0].data_ptr(),
                     out_b[1].data_ptr(), out_b[2].data_ptr(), M, V, H, hidden.stride(0), weight.stride(0), scale,
                     stream)
        assert rc == 0
        torch.cuda.synchronize()
        for a, b, name in zip(out_a, out_b, ("logprob", "entropy", "lse")):
            assert torch.allclose(a, b, atol=3e-2, rtol=1e-2), f"call {call}: {name} differs by {(a - b).abs().max()}"
        ref = torch.log_softmax(hidden.float() @ weight.float().t() * scale, -1).gather(1, labels.long()[:, None])[:, 0]
        assert torch.allclose(out_b[0], ref, atol=3e-2, rtol=1e-2)
    _lib.check_status("noalloc")
    # beyond the fixed scratch: refused with the documented code, nothing launched
    too_many_rows = 1310720 // ((32000 + 127) // 128) + 1
    rc = noalloc(hidden.data_ptr(), weight.data_ptr(), labels.data_ptr(), None, out_b[0].data_ptr(),
                 out_b[1].data_ptr(), out_b[2].data_ptr(), too_many_rows, 32000, 256, 256, 256, 1.0, stream)
    assert rc == 301
