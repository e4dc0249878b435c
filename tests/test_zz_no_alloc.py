"""The argmax entry point that allocates nothing (dispec_b200/csrc/no_alloc.h).

Some programs that call the kernels through the C ABI may not allocate device memory at all:
they gave the device to an arena of their own, or sit in a loop where an allocation's
synchronisation is not acceptable, or have no tensor library at hand.  For them the library
carries its scratch memory inside its own image.  This test calls that entry point through
its exported C symbol, twice in a row on different inputs (the scratch keeps the first
call's contents), and compares with the ordinary entry point; it also checks that a batch
beyond the built-in scratch is refused with a message.  The file name makes pytest collect
it after every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def call_static(lib, logits):
    out = torch.full((logits.shape[0],), -7, dtype=torch.int32, device=logits.device)
    rc = lib.dsp_argmax_static(ctypes.c_void_p(logits.data_ptr()), ctypes.c_long(logits.stride(0)),
                               logits.shape[0], logits.shape[1], ctypes.c_void_p(out.data_ptr()),
                               ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, out


def test_argmax_without_allocation_matches_the_ordinary_entry_point():
    from dispec_b200 import ops
    from dispec_b200.ops import library
    lib = library.core()
    lib.dsp_argmax_static_max_rows.restype = ctypes.c_int
    max_rows = lib.dsp_argmax_static_max_rows()
    assert max_rows == 1024
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(77)
    first = torch.randn(37, 151937, generator=g).to(dev)       # many chunks, a ragged last one
    second = torch.randn(5, 3001, generator=g).to(dev)         # a single chunk, fewer rows
    second[2, 17] = second[2, 2900] = 50.0                     # a tie: the lowest index wins
    torch.cuda.synchronize()
    for logits in (first, second):
        rc, got = call_static(lib, logits)
        assert rc == 0, lib.dsp_last_error()
        want = ops.argmax(logits)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        assert torch.equal(got.cpu().long(), logits.cpu().argmax(-1))
    assert int(call_static(lib, second)[1][2]) == 17
    # more rows than the built-in scratch holds: refused, nothing launched
    big = torch.zeros((max_rows + 1, 8), device=dev)
    rc, out = call_static(lib, big)
    assert rc != 0 and b"at most 1024" in lib.dsp_last_error()
    torch.cuda.synchronize()
    assert int(out[0]) == -7
