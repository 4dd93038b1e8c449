"""The library's allocation-free entry point, called the way a C program would: through its
exported symbol ``fwb_argmax_no_alloc``, with raw device pointers.

Callers that cannot allocate (inside a stream capture, under a fixed memory budget, in a
latency-critical loop) get greedy sampling from it without any scratch buffer of their own.
The test checks it against a host computation of its own (the first place at which a row
reaches its maximum) and against the library's ordinary argmax, on two calls in a row -- the second
smaller than the first, so stale contents of the shared scratch array would show -- and that a
problem beyond the stated maximum is refused with a readable reason.  It is collected last
(``zz``) so that a run which stops at the first failure has already run everything else.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def entry_point():
    from flyweight_b200.kernels import lib
    library = lib.library()
    fn = library.fwb_argmax_no_alloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    library.fwb_no_alloc_last_error.restype = ctypes.c_char_p
    return fn, library.fwb_no_alloc_last_error


def call(fn, logits, out):
    stream = torch.cuda.current_stream().cuda_stream
    return fn(logits.data_ptr(), logits.shape[0], logits.shape[1], out.data_ptr(), stream)


def test_two_calls_in_a_row_match_the_ordinary_argmax():
    from flyweight_b200.sampling import sampler
    fn, _ = entry_point()
    generator = torch.Generator().manual_seed(5)
    for rows, vocab in ((64, 65536), (3, 50001)):          # the second call is the smaller one
        logits = torch.randn(rows, vocab, generator=generator).to("cuda:0")
        logits[0, [11, vocab - 1]] = 40.0                   # equal maxima: the lower id wins
        logits[rows - 1, :] = 0.0                           # a constant row: id 0
        logits[1] = -logits[1].abs() - 1.0                  # all negative but two zeros of either
        logits[1, 5], logits[1, 9] = -0.0, 0.0              # sign: equal values, the lower id wins
        out = torch.full((rows,), -7, dtype=torch.int32, device="cuda:0")
        assert call(fn, logits, out) == 0
        torch.cuda.synchronize()
        # independent of the library: the first place at which a row reaches its maximum
        host = logits.cpu().numpy()
        first_maximum = [int(np.flatnonzero(row == row.max())[0]) for row in host]
        assert out.tolist() == first_maximum
        assert torch.equal(out, sampler.argmax(logits))     # and the library's ordinary argmax agrees
        assert out[0].item() == 11 and out[rows - 1].item() == 0 and out[1].item() == 5


def test_sizes_beyond_the_maximum_are_refused_with_a_reason():
    fn, last_error = entry_point()
    logits = torch.zeros(4, 128, device="cuda:0")
    out = torch.zeros(4, dtype=torch.int32, device="cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    assert fn(logits.data_ptr(), 257, 128, out.data_ptr(), stream) == -3
    assert b"at most 256 rows" in last_error()
    assert fn(None, 4, 128, out.data_ptr(), stream) == -1
    assert call(fn, logits, out) == 0                       # and it still works afterwards
    torch.cuda.synchronize()
    assert out.tolist() == [0, 0, 0, 0]
