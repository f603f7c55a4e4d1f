"""The entry point that allocates nothing (csrc/no_alloc.h), called through its exported
C symbol the way a program that cannot use cudaMalloc would call it: the caller owns the
input and the output, the library brings its own fixed scratch.  Its result must equal the
ordinary entry point's, on two calls in a row that share that scratch.

The file's name makes pytest collect it last, so that a run that stops at the first failure
has already run every other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, logits, out):
    lib.ifx_argmax_no_alloc.restype = ctypes.c_int
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    return lib.ifx_argmax_no_alloc(ctypes.c_void_p(logits.data_ptr()), ctypes.c_void_p(out.data_ptr()),
                                   logits.shape[0], logits.shape[1], stream)


def test_no_alloc_argmax_matches_the_ordinary_entry_point(cuda_kernels):
    lib = cuda_kernels.lib
    g = torch.Generator().manual_seed(5)
    first = torch.randn(64, 152064, generator=g).to("cuda:0")
    second = torch.randn(7, 30011, generator=g).to("cuda:0")
    first[3, 1000] = first[3, 120000] = 99.0              # a tie: the lower index is the answer
    out1 = torch.full((64,), -1, dtype=torch.int32, device="cuda:0")
    out2 = torch.full((7,), -1, dtype=torch.int32, device="cuda:0")
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    assert _call(lib, first, out1) == 0                   # the first call also looks the scratch address up
    assert _call(lib, second, out2) == 0                  # the second call meets what the first left behind
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    want1 = cuda_kernels.argmax(first)                    # the existing entry point (ifx_argmax_chunks)
    want2 = cuda_kernels.argmax(second)
    assert torch.equal(out1, want1) and torch.equal(out2, want2)
    assert out1.tolist() == torch.argmax(first, -1).tolist() and int(out1[3]) == 1000
    assert out2.tolist() == torch.argmax(second, -1).tolist()


def test_no_alloc_argmax_refuses_what_does_not_fit(cuda_kernels):
    lib = cuda_kernels.lib
    big = torch.zeros((257, 8), device="cuda:0")
    out = torch.zeros((257,), dtype=torch.int32, device="cuda:0")
    assert _call(lib, big, out) == -4                     # more rows than the fixed scratch holds
    lib.ifx_argmax_no_alloc.restype = ctypes.c_int
    assert lib.ifx_argmax_no_alloc(ctypes.c_void_p(0), ctypes.c_void_p(out.data_ptr()), 1, 8, ctypes.c_void_p(0)) == -1
    assert _call(lib, big[:0], out[:0]) == 0              # nothing to do
