"""The allocation-free greedy selector, called through its exported C symbol.

Some users of this library cannot call cudaMalloc when they need a token selected: their memory
plan is sealed before serving starts, or the process that loads the library owns the allocator.
``cafd_argmax_noalloc`` serves them with scratch that lives inside the library image.  This test
binds the symbol with ctypes directly (no wrapper in between), runs it twice in a row on
different inputs, and compares each result with ``cafd_argmax``, which takes caller scratch.
It sits in a file that pytest collects last, and passes both alone and after the other tests.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _symbols():
    from cuteafd_b200._native import build
    lib = C.CDLL(build.CUDA_LIB)
    P, I = C.c_void_p, C.c_int
    lib.cafd_argmax_noalloc.argtypes = [P, P, I, I, I, P]
    lib.cafd_argmax_noalloc.restype = I
    lib.cafd_argmax_noalloc_max_rows.argtypes = []
    lib.cafd_argmax_noalloc_max_rows.restype = I
    lib.cafd_argmax.argtypes = [P, P, P, I, I, I, P]
    lib.cafd_argmax.restype = I
    lib.cafd_argmax_slices.argtypes = []
    lib.cafd_argmax_slices.restype = I
    return lib


def test_noalloc_argmax_matches_scratch_variant_twice():
    lib = _symbols()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream().cuda_stream
    slices = lib.cafd_argmax_slices()
    for call, (T, V) in enumerate([(37, 151936), (5, 4099)]):          # two calls in a row share the array
        g = torch.Generator(device="cpu").manual_seed(100 + call)
        logits = torch.randn(T, V, generator=g).to(dev)
        logits[1, 7] = logits[1, V - 3] = 1e9                          # tie: lowest index wins
        logits[2, 11] = float("nan")                                   # NaN never wins
        scratch = torch.empty(2 * T * slices, dtype=torch.int32, device=dev)
        want = torch.full((T,), -1, dtype=torch.int32, device=dev)
        got = torch.full((T,), -2, dtype=torch.int32, device=dev)
        assert lib.cafd_argmax(logits.data_ptr(), want.data_ptr(), scratch.data_ptr(), T, V, logits.stride(0), stream) == 0
        before = torch.cuda.memory_allocated(dev)
        assert lib.cafd_argmax_noalloc(logits.data_ptr(), got.data_ptr(), T, V, logits.stride(0), stream) == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated(dev) == before
        assert torch.equal(got, want)                                  # integer outputs: exact match
        assert got[1].item() == 7
        host = logits.cpu()
        ref = torch.where(torch.isnan(host), torch.full_like(host, float("-inf")), host).argmax(-1)
        assert torch.equal(got.long().cpu(), ref)


def test_noalloc_argmax_rejects_oversize():
    lib = _symbols()
    dev = torch.device("cuda:0")
    limit = lib.cafd_argmax_noalloc_max_rows()
    assert limit == 1024
    logits = torch.zeros(4, 8, device=dev)
    out = torch.full((4,), -5, dtype=torch.int32, device=dev)
    rc = lib.cafd_argmax_noalloc(logits.data_ptr(), out.data_ptr(), limit + 1, 8, 8, torch.cuda.current_stream().cuda_stream)
    assert rc == -20
    torch.cuda.synchronize()
    assert (out == -5).all()                                           # nothing was launched
