"""The argmax entry point for callers that cannot allocate device memory (csrc/sampling_noalloc.h),
called through its exported C symbol and compared with the ordinary entry point, which takes its
scratch from the caller.  Two calls in a row share the library's built-in scratch array: the second
must not be disturbed by what the first left there.

The file sorts last on purpose, so that a run that stops at the first failure has run every other test."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _library():
    from jax_llm_examples_b200.kernels import api

    lib = api.library("sampling")
    fn = lib.jlx_argmax_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p]
    return api, lib, fn


def test_no_alloc_argmax_matches_the_ordinary_one_twice_in_a_row():
    api, lib, fn = _library()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    gen = torch.Generator(device="cuda").manual_seed(11)
    # The first call on a device looks up the built-in array's address, which may make the driver load the
    # library's device code: let that happen before free memory is measured.
    warm = torch.zeros(1, 8, device="cuda")
    assert fn(warm.data_ptr(), 1, 8, 8, torch.empty(1, device="cuda", dtype=torch.int32).data_ptr(), stream) == 0
    torch.cuda.synchronize()
    for M, V in ((5, 1003), (64, 202048)):  # the second call reuses (and overwrites) what the first left
        logits = torch.randn(M, V, device="cuda", generator=gen)
        logits[0, 7] = logits[0, V - 2] = 50.0  # a tie: the lower index must win in both
        logits[M - 1, V - 1] = 60.0
        want = torch.empty(M, device="cuda", dtype=torch.int32)
        api.argmax(logits, want, torch.empty(32 * M, device="cuda"), torch.empty(32 * M, device="cuda", dtype=torch.int32))
        got = torch.full((M,), -1, device="cuda", dtype=torch.int32)
        torch.cuda.synchronize()
        # Free memory as the driver counts it (cudaMemGetInfo): a cudaMalloc inside the library would show here,
        # while torch's own counters only see torch's allocator.
        free_before, torch_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
        rc = fn(logits.data_ptr(), M, V, V, got.data_ptr(), stream)
        assert rc == 0, lib.jlx_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before and torch.cuda.memory_allocated() == torch_before
        assert got.tolist() == want.tolist()  # token ids: equal, not merely close
        assert got[0].item() == 7 and got[M - 1].item() == V - 1


def test_no_alloc_argmax_refuses_more_rows_than_its_scratch_holds():
    api, lib, fn = _library()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    logits = torch.zeros(257, 16, device="cuda")
    out = torch.full((257,), -1, device="cuda", dtype=torch.int32)
    rc = fn(logits.data_ptr(), 257, 16, 16, out.data_ptr(), stream)
    assert rc != 0 and "256" in lib.jlx_last_error().decode()
    torch.cuda.synchronize()
    assert (out == -1).all()  # nothing ran
