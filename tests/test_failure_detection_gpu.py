"""What happens when a kernel gives up a wait: every wait on a barrier inside the kernels is bounded; a kernel
whose wait runs out raises a bit in the engine's status word and returns, and the host turns that bit into an
error after the step.  The wait is made to run out the harmless way: a kernel of this test's own
(tests/csrc/wait_timeout_probe.cu) waits, with the package's own wait function and a limit of a few thousand
polls, on a barrier that nothing arrives at.  Nothing faults, traps or hangs."""

import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_becomes_an_engine_error(model_dirs):
    import jax_llm_examples_b200 as J
    from jax_llm_examples_b200.kernels import api, build

    lib = ctypes.CDLL(str(build.build_source(os.path.join(os.path.dirname(__file__), "csrc", "wait_timeout_probe.cu"))))
    lib.jlx_last_error.restype = ctypes.c_char_p
    model = J.load_model(model_dirs["tiny_a"], "bfloat16", "cuda")
    eng = J.Engine(model, max_tokens=64, page_size=16, max_slots=2)
    slot = eng.new_request()
    eng.step([J.StepEntry(slot, [1, 2, 3], [2])])
    eng.check_status()  # a healthy step raises nothing

    gave_up = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.jlx_test_wait_that_runs_out(ctypes.c_void_p(eng.status.data_ptr()), ctypes.c_uint(3000),
                                         ctypes.c_void_p(gave_up.data_ptr()), stream)
    assert rc == 0, lib.jlx_last_error().decode()
    torch.cuda.synchronize()
    assert int(gave_up) == 1
    with pytest.raises(J.EngineError, match="bounded wait"):
        eng.check_status()
    eng.check_status()  # the word was cleared: the engine goes on
    logits = eng.step([J.StepEntry(slot, [4], [0])])
    eng.check_status()
    assert torch.isfinite(logits).all()
    # the limit itself is refused when it is not small
    assert lib.jlx_test_wait_that_runs_out(ctypes.c_void_p(eng.status.data_ptr()), ctypes.c_uint(10 ** 7),
                                           ctypes.c_void_p(gave_up.data_ptr()), stream) != 0
    assert api.STATUS_BITS[8].startswith("a bounded wait")
