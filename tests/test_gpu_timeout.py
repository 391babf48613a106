"""GPU: a bounded device wait that runs out ends by itself and surfaces as WM_ERR_TIMEOUT.

The reference tests its transport deadline (ActivationTransportRunOptions.deadline_after ->
NotifyErrorCode::TransportTimeout, src/cuda/activation_transport/execution.cuh:1243-1250,
tests/run_control_protocol_regressions.py).  Here the failure is made on the HOST side only: the wait
kernel of the runtime is pointed at a flag word that nothing ever advances, with a budget of about a
millisecond.  The kernel gives up, records a status and returns normally; nothing faults, traps or keeps
spinning, and the runtime stays usable.
"""
import ctypes

import pytest
import torch

from oracle import moe_oracle as O
from weftmoe_b200 import SingleRankGroup, TensorRuntime, _lib

pytestmark = pytest.mark.gpu

SHORT_BUDGET_CYCLES = 2_000_000   # about 1 ms at 2 GHz


def bits(t):
    return t.contiguous().view(torch.int16)


def test_a_wait_that_runs_out_reports_timeout_and_leaves_the_runtime_usable():
    lib = _lib.load()
    cfg = dict(experts=8, top_k=2, hidden=512, intermediate=512, tokens=64)
    d = {k: v.cuda() for k, v in O.make_inputs(cfg, seed=5).items()}
    rt = TensorRuntime(group=SingleRankGroup(), experts=8, top_k=2, hidden=512, intermediate=512, max_tokens=64,
                       max_rows=128, training=False)
    args = (d["x"], d["routes"], d["gates"], d["w1"], d["w2"])
    before = rt.inference_eager(*args).clone()
    native = rt.native
    stream = native.stream.cuda_stream
    flag = torch.zeros(32, dtype=torch.int32, device="cuda")      # never advanced by anyone
    code = ctypes.c_int32(-1)
    try:
        assert lib.wm_debug_set_wait_budget(SHORT_BUDGET_CYCLES) == _lib.WM_OK
        # 1. a satisfied wait (target 0 <= flag) leaves the status clean
        _lib.check(lib.wm_debug_wait_flag(native.handle, _lib.ptr(flag), 0, stream))
        _lib.check(lib.wm_status_poll(native.handle, ctypes.byref(code), stream))
        assert code.value == _lib.WM_OK
        # 2. a wait for generation 1 on a word that stays 0 runs out after about a millisecond
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(native.stream):
            start.record()
            _lib.check(lib.wm_debug_wait_flag(native.handle, _lib.ptr(flag), 1, stream))
            stop.record()
        stop.synchronize()                                         # the kernel returned by itself
        assert 0.2 < start.elapsed_time(stop) < 200.0              # ms: the short budget, not the 2 s default
        _lib.check(lib.wm_status_poll(native.handle, ctypes.byref(code), stream))
        assert code.value == _lib.WM_ERR_TIMEOUT
        assert "wait" in _lib.last_error()
        # 3. the poll cleared the word: the next poll is clean
        _lib.check(lib.wm_status_poll(native.handle, ctypes.byref(code), stream))
        assert code.value == _lib.WM_OK
    finally:
        lib.wm_debug_set_wait_budget(0)
    # 4. the context and the runtime are intact: the same call gives the same bits as before
    after = rt.inference_eager(*args)
    assert torch.equal(bits(after), bits(before))
    rt.close()


def test_public_api_raises_runtime_error_on_a_timed_out_wait():
    """Through the Python boundary the same condition is a RuntimeError at the next synchronising call
    (the reference maps TransportTimeout to RuntimeError, weftmoe/runtime.py:186)."""
    lib = _lib.load()
    rt = TensorRuntime(group=SingleRankGroup(), experts=8, top_k=2, hidden=512, intermediate=512, max_tokens=8,
                       max_rows=16, training=False)
    flag = torch.zeros(32, dtype=torch.int32, device="cuda")
    try:
        lib.wm_debug_set_wait_budget(SHORT_BUDGET_CYCLES)
        _lib.check(lib.wm_debug_wait_flag(rt.native.handle, _lib.ptr(flag), 7, rt.native.stream.cuda_stream))
        with pytest.raises(RuntimeError):
            rt.native.drain_eager_inference()
    finally:
        lib.wm_debug_set_wait_budget(0)
    rt.native.drain_eager_inference()   # clean again
    rt.close()
