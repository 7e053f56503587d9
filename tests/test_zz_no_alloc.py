"""The allocation-free LSTM entry point (souffle_lstm_forward_static) against the plan-based one.

It exists for hosts that cannot call cudaMalloc while running (their own pool owns the GPU's memory, or
an allocation's implicit device synchronisation is not acceptable), so its scratch is a fixed array in the
library.  Collected last on purpose: a failure here must not hide any other test's result.  Runs the
call twice in a row because every call re-uses the same scratch array and must clear what it needs clean.
"""
import ctypes as C

import pytest
import torch

from oracle import souffle_oracle as so

pytestmark = pytest.mark.gpu


def _static_forward(lib, desc, w_in, w_st, x):
    from souffle_models_b200 import _lib
    y = torch.full_like(x, float("nan"))
    status = torch.full((4,), -1, dtype=torch.int32, device="cuda")
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check(lib.souffle_lstm_forward_static(C.byref(desc), w_in.data_ptr(), w_st.data_ptr(), None, x.data_ptr(),
                                               y.data_ptr(), status.data_ptr(), st))
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    return y


@pytest.mark.parametrize("layers,hidden,steps", [(10, 256, 100), (3, 64, 8)])
def test_static_entry_matches_plan_entry_twice(layers, hidden, steps):
    from souffle_models_b200 import _lib, lstm
    lib = _lib.load()
    x, w_in, w_st = so.make_lstm_params(layers, hidden, steps, seed=4321)
    w_in, w_st, xd = w_in.cuda(), w_st.cuda(), x.float().cuda().reshape(steps, hidden)
    plan = lstm.LstmStack(w_in, w_st, steps)
    want = plan.forward(xd.reshape(1, steps, hidden)).reshape(steps, hidden)
    plan.status()
    desc = _lib.LstmDesc(layers=layers, hidden=hidden, steps=steps)
    for _ in range(2):                                   # second call re-uses the scratch of the first
        got = _static_forward(lib, desc, w_in, w_st, xd)
        assert torch.isfinite(got).all()
        assert (got - want).abs().max().item() <= 1e-6   # same kernel, same arithmetic order
    assert (want.cpu() - so.lstm_forward(x, w_in.cpu(), w_st.cpu())[0]).abs().max() < 5e-3


def test_static_entry_rejects_shapes_beyond_its_scratch():
    from souffle_models_b200 import _lib
    lib = _lib.load()
    desc = _lib.LstmDesc(layers=16, hidden=256, steps=100)      # 409,600 values > 393,216
    dummy = torch.zeros(64, dtype=torch.float32, device="cuda")
    rc = lib.souffle_lstm_forward_static(C.byref(desc), dummy.data_ptr(), dummy.data_ptr(), None, dummy.data_ptr(),
                                         dummy.data_ptr(), None, None)
    assert rc == 1 and b"exceeds the built-in scratch" in lib.souffle_last_error()
