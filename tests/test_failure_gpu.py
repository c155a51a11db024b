"""Failure detection on the device without a fault: a bounded wait on a peer flag that nothing sets runs out,
the kernel returns, the host reads a status word and raises a typed error, and the context stays usable."""
import time
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_peer_flag_wait_runs_out_and_is_reported():
    from poot_b200.ops import cuda_ops as K
    from poot_b200.ops._lib import check
    _P = c_void_p
    K.register_signature("poot_tp_begin_step", [_P, _P, _P])
    K.register_signature("poot_tp_norm", [_P, _P, _P, _P, _P, c_int, c_int, c_float, c_int, c_int, c_int, c_int, c_int,
                                          c_int, c_int, _P, _P, _P, _P, _P, _P])
    dev = torch.device("cuda")
    world, H, rows = 2, 256, 1
    flags = [torch.zeros(256, dtype=torch.int32, device=dev) for _ in range(world)]       # nobody ever sets these
    inbox = torch.zeros(2 * world * 128 * H, dtype=torch.bfloat16, device=dev)
    epoch = torch.zeros(1, dtype=torch.int32, device=dev)
    ticket = torch.zeros(1, dtype=torch.int32, device=dev)
    h = torch.ones(rows, H, dtype=torch.bfloat16, device=dev)
    w = torch.ones(H, dtype=torch.bfloat16, device=dev)
    x = torch.zeros(rows, H, dtype=torch.bfloat16, device=dev)
    fp = (c_void_p * world)(*[f.data_ptr() for f in flags])
    st = K.status_word(dev)
    K.check_status()
    K.set_step_budget(0.5, dev)                      # the waits of this "step" share half a second
    check(K.fn("poot_tp_begin_step")(epoch.data_ptr(), st.data_ptr(), K._stream()), "begin")
    t0 = time.time()
    check(K.fn("poot_tp_norm")(h.data_ptr(), inbox.data_ptr(), w.data_ptr(), None, x.data_ptr(), rows, H, 1e-5, world, 0,
                               128, 0, 3, 0, 2, epoch.data_ptr(), flags[0].data_ptr(), fp, ticket.data_ptr(),
                               st.data_ptr(), K._stream()), "tp_norm")
    torch.cuda.synchronize()
    waited = time.time() - t0
    K.set_step_budget(K.DEFAULT_STEP_BUDGET_S, dev)
    assert 0.3 < waited < 5.0                        # the wait ended at the step deadline
    with pytest.raises(K.DeviceWaitTimeout, match="step deadline") as err:
        K.check_status()
    assert err.value.code == 7 and err.value.detail == 0      # site 0, rank 0's flag never came
    K.check_status()                                 # the word was cleared by the report
    assert float(torch.ones(8, device=dev).sum()) == 8.0        # the context is still usable
