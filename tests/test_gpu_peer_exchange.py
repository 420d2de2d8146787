"""The peer-memory amax exchange on ONE GPU: a world of one rank exchanges with itself (its own state array is the only
peer), which exercises the slot / call-number logic -- both slot sets, many calls, a stale array -- and the argument
checks.  The two-rank form runs in tests/test_gpu_multi.py."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_single_rank_exchange_over_many_calls():
    from cublade_b200 import _native as Nat
    from cublade_b200.bindings.cuda.split_phase import amax_peer_exchange, peer_exchange_state_bytes

    state = torch.zeros(peer_exchange_state_bytes() // 8, dtype=torch.int64, device="cuda")
    for i, v in enumerate([0.0, 3.5, 1e-30, 6.5e4, 0.25, 448.0, 7.0]):
        a = torch.tensor([v], dtype=torch.float32, device="cuda")
        got = amax_peer_exchange(a, [state.data_ptr()], 0)
        assert got.item() == a.item(), f"call {i}"
    torch.cuda.synchronize()
    assert int(state[32].item()) == 7  # the rank's call counter
    assert Nat.device_error_state() == 0


def test_argument_checks():
    from cublade_b200 import _native as Nat

    L = Nat.lib()
    a = torch.zeros(1, dtype=torch.float32, device="cuda")
    out = torch.zeros(1, dtype=torch.float32, device="cuda")
    state = torch.zeros(64, dtype=torch.int64, device="cuda")
    ptrs = (ctypes.c_void_p * 17)(*([state.data_ptr()] * 17))
    assert L.cb_amax_peer_exchange(a.data_ptr(), ptrs, 0, 17, out.data_ptr(), None) == 4   # CB_ERR_RANGE: more than 16 ranks
    assert L.cb_amax_peer_exchange(a.data_ptr(), ptrs, 2, 2, out.data_ptr(), None) == 4    # rank outside the world
    assert L.cb_amax_peer_exchange(None, ptrs, 0, 1, out.data_ptr(), None) == 1            # CB_ERR_ARGUMENT
    assert L.cb_peer_exchange_max_ranks() == 16 and L.cb_peer_exchange_state_bytes() == 33 * 8
