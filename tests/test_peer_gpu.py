"""The peer-memory all-reduce kernel on ONE GPU, through the C ABI: a two-rank group inside this process whose second rank
never arrives (its flag lives in the GPU's own memory and nobody sets it). The kernel's bounded wait must run out, the
failure must be reported at the next synchronisation, and the library must stay usable; when the missing rank's
payload and flag are then posted from the host, the next call must return the sum. Nothing here faults, traps or
hangs the device: the wait returns by itself after its cycle budget."""
import ctypes

import numpy as np
import pytest

from cgt_b200 import runtime
from tests.gpu_util import Dev, code, longs

pytestmark = pytest.mark.gpu


def _allreduce(L, ins, outs):
    n = len(ins)
    pin = (ctypes.c_void_p * n)(*[d.ptr for d in ins])
    pout = (ctypes.c_void_p * n)(*[d.ptr for d in outs])
    return L.cgtb_peer_allreduce_sum(n, pin, pout, longs([int(np.prod(d.shape)) for d in ins]))


def test_missing_rank_times_out_and_the_library_stays_usable(rt):
    L = runtime.lib()
    assert L.cgtb_peer_world() == 1
    runtime.check(L.cgtb_peer_selftest_open(1 << 16), "selftest open")
    try:
        assert L.cgtb_peer_world() == 2 and L.cgtb_peer_slot_bytes() == 1 << 16
        runtime.check(L.cgtb_peer_set_wait_cycles(2_000_000), "wait budget")   # about a millisecond
        rs = np.random.RandomState(3)
        a, b = rs.randn(1001).astype("f4"), rs.randn(7, 11).astype("f4")
        da, db = Dev(a), Dev(b)
        oa, ob = Dev(np.full(a.shape, 5.0, "f4")), Dev(np.full(b.shape, 5.0, "f4"))
        # 1. the other rank never arrives: the call returns, the failure surfaces at the synchronisation
        runtime.check(_allreduce(L, [da, db], [oa, ob]), "peer allreduce (launch)")
        rc = L.cgtb_synchronize()
        assert rc != 0 and "did not arrive" in runtime.last_error()
        assert np.array_equal(oa.get(), np.full(a.shape, 5.0, "f4"))   # the sum was skipped, nothing half-written
        # 2. the library is healthy: an unrelated kernel runs and synchronises cleanly
        sq = Dev(shape=a.shape, dtype="f4")
        runtime.check(L.cgtb_unary(10, code("f4"), code("f4"), a.size, da.ptr, sq.ptr), "unary")
        runtime.synchronize()
        assert np.array_equal(sq.get(), a * a)
        # 3. the missing rank's payload and flag are posted for the next call: it completes with the sum, twice in a row
        for rep in range(2):
            # the slot's layout: every tensor starts at a multiple of four elements (1001 -> the second one at 1004)
            pa, pb = rs.randn(a.size).astype("f4"), rs.randn(*b.shape).astype("f4")
            peer = np.zeros(1004 + 80, "f4")
            peer[:a.size] = pa
            peer[1004:1004 + b.size] = pb.ravel()
            runtime.check(L.cgtb_peer_selftest_post(peer.ctypes.data_as(ctypes.c_void_p), peer.size), "post")
            runtime.check(_allreduce(L, [da, db], [oa, ob]), "peer allreduce")
            runtime.synchronize()
            assert np.array_equal(oa.get(), a + pa)
            assert np.array_equal(ob.get(), b + pb)
        # a payload beyond the slot is refused before anything is launched
        big = Dev(shape=((1 << 16) // 4 + 1,), dtype="f4")
        assert _allreduce(L, [big], [big]) != 0 and "exceed the slot" in runtime.last_error()
    finally:
        L.cgtb_peer_close()
    assert L.cgtb_peer_world() == 1
