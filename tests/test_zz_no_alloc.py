"""The allocation-free reduction entry point, called through the C ABI and compared with cgtb_reduce.

Collected last (file name) so that it also runs after every other GPU test has used the runtime's
pools; it passes alone as well."""
import ctypes

import numpy as np
import pytest

from cgt_b200 import runtime
from tests.gpu_util import Dev, call, code, ints, longs

pytestmark = pytest.mark.gpu

CASES = [
    # (R0, K, R1): bias gradient of the CIFAR convnet, a column block, a full sum, one block per output
    (128, 32, 1024),
    (64, 7, 333),
    (1, 1, 300000),
    (3, 2000, 65),
    (128, 10, 2),
]


def _signatures():
    L = runtime.lib()
    L.cgtb_reduce_rkr_f32_static.restype = ctypes.c_int
    L.cgtb_reduce_rkr_f32_static.argtypes = [ctypes.c_int, ctypes.c_long, ctypes.c_long, ctypes.c_long, ctypes.c_void_p,
                                             ctypes.c_void_p]
    L.cgtb_reduce_static_max_k.restype = ctypes.c_long
    return L


@pytest.mark.parametrize("kind", [0, 1])
def test_static_reduce_matches_pooled_reduce_twice(rt, kind):
    _signatures()
    rs = np.random.RandomState(11)
    for rep in range(2):  # two calls in a row share the fixed array: the second must not see the first
        for (R0, K, R1) in CASES:
            x = rs.randn(R0, K, R1).astype("f4")
            dx = Dev(x)
            want, got = Dev(shape=(1, K, 1), dtype="f4"), Dev(np.full((K,), 7.0, "f4"))
            call("cgtb_reduce", kind, code("f4"), 3, longs((R0, K, R1)), ints((1, 0, 1)), dx.ptr, want.ptr)
            call("cgtb_reduce_rkr_f32_static", kind, R0, K, R1, dx.ptr, got.ptr)
            w, g = want.get().reshape(K), got.get()
            assert np.array_equal(w, g), (rep, R0, K, R1)
            exact = x.astype("f8").sum(axis=(0, 2)) if kind == 0 else x.max(axis=(0, 2))
            assert np.allclose(g, exact, rtol=1e-4, atol=1e-5 * np.sqrt(R0 * R1))


def test_static_reduce_back_to_back_without_sync(rt):
    """Two calls queued on the runtime stream with no host synchronisation in between."""
    L = _signatures()
    rs = np.random.RandomState(12)
    a, b = rs.randn(128, 32, 1024).astype("f4"), rs.randn(96, 5, 700).astype("f4")
    da, db = Dev(a), Dev(b)
    oa, ob = Dev(shape=(32,), dtype="f4"), Dev(shape=(5,), dtype="f4")
    runtime.check(L.cgtb_reduce_rkr_f32_static(0, 128, 32, 1024, da.ptr, oa.ptr), "static reduce")
    runtime.check(L.cgtb_reduce_rkr_f32_static(0, 96, 5, 700, db.ptr, ob.ptr), "static reduce")
    runtime.synchronize()
    wa, wb = Dev(shape=(1, 32, 1), dtype="f4"), Dev(shape=(1, 5, 1), dtype="f4")
    call("cgtb_reduce", 0, code("f4"), 3, longs(a.shape), ints((1, 0, 1)), da.ptr, wa.ptr)
    call("cgtb_reduce", 0, code("f4"), 3, longs(b.shape), ints((1, 0, 1)), db.ptr, wb.ptr)
    assert np.array_equal(oa.get(), wa.get().reshape(-1))
    assert np.array_equal(ob.get(), wb.get().reshape(-1))


def test_static_reduce_allocates_nothing_and_refuses_oversize(rt):
    L = _signatures()
    x = Dev(np.ones((4, 8, 64), "f4"))
    out = Dev(shape=(8,), dtype="f4")
    call("cgtb_reduce_rkr_f32_static", 0, 4, 8, 64, x.ptr, out.ptr)  # set-up call
    stats = lambda: runtime.pool_stats()
    before = stats()
    for _ in range(3):
        call("cgtb_reduce_rkr_f32_static", 0, 4, 8, 64, x.ptr, out.ptr)
    assert stats() == before  # the runtime's pools were not touched
    assert np.array_equal(out.get(), np.full((8,), 256.0, "f4"))
    kmax = L.cgtb_reduce_static_max_k()
    assert kmax == 8192
    rc = L.cgtb_reduce_rkr_f32_static(0, 1, kmax + 1, 4, x.ptr, out.ptr)
    assert rc != 0
    msg = runtime.last_error()
    assert "beyond the maximum" in msg and str(kmax) in msg
    rc = L.cgtb_reduce_rkr_f32_static(0, 1 << 30, 2, 4, x.ptr, out.ptr)
    assert rc != 0 and "beyond the maximum" in runtime.last_error()
    # a pure column reduction is not split, needs no scratch and is served by cgtb_reduce only
    rc = L.cgtb_reduce_rkr_f32_static(0, 16, 8, 1, x.ptr, out.ptr)
    assert rc != 0 and "use cgtb_reduce" in runtime.last_error()
    # an error leaves the entry point usable
    call("cgtb_reduce_rkr_f32_static", 1, 4, 8, 64, x.ptr, out.ptr)
    assert np.array_equal(out.get(), np.ones((8,), "f4"))
