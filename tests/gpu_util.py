"""Helpers for the GPU parity tests: move numpy arrays to device memory owned by the runtime pool and
call the plain-pointer C ABI of libcgt_b200.so."""
import ctypes

import numpy as np

from cgt_b200 import runtime


class Dev(object):
    """numpy array copied to the device; `.ptr` is the device address, `.get()` copies back."""

    def __init__(self, arr=None, shape=None, dtype=None):
        if arr is not None:
            arr = np.asarray(arr, order="C")
            self.w = runtime.device_array(arr)
            self.shape, self.dtype = arr.shape, arr.dtype
        else:
            self.w = runtime.device_array(np.zeros(shape, dtype))
            self.shape, self.dtype = tuple(shape), np.dtype(dtype)

    @property
    def ptr(self):
        return ctypes.c_void_p(self.w.data)

    def get(self):
        return self.w.to_numpy()


def code(dtype):
    return runtime._dtype_code(dtype)


def longs(xs):
    return (ctypes.c_long * max(len(xs), 1))(*[int(x) for x in xs])


def ints(xs):
    return (ctypes.c_int * max(len(xs), 1))(*[int(x) for x in xs])


def call(name, *args):
    L = runtime.lib()
    rc = getattr(L, name)(*args)
    runtime.check(rc, name)
    runtime.synchronize()
