"""TEST INFRASTRUCTURE, NOT PRODUCT CODE.

numpy-facing bindings of the CPU checker libraries:

* ``liboracle.so`` (``cgt_oracle.cpp``): restatement of the reference's native CPU kernels;
* ``_ref/libcgt_ref.so`` (``ref_shim.cpp``): the reference's own headers, when built.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline / reference arm may
import this module. Nothing under ``cgt_b200/`` does.

Every function takes and returns C-contiguous numpy arrays. ``impl="port"`` runs the restatement,
``impl="ref"`` runs the reference's own code (raises if it was not built or does not cover the case).
Mul22 is OpenBLAS sgemm through numpy (reference call: cgt/core.py:2196-2205).
"""
import ctypes
import math
import os.path as osp

import numpy as np

HERE = osp.dirname(osp.abspath(__file__))

UNARY = {"abs": 0, "ceil": 1, "cos": 2, "exp": 3, "iceil": 4, "ifloor": 5, "log": 6, "neg": 7, "sign": 8,
         "sin": 9, "square": 10, "sqrt": 11, "tanh": 12, "sigmoid": 13, "softplus": 14, "cast": 15}
BINARY = {"*": 0, "+": 1, "-": 2, "/": 3, "<": 4, ">": 5, "<=": 6, ">=": 7, "**": 8, "==": 9, "!=": 10}
DTYPE_NUM = {"i1": 1, "i2": 3, "i4": 5, "i8": 7, "f4": 11, "f8": 12}

_c_long = ctypes.c_long
_c_int = ctypes.c_int
_c_double = ctypes.c_double
_vp = ctypes.c_void_p


def _load(path):
    if not osp.exists(path):
        return None
    return ctypes.CDLL(path)


def _ensure_built():
    path = osp.join(HERE, "liboracle.so")
    if not osp.exists(path):
        from . import build_oracle
        build_oracle.build_restatement()
    return path


_port = _load(_ensure_built())
_ref = _load(osp.join(HERE, "_ref", "libcgt_ref.so"))


def have_ref():
    return _ref is not None


def _dt(a):
    a = np.dtype(a)
    return DTYPE_NUM["%s%d" % ("f" if a.kind == "f" else "i", a.itemsize)]


def _p(a):
    return ctypes.c_void_p(a.ctypes.data)


def _suffix(dtype):
    return {np.dtype("f4"): "f32", np.dtype("f8"): "f64"}[np.dtype(dtype)]


def _lib(impl):
    if impl == "port":
        return _port, "orc_"
    if impl == "ref":
        if _ref is None:
            raise RuntimeError("oracle/_ref was not built (reference tree absent)")
        return _ref, "ref_"
    raise ValueError(impl)


def _c(a, dtype=None):
    return np.asarray(a, dtype=dtype, order="C")  # keeps 0-d arrays 0-d


# ------------------------------------------------------------------------------------------------
# shapes
# ------------------------------------------------------------------------------------------------
def conv_out_size(size, k, pad, stride):
    """(H + 2p - k) // s + 1 : cgt/nn_ops/im2col.py:39-40"""
    return (size + 2 * pad - k) // stride + 1


def pool_out_size(size, k, pad, stride):
    """iceil((H + 2p - k) / s) with a double division and NO +1 : cgt/nn_ops/max_pool_2d.py:40-41"""
    return int(math.ceil((size + 2 * pad - k + 0.0) / stride))


# ------------------------------------------------------------------------------------------------
# im2col / col2im
# ------------------------------------------------------------------------------------------------
def im2col(x, kernel, pad, stride, impl="port"):
    x = _c(x)
    B, C, H, W = x.shape
    (kh, kw), (ph, pw), (sh, sw) = kernel, pad, stride
    Ho, Wo = conv_out_size(H, kh, ph, sh), conv_out_size(W, kw, pw, sw)
    col = np.empty((B, Ho, Wo, C * kh * kw), x.dtype)
    lib, pre = _lib(impl)
    f = getattr(lib, pre + "im2col_" + _suffix(x.dtype))
    f.restype = _c_int
    rc = f(_p(x), _c_long(B), C, H, W, kh, kw, ph, pw, sh, sw, _p(col))
    if impl == "ref" and rc != 0:
        raise RuntimeError("geometry %s not instantiated in ref_shim.cpp" % ((kernel, pad, stride),))
    return col


def col2im(col, xshape, kernel, pad, stride, impl="port"):
    col = _c(col)
    B, C, H, W = xshape
    (kh, kw), (ph, pw), (sh, sw) = kernel, pad, stride
    im = np.empty((B, C, H, W), col.dtype)
    lib, pre = _lib(impl)
    f = getattr(lib, pre + "col2im_" + _suffix(col.dtype))
    f.restype = _c_int
    rc = f(_p(col), _c_long(B), C, H, W, kh, kw, ph, pw, sh, sw, _p(im))
    if impl == "ref" and rc != 0:
        raise RuntimeError("geometry %s not instantiated in ref_shim.cpp" % ((kernel, pad, stride),))
    return im


# ------------------------------------------------------------------------------------------------
# max pool
# ------------------------------------------------------------------------------------------------
def max_pool(x, kernel, pad, stride, impl="port"):
    x = _c(x)
    B, C, H, W = x.shape
    (kh, kw), (ph, pw), (sh, sw) = kernel, pad, stride
    PH, PW = pool_out_size(H, kh, ph, sh), pool_out_size(W, kw, pw, sw)
    top = np.empty((B, C, PH, PW), x.dtype)
    mask = np.empty((B, C, PH, PW), np.int32)
    lib, pre = _lib(impl)
    f = getattr(lib, pre + "max_pool_" + _suffix(x.dtype))
    f.restype = None
    f(_p(x), _c_long(B), C, H, W, kh, kw, ph, pw, sh, sw, PH, PW, _p(top), _p(mask))
    return top, mask


def max_pool_pullback(xshape, mask, gtop, impl="port"):
    mask = _c(mask, np.int32)
    gtop = _c(gtop)
    B, C, H, W = xshape
    PH, PW = mask.shape[2:]
    gx = np.empty((B, C, H, W), gtop.dtype)
    lib, pre = _lib(impl)
    f = getattr(lib, pre + "max_pool_pullback_" + _suffix(gtop.dtype))
    f.restype = None
    f(_p(mask), _p(gtop), _c_long(B), C, PH, PW, H, W, _p(gx))
    return gx


# ------------------------------------------------------------------------------------------------
# cross-channel LRN
# ------------------------------------------------------------------------------------------------
def lrn_forward(x, size, alpha, beta, impl="port"):
    x = _c(x)
    N, C, H, W = x.shape
    assert C >= size, "the reference kernels assume channels >= localsize (lrn.cuh:20-29)"
    top = np.empty_like(x)
    scale = np.empty_like(x)
    lib, pre = _lib(impl)
    f = getattr(lib, pre + "lrn_forward_" + _suffix(x.dtype))
    f.restype = None
    f(_p(x), _c_long(N), C, H, W, size, _c_double(alpha), _c_double(beta), _p(top), _p(scale))
    return top, scale


def lrn_backward(x, top, scale, gtop, size, alpha, beta, impl="port"):
    x, top, scale, gtop = _c(x), _c(top), _c(scale), _c(gtop)
    N, C, H, W = x.shape
    gx = np.empty_like(x)
    lib, pre = _lib(impl)
    f = getattr(lib, pre + "lrn_backward_" + _suffix(x.dtype))
    f.restype = None
    f(_p(x), _p(top), _p(scale), _p(gtop), _c_long(N), C, H, W, size, _c_double(alpha), _c_double(beta), _p(gx))
    return gx


# ------------------------------------------------------------------------------------------------
# elementwise
# ------------------------------------------------------------------------------------------------
def unary(opname, x, out_dtype):
    x = _c(x)
    out = np.empty(x.shape, out_dtype)
    rc = _port.orc_unary(UNARY[opname], _dt(x.dtype), _dt(out.dtype), _c_long(x.size), _p(x), _p(out))
    assert rc == 0
    return out


def binary(opname, x, y, out_dtype):
    """x and y have identical shapes, or one of them is 0-d (cgt/core.py:1380-1386)."""
    x, y = _c(x), _c(y)
    sx, sy = x.ndim == 0, y.ndim == 0
    shape = y.shape if sx else x.shape
    if not (sx or sy):
        assert x.shape == y.shape, "no implicit broadcasting"
    out = np.empty(shape, out_dtype)
    rc = _port.orc_binary(BINARY[opname], _dt(x.dtype), _dt(y.dtype), _dt(out.dtype), _c_long(out.size),
                          _p(x), _p(y), _p(out), int(sx), int(sy))
    assert rc == 0
    return out


# ------------------------------------------------------------------------------------------------
# reductions and data movement
# ------------------------------------------------------------------------------------------------
def _longs(xs):
    return (ctypes.c_long * max(len(xs), 1))(*xs)


def _ints(xs):
    return (ctypes.c_int * max(len(xs), 1))(*xs)


def reduce(kind, x, axes):
    """kind in {"sum", "max"}; keepdims always (cgt/core.py:1701-1704)."""
    x = _c(x)
    red = [1 if i in axes else 0 for i in range(x.ndim)]
    oshape = tuple(1 if r else s for r, s in zip(red, x.shape))
    out = np.empty(oshape, x.dtype)
    rc = _port.orc_reduce({"sum": 0, "max": 1}[kind], _dt(x.dtype), x.ndim, _longs(x.shape), _ints(red), _p(x), _p(out))
    assert rc == 0
    return out


def repeat(x, axes, reps):
    x = _c(x)
    oshape = list(x.shape)
    for ax, r in zip(axes, reps):
        assert x.shape[ax] == 1
        oshape[ax] = int(r)
    out = np.empty(oshape, x.dtype)
    rc = _port.orc_repeat(_dt(x.dtype), x.ndim, _longs(oshape), _ints([1 if i in axes else 0 for i in range(x.ndim)]),
                          _p(x), _p(out))
    assert rc == 0
    return out


def transpose(x, axes):
    x = _c(x)
    out = np.empty([x.shape[a] for a in axes], x.dtype)
    rc = _port.orc_transpose(_dt(x.dtype), x.ndim, _longs(x.shape), _ints(list(axes)), _p(x), _p(out))
    assert rc == 0
    return out


def _split(shape, axis):
    outer = int(np.prod(shape[:axis], dtype=np.int64))
    inner = int(np.prod(shape[axis + 1:], dtype=np.int64))
    return outer, int(shape[axis]), inner


def getsli(x, axis, start, stop, step):
    x = _c(x)
    n_out = int(math.ceil((stop - start + 0.0) / step))  # ceil_divide, cgt/core.py:1788
    oshape = list(x.shape)
    oshape[axis] = n_out
    out = np.empty(oshape, x.dtype)
    outer, n_in, inner = _split(x.shape, axis)
    rc = _port.orc_getsli(_dt(x.dtype), _c_long(outer), _c_long(n_in), _c_long(inner), _c_long(start), _c_long(step),
                          _c_long(n_out), _p(x), _p(out))
    assert rc == 0
    return out


def incsli(x, axis, start, stop, step, inc):
    x, inc = _c(x), _c(inc)
    out = np.empty_like(x)
    outer, n_x, inner = _split(x.shape, axis)
    rc = _port.orc_incsli(_dt(x.dtype), _c_long(outer), _c_long(n_x), _c_long(inner), _c_long(start), _c_long(step),
                          _c_long(inc.shape[axis]), _p(x), _p(inc), _p(out))
    assert rc == 0
    return out


def getflat(x, k):
    x, k = _c(x), _c(k, np.int64)
    out = np.empty(k.shape, x.dtype)
    rc = _port.orc_getflat(_dt(x.dtype), _c_long(k.size), _p(x), _p(k), _p(out))
    assert rc == 0
    return out


def incflat(x, k, p):
    x, k, p = _c(x), _c(k, np.int64), _c(p)
    out = np.empty_like(x)
    rc = _port.orc_incflat(_dt(x.dtype), _c_long(x.size), _c_long(k.size), _p(x), _p(k), _p(p), _p(out))
    assert rc == 0
    return out


def concatenate(xs, axis):
    xs = [_c(x) for x in xs]
    oshape = list(xs[0].shape)
    oshape[axis] = sum(x.shape[axis] for x in xs)
    out = np.empty(oshape, xs[0].dtype)
    pos = 0
    for x in xs:
        outer, n_in, inner = _split(x.shape, axis)
        rc = _port.orc_concat_part(_dt(x.dtype), _c_long(outer), _c_long(n_in), _c_long(oshape[axis]), _c_long(inner),
                                   _c_long(pos), _p(x), _p(out))
        assert rc == 0
        pos += n_in
    return out


def fill(value, shape, dtype):
    out = np.empty(shape, dtype)
    kind = np.dtype(dtype).kind
    rc = _port.orc_fill(_dt(dtype), _c_long(out.size), _c_double(float(value)), _c_long(int(value) if kind == "i" else 0),
                        _p(out))
    assert rc == 0
    return out


def arange(start, stop, step):
    """cgt/core.py:1037-1048 : size = (stop-start)/step with C integer division, dtype i8"""
    size = int((stop - start) / step) if step else 0
    return (start + step * np.arange(size, dtype=np.int64)).astype(np.int64)


# ------------------------------------------------------------------------------------------------
# GEMM (OpenBLAS through numpy)
# ------------------------------------------------------------------------------------------------
def mul22(A, B, tA=False, tB=False):
    A, B = _c(A), _c(B)
    a = A.T if tA else A
    b = B.T if tB else B
    return np.ascontiguousarray(a @ b)


def batched_mul22(A, B, tA=False, tB=False):
    A, B = _c(A), _c(B)
    return np.stack([mul22(a, b, tA, tB) for a, b in zip(A, B)])
