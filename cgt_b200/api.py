"""numpy-like symbolic API (counterpart of the reference's cgt/api.py and cgt/api_autogen.py).

Every function builds graph nodes through ``core.Result``; none touches data. The subset is what the
compiled-graph path needs: variable constructors, elementwise wrappers, broadcast, cast, constant,
dot, fill/zeros/ones, reshape/flatten/transpose/dimshuffle, shape/size, arange, sum/max/mean/norm/prod,
subtensor / inc_subtensor (cases 1-3), concatenate/stack, shared, sub2ind, tuple helpers.
"""
import operator
from functools import reduce

import numpy as np

from . import core, utils

cgt = None  # the package namespace; set by cgt_b200/__init__.py


# ---------------------------------------------------------------- variable constructors
def _argument(ndim):
    def make(name=None, dtype=None, fixed_shape=None):
        return core.Argument(core.TensorType(cgt.floatX if dtype is None else dtype, ndim), name, fixed_shape=fixed_shape)
    make.__doc__ = ("Symbolic argument of rank %d. `fixed_shape` is a tuple of int or None giving the known "
                    "shape components; known sizes become compile-time constants." % ndim)
    return make


scalar = _argument(0)
vector = _argument(1)
matrix = _argument(2)
tensor3 = _argument(3)
tensor4 = _argument(4)


def tensor(dtype, ndim, name=None, fixed_shape=None):
    return core.Argument(core.TensorType(cgt.floatX if dtype is None else dtype, ndim), name, fixed_shape=fixed_shape)


# ---------------------------------------------------------------- elementwise wrappers (api_autogen.py)
def _unary(opname):
    def f(x):
        return core.Result(core.ElwiseUnary(opname), [x])
    f.__doc__ = "Applies function %s elementwise to argument x" % opname
    return f


abs = _unary("abs")  # pylint: disable=W0622
ceil = _unary("ceil")
cos = _unary("cos")
exp = _unary("exp")
iceil = _unary("iceil")
ifloor = _unary("ifloor")
log = _unary("log")
negative = _unary("neg")
sigmoid = _unary("sigmoid")
sign = _unary("sign")
sin = _unary("sin")
sqrt = _unary("sqrt")
square = _unary("square")
tanh = _unary("tanh")


def _binary(opname):
    def f(x, y):
        return core.elwise_binary(opname, x, y)
    f.__doc__ = "Applies function %s elementwise to arguments x,y" % opname
    return f


add = _binary("+")
divide = _binary("/")
equal = _binary("==")
greater = _binary(">")
greater_equal = _binary(">=")
less = _binary("<")
less_equal = _binary("<=")
multiply = _binary("*")
not_equal = _binary("!=")
power = _binary("**")
subtract = _binary("-")


# ---------------------------------------------------------------- symbolic functions
def add_multi(xs):
    """xs[0] + xs[1] + ... as a left fold, which fixes the floating-point order (cgt/api.py:53-57)."""
    return reduce(operator.add, xs)


def mul_multi(xs):
    return reduce(operator.mul, xs) if len(xs) > 0 else constant(np.array(1, dtype="i8"))


def arange(start, stop=None, step=1, dtype=None):
    if stop is None:
        (start, stop) = (0, start)
    if dtype is None:
        dtype = "i8"
    return core.Result(core.Arange(dtype), [start, stop, step])


def batched_matmul(x, y):
    """x_nij, y_njk -> z_nik"""
    return core.Result(core.BatchedMul22(False, False), [x, y])


def broadcast(opname, a, b, bcpat):
    """Elementwise binary op with explicit expansion of singleton axes.

    bcpat: "x1,1x"-style pattern, one string per operand; '1' marks a singleton axis that is
    repeated to the other operand's extent (cgt/api.py:92-120).
    """
    x, y = a, b
    (xpat, ypat) = bcpat.split(",")
    (xbcaxes, ybcaxes) = [[i for (i, letter) in enumerate(pat) if letter == "1"] for pat in (xpat, ypat)]
    assert x.ndim == y.ndim
    if xbcaxes:
        x = core.Result(core.Repeat(xbcaxes), [x] + [size(y, ax) for ax in xbcaxes])
    if ybcaxes:
        y = core.Result(core.Repeat(ybcaxes), [y] + [size(x, ax) for ax in ybcaxes])
    return core.elwise_binary(opname, x, y)


def _get_nu_cast(dtype):
    def _nu_cast(x, out=None):
        r = np.asarray(x).astype(dtype)
        if out is None:
            return r
        out[...] = r
    return _nu_cast


def cast(x, dtype):
    """Convert variable x to `dtype` (an ElwiseUnary with the identity expression, cgt/api.py:131-143)."""
    x = core.as_node(x)
    if x.dtype == dtype:
        return x
    diff = core.dtype_kind(dtype) in "cf"
    opname = "cast_to_%s" % dtype
    ui = core.UnaryInfo(opname, _get_nu_cast(dtype), diff, dtype,
                        lambda x, y, gy: cast(gy, x.dtype) if diff else None, "x")
    return core.Result(core.ElwiseUnary(opname, ui), [x])


def ceil_divide(x, y):
    return iceil(x / y)


def floor_divide(x, y):
    return ifloor(x / y)


def concatenate(xs, axis=0):
    return core.Result(core.Concatenate(axis), list(xs))


def constant(val):
    if isinstance(val, tuple):
        raise core.Todo("tuple constants")
    return core.Result(core.ConstantTensor(core.as_valid_array(val)), [])


def dot(x, y):
    x, y = core.as_node(x), core.as_node(y)
    if x.ndim == 2 and y.ndim == 2:
        return core.Result(core.Mul22(False, False), [x, y])
    raise NotImplementedError("dot is implemented for matrix x matrix on this backend")


def fill(val, shape):  # pylint: disable=W0621
    assert isinstance(shape, list)
    val = core.as_node(val)
    if isinstance(val.op, core.Constant):
        return core.Result(core.Fill(val.op.value), shape)
    singleton = reshape(val, [1] * len(shape))
    return core.Result(core.Repeat(list(range(len(shape)))), [singleton] + shape)


def flatten(x):
    return reshape(x, [mul_multi(shape(x))])


def _iscolon(sli):
    return isinstance(sli, slice) and sli.start is None and sli.stop is None and sli.step is None


def _is_int_scalar(x):
    return (isinstance(x, (int, np.integer)) and not isinstance(x, bool)) \
        or (isinstance(x, core.Node) and x.ndim == 0 and core.dtype_kind(x.dtype) == "i")


def _is1dintarray(x):
    if isinstance(x, core.Node):
        return x.ndim == 1 and core.dtype_kind(x.dtype) == "i"
    return isinstance(x, np.ndarray) and x.ndim == 1 and x.dtype.kind == "i"


def subtensor(x, slis):
    """x[slis] for: (1) ':' / None, (2) ':' / slice / int, (3) x.ndim int vectors (cgt/api.py:288-350)."""
    return _subtensor(x, slis)


def inc_subtensor(x, slis, y):
    """Copy of x with x[slis] += y (in place when the compiler can alias the buffers)."""
    return _subtensor(x, slis, y)


def _subtensor(x, slis, y=None):
    x = core.as_node(x)
    if y is not None:
        y = core.as_node(y)
    assert x.is_tensor()
    slis = list(slis) if isinstance(slis, (list, tuple)) else [slis]
    if all(_iscolon(sli) or sli is None for sli in slis):
        assert y is None
        return _subtensor1(x, slis)
    elif all(_iscolon(sli) or isinstance(sli, slice) or _is_int_scalar(sli) for sli in slis):
        if y is not None:
            assert sum(not _iscolon(sli) for sli in slis) == 1, \
                "currently can only increment subtensor involving a slice along one axis"
        return _subtensor2(x, slis, y)
    elif len(slis) == x.ndim and all(_is1dintarray(sli) for sli in slis):
        return _subtensor3(x, slis, y)
    raise ValueError("Tried to index with slices %s. See cgt.subtensor docstring for valid indexing expressions" % slis)


def _subtensor1(x, slis):
    axidx = 0
    newshape = []
    for sli in slis:
        if _iscolon(sli):
            newshape.append(size(x, axidx))
            axidx += 1
        else:
            newshape.append(1)
    return x.reshape(newshape)


def _subtensor2(x, slis, y):
    dims2drop = []
    for (ax, sli) in enumerate(slis):
        if _iscolon(sli):
            continue
        if _is_int_scalar(sli):
            if y is None:
                dims2drop.append(ax)
            else:
                yshape = cgt.shape(y)
                yshape.insert(ax, 1)
                y = y.reshape(yshape)
            sli = slice(sli, sli + 1, 1)
        step = 1 if sli.step is None else sli.step
        assert isinstance(step, (int, core.Node)), "step of a slice should be an integer or a symbolic variable"
        if isinstance(step, int) and step < 0:
            start = size(x, ax) - 1 if sli.start is None else sli.start
            stop = -1 if sli.stop is None else sli.stop
        else:
            start = 0 if sli.start is None else sli.start
            stop = size(x, ax) if sli.stop is None else sli.stop
        if y is None:
            x = core.Result(core.GetSli(ax), [x, start, stop, step])
        else:
            return core.Result(core.IncSli(ax), [x, start, stop, step, y])
    return _dropdims(x, dims2drop)


def _subtensor3(x, slis, y):
    slis = [core.as_node(s) for s in slis]
    flatinds = sub2ind(slis, shape(x))
    if y is None:
        return core.Result(core.GetFlatIndices(), [x, flatinds])
    return core.Result(core.IncFlatIndices(), [x, flatinds, y])


def make_tuple(*xs):
    return core.Result(core.MakeTuple(), list(xs))


def max(x, axis=None, keepdims=False):  # pylint: disable=W0622
    axes = _red_axes(axis, x.ndim)
    out = core.Result(core.Max(axes), [x])
    if not keepdims:
        out = _dropdims(out, axes)
    return out


def mean(x, axis=None, keepdims=False):
    """sum / number of elements; the divisor is an int64 scalar, so the division is carried out in
    double and narrowed (cgt/api.py:470-476)."""
    if x.dtype == "i1":
        x = cgt.cast(x, cgt.floatX)
    axes = _red_axes(axis, x.ndim)
    return sum(x, axis=axes, keepdims=keepdims) / mul_multi([size(x, ax) for ax in axes])


def norm(x, axis=None, p=2, keepdims=False):
    if p == 2:
        return sqrt(square(x).sum(axis=axis, keepdims=keepdims))
    return power(power(x, p).sum(axis=axis, keepdims=keepdims), 1.0 / p)


def ones(shape, dtype=None):  # pylint: disable=W0621
    if dtype is None:
        dtype = cgt.floatX
    return core.Result(core.Fill(np.array(1, dtype)), list(shape))


def ones_like(x):
    return ones(shape(x), x.dtype)


def zeros(shape, dtype=None):  # pylint: disable=W0621
    if dtype is None:
        dtype = cgt.floatX
    return core.Result(core.Fill(np.array(0, dtype)), list(shape))


def zeros_like(x):
    return zeros(shape(x), x.dtype)


def prod(x, axis=None, keepdims=False):
    return cgt.exp(cgt.sum(cgt.log(x), axis=axis, keepdims=keepdims))


def repeat(x, repeats, axis):
    return core.Result(core.Repeat([axis]), [x, core.as_node(repeats)])


def reshape(x, shp):
    shp = [core.as_node(s) for s in shp]
    assert all(s.ndim == 0 and core.dtype_kind(s.dtype) == "i" for s in shp)
    return core.Result(core.Reshape(), [x] + list(shp))


def set_precision(prec):
    """prec in {"single", "double"}: global float dtype."""
    assert prec in ("single", "double")
    if prec == "single":
        cgt.floatX, cgt.complexX = "f4", "c8"
    else:
        cgt.floatX, cgt.complexX = "f8", "c16"
    core.floatX, core.complexX = cgt.floatX, cgt.complexX


def get_precision():
    return {"f4": "single", "f8": "double"}[cgt.floatX]


def shape(x):
    x = core.as_node(x)
    if isinstance(x.typ, core.TensorType):
        return [size(x, i) for i in range(x.ndim)]
    return tuple(map(shape, x.parents))


def shared(value, name=None, device=None, fixed_shape_mask=None):
    """Variable with a persistent value that updates can change (device memory for devtype "gpu")."""
    op = core.InMemoryData(value, device=device, fixed_shape_mask=fixed_shape_mask)
    return core.Result(op, [], name=name)


def size(x, axis):
    return core.Result(core.Size(axis), [x])


def stack(tensors, axis=0):
    assert len(tensors) > 0 and 0 <= axis <= tensors[0].ndim
    shp = shape(tensors[0])
    newshp = shp[:axis] + [1] + shp[axis:]
    return concatenate([reshape(t, newshp) for t in tensors], axis=axis)


def sub2ind(subs, shp):
    """Flat index of multi-indices, row-major (cgt/api.py:630-639)."""
    ndim = len(shp)
    assert ndim >= 1
    strides = [None] * (ndim - 1) + [1]
    for i in range(ndim - 2, -1, -1):
        strides[i] = shp[i + 1] * strides[i + 1]
    return add_multi([stride * sub for (stride, sub) in utils.safezip(strides, subs)])


def sum(x, axis=None, keepdims=False):  # pylint: disable=W0622
    axes = _red_axes(axis, x.ndim)
    if len(axes) == 0:
        return x
    out = core.Result(core.Sum(axes), [x])
    if not keepdims:
        out = _dropdims(out, axes)
    return out


def transpose(arr, axes=None):
    if axes is None:
        assert arr.ndim == 2
        axes = [1, 0]
    else:
        assert isinstance(axes, (list, tuple)) and len(axes) == arr.ndim
        axes = list(axes)
    if axes == list(range(arr.ndim)):
        return arr
    return core.Result(core.Transpose(axes), [arr])


def tuple_index(x, i):
    return core.Result(core.TupleIndex(i), [x])


def _dropdims(x, axes):
    return reshape(x, [size(x, i) for i in range(x.ndim) if i not in axes])


def _red_axes(axis, ndim):
    if axis is None:
        return list(range(ndim))
    elif isinstance(axis, int):
        return [axis]
    elif isinstance(axis, (list, tuple)):
        return list(axis)
    raise ValueError("invalid argument 'axis'=%s" % axis)


def dimshuffle(arr, pattern):
    """Permute axes and insert singleton axes ('x'), e.g. [1, 0, 'x'] (cgt/api.py:744-785)."""
    assert isinstance(pattern, list)
    if pattern == list(range(arr.ndim)):
        return arr
    shapes, x_idxs, clean = [], [], []
    array_shape = arr.shape
    for (idx, p) in enumerate(pattern):
        if p == "x":
            shapes.append(1)
            x_idxs.append(idx)
        else:
            shapes.append(array_shape[p])
            clean.append(p)
    assert len(clean) == arr.ndim
    result = transpose(arr, clean)
    if x_idxs:
        result = reshape(result, shapes)
    return result
