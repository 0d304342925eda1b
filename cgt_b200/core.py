"""Graph core of the B200 backend: types, nodes, the Op contract, reverse-mode differentiation, the
simplifier, and the configuration dictionary.

Mirrors the operator API of the reference's ``cgt/core.py`` (Node :169, Op :393, Result :511,
pullback :633, grad :713, NativeCompileInfo :734, simplify_and_analyze :2546, config :2948-3033) so
that model code and user-defined Ops written against that API run unchanged, in Python 3. The Ops
defined here return ``NativeCompileInfo`` objects that name a prebuilt entry point of
``libcgt_b200.so`` instead of carrying generated C++ text; Ops that do carry code strings are still
compiled at run time by ``compilation.nci2callable``.
"""
import ctypes
import hashlib
import math
import os
import pickle
import traceback
from collections import defaultdict, namedtuple
from functools import reduce

import numpy as np

from . import utils

# set by cgt_b200/__init__.py once the package namespace exists (the reference does `import cgt`)
cgt = None

floatX = "f4"
complexX = "c8"


# ================================================================
# Datatypes
# ================================================================

class Dtype:
    @staticmethod
    def canon(dt):
        """Canonical dtype string; every float maps to the configured floatX (cgt/core.py:12-32)."""
        dt = np.dtype(dt)
        k = dt.kind
        if k == "f":
            return cgt.floatX
        elif k in "biu":
            return "i" + str(dt.itemsize)
        elif k == "c":
            return cgt.complexX
        raise ValueError("Invalid dtype %s" % dt)


def as_valid_array(x, dtype=None):
    """numpy array of a valid dtype, C-contiguous (cgt/core.py:34-43)."""
    if not isinstance(x, np.ndarray):
        x = np.asarray(x, dtype=dtype)
    if dtype is None:
        dtype = Dtype.canon(x.dtype)
    x = x.astype(dtype, copy=False)
    if not x.flags.c_contiguous:
        x = np.ascontiguousarray(x) if x.ndim > 0 else x.copy()
    return x


def as_valid_tuple(x):
    return tuple(as_valid_array(a) for a in x)


class Type(object):
    pass


class TensorType(Type):
    """n-dimensional array type; scalars are 0-dimensional (cgt/core.py:61-76)."""

    def __init__(self, dtype, ndim):
        self.dtype = Dtype.canon(dtype)
        self.ndim = ndim

    def __repr__(self):
        return "Tensor(%s,%s)" % (self.dtype, self.ndim)

    def __eq__(self, other):
        return isinstance(other, TensorType) and self.dtype == other.dtype and self.ndim == other.ndim

    def __hash__(self):
        return hash((self.dtype, self.ndim))


class TupleType(Type):
    """Tuple of tensor types (cgt/core.py:78-99)."""

    def __init__(self, *eltypes):
        assert all(isinstance(t, TensorType) for t in eltypes)
        self.eltypes = tuple(eltypes)
        self.dtype = "O"

    def __len__(self):
        return len(self.eltypes)

    def __getitem__(self, i):
        return self.eltypes[i]

    def __iter__(self):
        return iter(self.eltypes)

    def __repr__(self):
        return "Tup(" + ",".join(map(str, self.eltypes)) + ")"

    def __eq__(self, other):
        return isinstance(other, TupleType) and self.eltypes == other.eltypes

    def __hash__(self):
        return hash((self.eltypes, self.dtype))


class Device(object):
    """Where a computation runs: devtype "cpu" or "gpu", and a device index (cgt/core.py:101-116)."""

    def __init__(self, devtype="cpu", idx=0):
        assert isinstance(devtype, str) and isinstance(idx, int)
        self.devtype = devtype
        self.idx = idx

    def __eq__(self, other):
        return self.devtype == other.devtype and self.idx == other.idx

    def __hash__(self):
        return hash((self.devtype, self.idx))

    def __repr__(self):
        return "%s/%s" % (self.devtype, self.idx)


def _promote(typ1, typ2):
    """Result dtype of an arithmetic op: complex > float > widest int (cgt/core.py:118-134)."""
    d1, s1, d2, s2 = typ1[0], int(typ1[1:]), typ2[0], int(typ2[1:])
    if d1 == "c" or d2 == "c":
        return cgt.complexX
    if d1 == "f" or d2 == "f":
        return cgt.floatX
    if d1 == "i" and d2 == "i":
        return "i%d" % max(s1, s2)
    raise ValueError("Don't know what to do with dtypes %s,%s" % (typ1, typ2))


def _promote_multi(xtypes):
    return reduce(_promote, xtypes)


def dtype_kind(dtype):
    assert isinstance(dtype, str)
    return dtype[0]


def _type_to_int(typ1):
    return "i8" if dtype_kind(typ1) in "fc" else typ1


# ================================================================
# Nodes
# ================================================================

class Node(object):
    """Node of the computation graph (cgt/core.py:169-376)."""

    counter = 0
    __array_priority__ = 1000

    def __init__(self, typ, op, parents, props=None, fixed_shape=None, name=None):
        self.typ = typ
        self.op = op
        self.parents = parents
        self.props = props or {}
        self._fixed_shape = fixed_shape
        self.name = name
        self.counter = Node.counter
        Node.counter += 1

    def __repr__(self):
        if self.op is None:
            return "Argument{%s,name='%s'}" % (self.typ, self.name)
        return "Result{%s}" % (str(self.op))

    def is_argument(self):
        return self.op is None

    def is_data(self):
        return self.op is not None and self.op.is_data_op

    def is_input(self):
        return self.is_argument() or self.is_data()

    def get_diff(self):
        return [] if self.op is None else self.op.get_diff(len(self.parents))

    def is_tensor(self):
        return isinstance(self.typ, TensorType)

    def is_tuple(self):
        return isinstance(self.typ, TupleType)

    def is_scalar(self):
        return self.is_tensor() and self.ndim == 0

    def get_hash(self, node2hash):
        if self.is_input() or self.op.is_random_op:
            return str(self.counter)
        h = hashlib.md5(self.op.get_hash())
        for p in self.parents:
            h.update(node2hash[p].encode())
        return h.hexdigest()

    def clone(self, newparents):
        if self.is_input():
            return self
        return Node(self.typ, self.op, newparents, props=self.props)

    def get_fixed_shape(self):
        if self.is_data():
            return self.op.get_fixed_shape()
        return (None,) * self.ndim if self._fixed_shape is None else self._fixed_shape

    # arithmetic
    def __neg__(self):
        return Result(ElwiseUnary("neg"), [self])

    def __add__(self, other):
        return elwise_binary("+", self, other)

    def __sub__(self, other):
        return elwise_binary("-", self, other)

    def __mul__(self, other):
        return elwise_binary("*", self, other)

    def __truediv__(self, other):
        return elwise_binary("/", self, other)

    __div__ = __truediv__

    def __pow__(self, other):
        return elwise_binary("**", self, other)

    def __floordiv__(self, other):
        return cgt.floor_divide(self, other)

    def __gt__(self, other):
        return cgt.greater(self, other)

    def __ge__(self, other):
        return cgt.greater_equal(self, other)

    def __lt__(self, other):
        return cgt.less(self, other)

    def __le__(self, other):
        return cgt.less_equal(self, other)

    def __radd__(self, other):
        return self.__add__(other)

    def __rsub__(self, other):
        return cgt.constant(other).__sub__(self)

    def __rmul__(self, other):
        return self.__mul__(other)

    def __rtruediv__(self, other):
        return cgt.constant(other).__truediv__(self)

    __rdiv__ = __rtruediv__

    def __rfloordiv__(self, other):
        return cgt.constant(other).__floordiv__(self)

    __hash__ = object.__hash__

    def __getitem__(self, slis):
        if self.is_tuple():
            assert isinstance(slis, int), "TupleType can be only be indexed by an int"
            return cgt.tuple_index(self, slis)
        return cgt.subtensor(self, slis)

    def __iter__(self):
        if self.is_tuple():
            return iter(unpack(self))
        raise TypeError("Array variable is not iterable")

    def __len__(self):
        if isinstance(self.typ, TupleType):
            return len(self.typ)
        raise ValueError("Node of type Tensor has no __len__")

    def __bool__(self):
        return True

    @property
    def shape(self):
        return cgt.shape(self)

    @property
    def ndim(self):
        return self.typ.ndim if isinstance(self.typ, TensorType) else 0

    @property
    def dtype(self):
        return self.typ.dtype

    @property
    def T(self):
        return cgt.transpose(self)

    def reshape(self, shp):
        assert isinstance(shp, (list, tuple))
        return cgt.reshape(self, shp)

    def dot(self, other):
        return cgt.dot(self, other)

    def sum(self, axis=None, keepdims=False):
        return cgt.sum(self, axis=axis, keepdims=keepdims)

    def prod(self, axis=None, keepdims=False):
        return cgt.prod(self, axis=axis, keepdims=keepdims)

    def max(self, axis=None, keepdims=False):
        return cgt.max(self, axis=axis, keepdims=keepdims)

    def mean(self, axis=None, keepdims=False):
        return cgt.mean(self, axis=axis, keepdims=keepdims)

    def transpose(self, axes=None):
        return cgt.transpose(self, axes=axes)

    def flatten(self):
        return cgt.flatten(self)

    def dimshuffle(self, pattern):
        return cgt.dimshuffle(self, pattern)


def _ndarray_type(value):
    assert isinstance(value, np.ndarray)
    return TensorType(value.dtype, value.ndim)


def _get_value_type(value):
    if isinstance(value, np.ndarray):
        return TensorType(value.dtype, value.ndim)
    elif isinstance(value, tuple):
        return TupleType(*map(_get_value_type, value))


def num_components(node):
    return len(node.typ) if isinstance(node.typ, TupleType) else 1


# ================================================================
# Op contract
# ================================================================

class Op(object):
    """An operation applied to data (cgt/core.py:393-490).

    Subclass attributes: ``return_type`` ("byref": writes into a pre-allocated output; "byval":
    returns a new object), ``writes_to_input`` (index of the input whose memory the output aliases, or
    -1), ``available_impls`` (subset of "python", "native_cpu", "native_gpu").

    One addition to the reference contract: ``host_inputs(n_inputs)`` lists the inputs a GPU
    implementation reads on the host at launch time (shape components, slice bounds); those stay on
    the host instead of being transported. It plays the role of the reference's ``gpu_deref_mask``,
    which is declared there but never consumed.
    """
    return_type = "byref"
    writes_to_input = -1
    available_impls = ()
    is_data_op = False
    is_random_op = False

    def shp_apply(self, parents):
        raise NotImplementedError

    def typ_apply(self, parent_types):
        raise NotImplementedError

    def get_diff(self, num_inputs):
        assert isinstance(num_inputs, int)
        return [True] * num_inputs

    def get_expr(self, parent_exprs):
        return "%s(%s)" % (str(self), ",".join(parent_exprs))

    def get_hash(self):
        items = sorted((k, repr(v)) for (k, v) in self.__dict__.items())
        return (type(self).__name__ + repr(items)).encode()

    def get_name(self):
        return type(self).__name__

    def get_replacement(self, _newparents, _analysis):
        return None

    def pullback(self, inputs, output, goutput):
        raise MethodNotDefined

    def pushforward(self, inputs, output, goutput):
        raise MethodNotDefined

    def get_native_compile_info(self, input_types, devtype):
        raise MethodNotDefined

    def get_py_func(self, input_types):
        raise MethodNotDefined

    def get_py_callable(self, input_types):
        func = self.get_py_func(input_types)
        return PyCallable(self, len(input_types), func)

    def host_inputs(self, num_inputs):
        return ()

    def __repr__(self):
        return type(self).__name__


def as_node(val_or_node):
    if isinstance(val_or_node, Node):
        return val_or_node
    elif isinstance(val_or_node, np.ndarray) or np.isscalar(val_or_node):
        return cgt.constant(val_or_node)
    elif isinstance(val_or_node, tuple):
        return cgt.make_tuple(*val_or_node)
    raise ValueError("expected numeric data or Node, got object of type %s" % type(val_or_node))


def default_props():
    props = {"default_device": _CONFIG["default_device"]}
    if _CONFIG["debug"]:
        props["stack"] = traceback.extract_stack()[:-3]
    return props


def Result(op, parents, typ=None, props=None, name=None):
    parents = [as_node(p) for p in parents]
    typ = op.typ_apply([p.typ for p in parents]) if typ is None else typ
    return Node(typ, op, parents, props=props or default_props(), name=name)


def Argument(typ, name=None, fixed_shape=None, props=None):
    return Node(typ, None, [], props=props or default_props(), fixed_shape=fixed_shape, name=name)


class GetData(Op):
    is_data_op = True
    return_type = "byval"
    available_impls = ("python", "native_cpu", "native_gpu")

    def __init__(self, typ):
        self.typ = typ

    def typ_apply(self, _):
        return self.typ


class InMemoryData(GetData):
    """Persistent array behind ``cgt.shared`` (cgt/core.py:534-586).

    The value lives in a runtime array on ``device`` (a GPU array for devtype "gpu"); the native
    callable returns that array, so an update expression writes straight into it.
    """

    def __init__(self, value, device=None, fixed_shape_mask=None):
        value = as_valid_array(value)
        GetData.__init__(self, _ndarray_type(value))
        self.device = device or get_config()["default_device"]
        self.dataptr = ctypes.c_void_p(0)
        self._value = None
        self.set_value(value)
        if fixed_shape_mask is None:
            fixed_shape_mask = (False,) * value.ndim
        elif fixed_shape_mask == "all":
            fixed_shape_mask = (True,) * value.ndim
        self.fixed_shape = tuple(s if fixed else None for (s, fixed) in zip(value.shape, fixed_shape_mask))

    def get_hash(self):
        return ("InMemoryData%d" % id(self)).encode()

    def get_py_func(self, _):
        def f(_reads):
            return self.get_value()
        return f

    def get_native_compile_info(self, _input_types, _devtype):
        return NativeCompileInfo(None, prebuilt="cgtb_op_in_memory_data",
                                 closure_triples=[("pptr", ctypes.c_void_p, self.get_pptr())], store_objects=self)

    def __repr__(self):
        return "Data{%s}" % (self.typ)

    def get_device(self):
        return self.device

    def get_value(self):
        return self._value.to_numpy()

    def get_shape(self):
        return self._value.shape

    def get_size(self):
        return self._value.size

    def set_value(self, value):
        from . import runtime
        value = np.asarray(value, dtype=self.typ.dtype)
        if self._value is not None and tuple(self._value.shape) == tuple(value.shape):
            self._value.set_from_numpy(value)  # keeps the buffer address (captured CUDA graphs stay valid)
        else:
            was_live = self._value is not None and self._value.handle is not None
            self._value = runtime.ArrayWrapper.from_numpy(value, self.device.devtype)
            runtime.lib().cgtb_state_version_bump()   # compiled functions must look at their storage again
            if was_live:  # compiled functions hold the address of `dataptr`: keep it pointing at a live array
                self.dataptr.value = self._value.ptr

    def get_pptr(self):
        """Address of the cell holding the runtime array's address; creates the array on first use."""
        self.dataptr.value = self._value.ptr
        return ctypes.addressof(self.dataptr)

    def get_fixed_shape(self):
        return self.fixed_shape


def _singleton_ones(dtype, ndim):
    return cgt.constant(np.ones((1,) * ndim, dtype))


def make_argument(typ):
    if isinstance(typ, TupleType):
        return Argument(TupleType(*typ))
    elif isinstance(typ, TensorType):
        return Argument(TensorType(typ.dtype, typ.ndim))
    raise ValueError("expected Tuple or Tensor. Got %s" % typ)


# ================================================================
# Differentiation (cgt/core.py:603-728)
# ================================================================

def differentiably_influences(outputs, nodelist=None):
    if nodelist is None:
        nodelist = list(topsorted(outputs))
    diset = set(outputs)
    for node in reversed(nodelist):
        if node in diset and not node.is_input():
            for (p, d) in utils.safezip(node.parents, node.get_diff()):
                if d:
                    diset.add(p)
    return diset


def differentiably_influenced_by(wrt, outputs=None, nodelist=None):
    assert (outputs is None) != (nodelist is None)
    if nodelist is None:
        nodelist = list(topsorted(outputs))
    dibset = set(wrt)
    for node in nodelist:
        if any(p in dibset and d for (p, d) in utils.safezip(node.parents, node.get_diff())):
            dibset.add(node)
    return dibset


def pullback(outputs, goutputs, wrt):
    """Reverse-mode propagation: gradients of `wrt` given gradients `goutputs` of `outputs`.

    Gradient terms of a node with several consumers are summed left to right in the order they were
    produced (``add_multi``), which fixes the floating-point summation order.
    """
    nodelist = list(topsorted(outputs))
    dio = differentiably_influences(outputs, nodelist=nodelist)
    dibw = differentiably_influenced_by(wrt, nodelist=nodelist)
    badwrtset = set(wrt).difference(dio)
    if badwrtset:
        raise NonDifferentiable("Outputs not differentiable wrt %s" % badwrtset)
    badoutset = set(outputs).difference(dibw)
    if badoutset:
        raise NonDifferentiable("Outputs %s not differentiable wrt any of %s" % (badoutset, badwrtset))

    var2gs = defaultdict(list)
    for (node, gnode) in utils.safezip(outputs, goutputs):
        var2gs[node] = [gnode]
    active = dio.intersection(dibw)

    for node in reversed(nodelist):
        if node not in active:
            continue
        if len(var2gs[node]) > 1 and node.is_tensor():
            var2gs[node] = [cgt.add_multi(var2gs[node])]
        gnode = var2gs[node][0]
        if node.is_input():
            continue
        if isinstance(node.op, TupleIndex):
            # gradient of a tuple-typed parent is kept as one list with a slot per component
            par = node.parents[0]
            if par not in var2gs:
                var2gs[par] = [[None for _ in par.typ]]
            var2gs[par][0][node.op.idx] = gnode
        else:
            gpars = node.op.pullback(node.parents, node, gnode)
            diffs = node.get_diff()
            for (par, gpar, d) in utils.safezip3(node.parents, gpars, diffs):
                assert (gpar is not None) == d
                if d:
                    var2gs[par].append(gpar)
    return [var2gs[node][0] for node in wrt]


def infer_shape(arr):
    """Tuple of int / None: the statically known shape of `arr`."""
    return tuple(x.op.value.item() if isinstance(x.op, Constant) else None for x in simplify(cgt.shape(arr)))


def grad(cost, wrt):
    """Gradient of scalar `cost` with respect to a variable or list of input variables."""
    assert cost.ndim == 0
    single_wrt = not isinstance(wrt, (list, tuple))
    wrtl = [wrt] if single_wrt else list(wrt)
    assert all(x.is_input() for x in wrtl), "Can only differentiate wrt Input nodes."
    gout = _singleton_ones(cost.dtype, 0)
    retval = pullback([cost], [gout], wrtl)
    return retval[0] if single_wrt else retval


# ================================================================
# Compile info and callables (cgt/core.py:734-856)
# ================================================================

class NativeCompileInfo(object):
    """What the compiler needs to turn an Op into a native callable.

    func_code: C++ source of the function, using the template names $function, $closure, $setup,
        $teardown; or None when `prebuilt` names an exported symbol of libcgt_b200.so with the
        byref / byval callable signature.
    closure_triples: list of (field name, ctypes type, value) laid out as the callable's closure struct.
    includes, link_flags, setup, teardown, gpu_deref_mask, store_objects, extra_srcs: as in the reference.
    """

    def __init__(self, func_code, closure_triples=None, includes=(), link_flags="", setup=False, teardown=False,
                 gpu_deref_mask=None, store_objects=(), extra_srcs=(), prebuilt=None, flags=0):
        self.op_str = None
        self.return_type = None
        self.n_in = None
        self.func_code = func_code
        self.closure_triples = closure_triples
        self.includes = list(includes)
        self.link_flags = link_flags
        self.setup = setup
        self.teardown = teardown
        self.gpu_deref_mask = gpu_deref_mask
        self.store_objects = store_objects
        self.extra_srcs = extra_srcs
        self.prebuilt = prebuilt
        self.flags = flags

    def involves_gpu(self):
        return self.gpu_deref_mask is not None


SrcFile = namedtuple("SrcFile", ["lang", "code"])


class PyCallable(object):
    """Callable backed by a Python function on numpy arrays (constant folding, user Ops)."""

    def __init__(self, op, n_in, func):
        self.op_str = str(op)
        self.return_type = op.return_type
        self.n_in = n_in
        self.func = func
        self.kind = "py"

    def call(self, *args):
        return self.func(*args)


class NativeCallable(object):
    """Callable backed by a function pointer acting on cgtObjects (cgt/core.py:816-856)."""

    def __init__(self, n_in, return_type, op_str, fptr, cldata=None, store_objects=None, setup_fptr=None,
                 teardown_fptr=None, flags=0):
        self.n_in = n_in
        self.return_type = return_type
        self.op_str = op_str
        self.fptr = fptr
        self.cldata = cldata
        self.store_objects = store_objects
        self.teardown_fptr = teardown_fptr
        self.flags = flags
        self.kind = "native"
        if setup_fptr is not None:
            setup_fptr()

    def __del__(self):
        if getattr(self, "teardown_fptr", None) is not None:
            self.teardown_fptr()

    def call(self, inputs, output=None):
        from . import runtime
        if self.return_type == "byref":
            runtime.apply_byref(self.fptr, self.cldata, inputs, output)
        else:
            raise Todo("direct call of a byval native callable")


# ================================================================
# Ops: constants
# ================================================================

class Constant(Op):
    available_impls = ("python", "native_cpu", "native_gpu")

    def __init__(self, value):
        self.value = value

    def get_value(self):
        return self.value


class ConstantTensor(Constant):
    """Constant array (cgt/core.py:874-942). byref: the value is copied into the output, which the
    placement pass may put on either device."""
    return_type = "byref"

    def __init__(self, value):
        Constant.__init__(self, as_valid_array(value))
        self._hash = None

    def get_expr(self, parent_exprs):
        return self._value_str()

    def __str__(self):
        return "Const{%s}" % self._value_str()

    __repr__ = __str__

    def _value_str(self):
        ndim = self.value.ndim
        return "%g" % self.value if ndim == 0 else "%s%g...%s" % ("[" * ndim, self.value.flat[0], "]" * ndim)

    def get_py_func(self, input_types):
        def f(_, write):
            np.copyto(write, self.value)
        return f

    def pullback(self, _inps, _out, _gout):
        return []

    def shp_apply(self, _inputs):
        return [cgt.constant(x) for x in self.value.shape]

    def typ_apply(self, input_types):
        assert len(input_types) == 0
        return _ndarray_type(self.value)

    def get_hash(self):
        if self._hash is None:
            self._hash = pickle.dumps((self.value.dtype.str, self.value.shape, self.value.tobytes()), -1)
        return self._hash

    def get_closure(self):
        shapeptr = ctypes.cast(self.value.ctypes.shape, ctypes.c_void_p).value
        return [("ndim", ctypes.c_int, self.value.ndim), ("shape", ctypes.c_void_p, shapeptr),
                ("dtype", ctypes.c_byte, self.value.dtype.num), ("data", ctypes.c_void_p, self.value.ctypes.data)]

    def get_native_compile_info(self, input_types, devtype):
        return NativeCompileInfo(None, prebuilt="cgtb_op_constant", closure_triples=self.get_closure(),
                                 store_objects=(self.value,))


class Fill(Op):
    """(shape...) -> array filled with a constant (cgt/core.py:966-1007)."""
    available_impls = ("python", "native_cpu", "native_gpu")

    def __init__(self, value):
        self.value = as_valid_array(value)
        assert self.value.ndim == 0 and self.value.dtype != "O"
        self.dtype = self.value.dtype
        self.tag = -1  # keeps CSE from merging the zero buffers that in-place increments write into

    def get_hash(self):
        return pickle.dumps((self.value.dtype.str, self.value.tobytes(), self.tag), -1)

    def get_diff(self, num_inputs):
        return [False] * num_inputs

    def __str__(self):
        return "Fill{%g}" % self.value

    __repr__ = __str__

    def get_py_func(self, input_types):
        def f(reads, write):
            write[...] = self.value
        return f

    def pullback(self, inputs, output, goutput):
        raise NonDifferentiable

    def shp_apply(self, inputs):
        return list(inputs)

    def typ_apply(self, input_types):
        assert all(map(_isintscalar, input_types)), "Fill Op should have integer scalars as arguments"
        return TensorType(self.dtype, len(input_types))

    def host_inputs(self, n):
        return tuple(range(n))

    def get_native_compile_info(self, _input_types, devtype):
        isint = self.value.dtype.kind == "i"
        return NativeCompileInfo(None, prebuilt="cgtb_op_fill", closure_triples=[
            ("fvalue", ctypes.c_double, float(self.value.item())),
            ("ivalue", ctypes.c_long, int(self.value.item()) if isint else 0)])


def _isintscalar(typ):
    return typ.dtype[0] == "i" and typ.ndim == 0


def _list_is_valid_sli(input_types):
    return len(input_types) == 3 and all(map(_isintscalar, input_types))


class Arange(Op):
    """(start, stop, step) -> 1-D int64 array produced on the host (cgt/core.py:1015-1048)."""
    available_impls = ("python", "native_cpu")
    return_type = "byval"

    def __init__(self, dtype="i8"):
        self.dtype = dtype

    def get_diff(self, num_inputs):
        return [False] * num_inputs

    def get_py_func(self, input_types):
        def f(reads):
            start, stop, step = [int(r) for r in reads]
            return np.arange(start, stop, step, self.dtype)
        return f

    def pullback(self, inputs, output, goutput):
        raise NonDifferentiable

    def shp_apply(self, inputs):
        start, stop, step = inputs
        return [(stop - start) // step]

    def typ_apply(self, input_types):
        assert _list_is_valid_sli(input_types)
        return TensorType(self.dtype, 1)

    def get_native_compile_info(self, input_types, devtype):
        return NativeCompileInfo(None, prebuilt="cgtb_op_arange")


# ================================================================
# Ops: elementwise
# ================================================================

def _no_grad():
    raise NonDifferentiable()


def _c_float_type(*dtypes):
    """The type C arithmetic is carried out in for operands of these numpy dtypes."""
    if any(d == np.float64 for d in dtypes):
        return np.float64
    if any(d == np.float32 for d in dtypes):
        return np.float32
    return None


def _py_unary(cname):
    """numpy evaluation of a unary C expression with C's promotions (compile-time folding only)."""
    def f(x, out=None):
        x = np.asarray(x)
        ft = _c_float_type(x.dtype)
        xm = x if ft is not None else x.astype(np.float64)  # integer arguments promote to double in <cmath>
        with np.errstate(all="ignore"):
            if cname == "abs": r = np.fabs(xm)
            elif cname == "ceil": r = np.ceil(xm)
            elif cname == "cos": r = np.cos(xm)
            elif cname == "exp": r = np.exp(xm)
            elif cname == "iceil": r = np.ceil(xm).astype(np.int32)
            elif cname == "ifloor": r = np.floor(xm).astype(np.int32)
            elif cname == "log": r = np.log(xm)
            elif cname == "neg": r = -x
            elif cname == "sign": r = 2 * (x > 0).astype(np.int32) - 1
            elif cname == "sin": r = np.sin(xm)
            elif cname == "square": r = x * x
            elif cname == "sqrt": r = np.sqrt(xm)
            elif cname == "tanh": r = np.tanh(xm)
            elif cname == "sigmoid": r = 1.0 / (1.0 + np.exp(-xm).astype(np.float64))
            elif cname == "softplus":
                r = np.where(xm > 0, xm + np.log(np.exp(-xm) + 1), np.log(1 + np.exp(xm)))
            elif cname == "cast": r = x
            else: raise MethodNotDefined(cname)
        if out is None:
            return r
        out[...] = r.astype(out.dtype)
    return f


UnaryInfo = namedtuple("UnaryInfo", ("short", "pyfunc", "diff", "typeinfo", "gradexpr", "cexpr"))

# name -> info; cexpr is the C expression of the reference table (cgt/core.py:1118-1134), kept for
# documentation and for Ops compiled from code strings; built-in names run prebuilt kernels.
UNARY_INFO = {
    "abs": UnaryInfo("abs", _py_unary("abs"), True, "s", lambda x, y, gy: gy * cgt.sign(x), "fabs(x)"),
    "ceil": UnaryInfo("ceil", _py_unary("ceil"), False, "i", lambda x, y, gy: _no_grad(), "ceil(x)"),
    "cos": UnaryInfo("cos", _py_unary("cos"), True, "f", lambda x, y, gy: -gy * cgt.sin(x), "cos(x)"),
    "exp": UnaryInfo("exp", _py_unary("exp"), True, "f", lambda x, y, gy: gy * cgt.exp(x), "exp(x)"),
    "iceil": UnaryInfo("iceil", _py_unary("iceil"), False, "i", lambda x, y, gy: _no_grad(), "(int)ceil(x)"),
    "ifloor": UnaryInfo("ifloor", _py_unary("ifloor"), False, "i", lambda x, y, gy: _no_grad(), "(int)floor(x)"),
    "log": UnaryInfo("log", _py_unary("log"), True, "f", lambda x, y, gy: gy / x, "log(x)"),
    "neg": UnaryInfo("negative", _py_unary("neg"), True, "s", lambda x, y, gy: -gy, "(-x)"),
    "sign": UnaryInfo("sign", _py_unary("sign"), False, "s", lambda x, y, gy: _no_grad(), "2*(x>0)-1"),
    "sin": UnaryInfo("sin", _py_unary("sin"), True, "f", lambda x, y, gy: gy * cgt.cos(x), "sin(x)"),
    "square": UnaryInfo("square", _py_unary("square"), True, "s", lambda x, y, gy: 2.0 * gy * x, "x*x"),
    "sqrt": UnaryInfo("sqrt", _py_unary("sqrt"), True, "f", lambda x, y, gy: gy / (2.0 * y), "sqrt(x)"),
    "tanh": UnaryInfo("tanh", _py_unary("tanh"), True, "f", lambda x, y, gy: gy * (1 - cgt.square(y)), "tanh(x)"),
    "sigmoid": UnaryInfo("sigmoid", _py_unary("sigmoid"), True, "f", lambda x, y, gy: gy * y * (1 - y),
                         "1.0/(1.0+exp(-x))"),
}

UNARY_OPCODE = {"abs": 0, "ceil": 1, "cos": 2, "exp": 3, "iceil": 4, "ifloor": 5, "log": 6, "neg": 7, "sign": 8,
                "sin": 9, "square": 10, "sqrt": 11, "tanh": 12, "sigmoid": 13, "softplus": 14}
CAST_OPCODE = 15


def _py_binary(opname):
    def f(x, y, out=None):
        x, y = np.asarray(x), np.asarray(y)
        ft = _c_float_type(x.dtype, y.dtype)
        if opname == "/":
            ft = np.float64
        elif opname == "**" and not (x.dtype == np.float32 and y.dtype == np.float32):
            ft = np.float64
        if ft is not None:
            xa, ya = x.astype(ft), y.astype(ft)
        else:  # integer operands: C promotes anything narrower than int to int
            it = np.promote_types(np.promote_types(x.dtype, y.dtype), np.int32)
            xa, ya = x.astype(it), y.astype(it)
        with np.errstate(all="ignore"):
            r = {"*": np.multiply, "+": np.add, "-": np.subtract, "/": np.divide, "<": np.less, ">": np.greater,
                 "<=": np.less_equal, ">=": np.greater_equal, "**": np.power, "==": np.equal,
                 "!=": np.not_equal}[opname](xa, ya)
        if out is None:
            return r
        out[...] = r.astype(out.dtype)
    return f


BinaryInfo = namedtuple("BinaryInfo", ("short", "pyfunc", "commutes", "diff", "typeinfo", "gradexpr", "cexpr"))

BINARY_INFO = {
    "*": BinaryInfo("multiply", _py_binary("*"), True, (True, True), "p", lambda x, y, z, gz: [y * gz, x * gz], "x*y"),
    "+": BinaryInfo("add", _py_binary("+"), True, (True, True), "p", lambda x, y, z, gz: [gz, gz], "x+y"),
    "-": BinaryInfo("subtract", _py_binary("-"), False, (True, True), "p", lambda x, y, z, gz: [gz, -gz], "x-y"),
    "/": BinaryInfo("divide", _py_binary("/"), False, (True, True), "f", lambda x, y, z, gz: [gz / y, -gz * z / y],
                    "(x+0.0)/y"),
    "<": BinaryInfo("less", _py_binary("<"), False, (False, False), "i1", lambda x, y, z, gz: _no_grad(), "x<y"),
    ">": BinaryInfo("greater", _py_binary(">"), False, (False, False), "i1", lambda x, y, z, gz: _no_grad(), "x>y"),
    "<=": BinaryInfo("less_equal", _py_binary("<="), False, (False, False), "i1", lambda x, y, z, gz: _no_grad(), "x<=y"),
    ">=": BinaryInfo("greater_equal", _py_binary(">="), False, (False, False), "i1", lambda x, y, z, gz: _no_grad(),
                     "x>=y"),
    "**": BinaryInfo("power", _py_binary("**"), False, (True, True), "p",
                     lambda x, y, z, gz: [gz * y * cgt.power(x, y - 1), gz * z * cgt.log(x)], "pow(x,y)"),
    "==": BinaryInfo("equal", _py_binary("=="), True, (False, False), "i1", lambda x, y, z, gz: _no_grad(), "x==y"),
    "!=": BinaryInfo("not_equal", _py_binary("!="), True, (False, False), "i1", lambda x, y, z, gz: _no_grad(), "x!=y"),
}

BINARY_OPCODE = {"*": 0, "+": 1, "-": 2, "/": 3, "<": 4, ">": 5, "<=": 6, ">=": 7, "**": 8, "==": 9, "!=": 10}

np2c = {"i1": "int8_t", "i2": "int16_t", "i4": "int32_t", "i8": "int64_t", "f4": "float", "f8": "double"}


class ElwiseUnary(Op):
    """Elementwise unary operation (cgt/core.py:1160-1241).

    Built-in names (UNARY_OPCODE), softplus and casts run the prebuilt vectorised kernel; an
    ``info`` with any other C expression is compiled at run time into a kernel of the same shape.
    """
    available_impls = ("python", "native_cpu", "native_gpu")

    def __init__(self, opname, info=None):
        self.opname = opname
        self.info = UNARY_INFO[opname] if info is None else info

    def get_diff(self, _):
        return [self.info.diff]

    def __str__(self):
        return self.info.short

    __repr__ = __str__

    def get_hash(self):
        return ("ElwiseUnary:" + self.opname).encode()

    def pullback(self, inputs, y, gy):
        return [self.info.gradexpr(inputs[0], y, gy)]

    def shp_apply(self, inputs):
        return cgt.shape(inputs[0])

    def typ_apply(self, input_types):
        typeinfo = self.info.typeinfo
        intype = input_types[0].dtype
        if typeinfo == "s":
            out_type = intype
        elif typeinfo == "i":
            out_type = _type_to_int(intype)
        elif typeinfo == "f":
            out_type = cgt.floatX
        else:
            assert typeinfo in (cgt.floatX, "f4", "f8", "i1", "i2", "i4", "i8")
            out_type = typeinfo
        return TensorType(out_type, input_types[0].ndim)

    def get_py_func(self, _):
        def f(reads, write):
            self.info.pyfunc(reads[0], out=write)
        return f

    def opcode(self):
        if self.opname in UNARY_OPCODE:
            return UNARY_OPCODE[self.opname]
        if self.opname.startswith("cast_to_"):
            return CAST_OPCODE
        return None

    def get_native_compile_info(self, input_types, devtype):
        code = self.opcode()
        if code is not None:
            return NativeCompileInfo(None, prebuilt="cgtb_op_elwise_unary", closure_triples=[("op", ctypes.c_int, code)])
        from . import codegen
        return codegen.unary_from_cexpr(self, input_types, devtype)


class ElwiseBinary(Op):
    """Elementwise binary operation (cgt/core.py:1243-1378). Shapes must match exactly or one side
    is a 0-d scalar (``scalar_mask``); there is no implicit broadcasting."""
    available_impls = ("python", "native_cpu", "native_gpu")

    def __init__(self, opname, scalar_mask, info=None):
        assert opname in BINARY_INFO
        self.opname = opname
        self.info = BINARY_INFO[opname] if info is None else info
        self.scalar_mask = tuple(scalar_mask)

    def get_diff(self, _):
        return BINARY_INFO[self.opname].diff

    def get_hash(self):
        return ("ElwiseBinary:" + self.opname).encode()

    def get_expr(self, parent_exprs):
        return "(%s %s %s)" % (parent_exprs[0], self.opname, parent_exprs[1])

    def __str__(self):
        return BINARY_INFO[self.opname].short

    __repr__ = __str__

    def get_replacement(self, parents, analysis):
        l, r = parents
        node2sv = analysis["node2sv"]
        out = None
        # a Fill on one side is a scalar in disguise
        if isinstance(l.op, Fill) and not self.scalar_mask[1]:
            out = Result(ElwiseBinary(self.opname, (True, False), self.info), [cgt.constant(l.op.value), r])
        elif isinstance(r.op, Fill) and not self.scalar_mask[0]:
            out = Result(ElwiseBinary(self.opname, (False, True), self.info), [l, cgt.constant(r.op.value)])
        elif l in node2sv and r in node2sv:
            out = self.info.pyfunc(node2sv[l], node2sv[r])
        elif self.opname == "*":
            if l in node2sv and node2sv[l] == 1: out = r
            if l in node2sv and node2sv[l] == -1: out = -r
            if r in node2sv and node2sv[r] == 1: out = l
            if r in node2sv and node2sv[r] == -1: out = -l
        elif self.opname == "+":
            if l in node2sv and node2sv[l] == 0: out = r
            if r in node2sv and node2sv[r] == 0: out = l
        elif self.opname == "**":
            if r in node2sv and node2sv[r] == 1: out = l
        if out is not None:
            outtyp = self.typ_apply([p.typ for p in parents])
            out = cgt.cast(out, outtyp.dtype)
            if out.ndim == 0 and outtyp.ndim > 0:
                ind4shape = 1 if self.scalar_mask[0] else 0
                outshape = analysis["node2shape"][parents[ind4shape]]
                out = cgt.fill(out, outshape)
        return out

    def pullback(self, inputs, z, gz):
        x, y = inputs
        gin = BINARY_INFO[self.opname].gradexpr(x, y, z, gz)
        return [cgt.sum(gv) if (v.ndim == 0 and gv.ndim > 0) else gv for (v, gv) in utils.safezip([x, y], gin)]

    def shp_apply(self, inputs):
        ind4shape = 1 if self.scalar_mask[0] else 0
        return cgt.shape(inputs[ind4shape])

    def typ_apply(self, input_types):
        assert ((input_types[0].ndim == 0) == self.scalar_mask[0]) and ((input_types[1].ndim == 0) == self.scalar_mask[1])
        if self.scalar_mask == (False, False):
            assert input_types[0].ndim == input_types[1].ndim
        typeinfo = BINARY_INFO[self.opname].typeinfo
        if typeinfo == "p":
            out_dtype = _promote(input_types[0].dtype, input_types[1].dtype)
        elif typeinfo == "f":
            out_dtype = cgt.floatX
        else:
            out_dtype = typeinfo
        ind4shape = 1 if self.scalar_mask[0] else 0
        return TensorType(out_dtype, input_types[ind4shape].ndim)

    def get_py_func(self, input_types):
        def f(reads, write):
            x, y = reads
            if self.scalar_mask == (False, False) and np.shape(x) != np.shape(y):
                raise RuntimeError("mismatched shapes %s %s. Note that implicit broadcasting isn't allowed. "
                                   "Use the broadcast(...) function" % (np.shape(x), np.shape(y)))
            self.info.pyfunc(x, y, out=write)
        return f

    def get_native_compile_info(self, input_types, devtype):
        return NativeCompileInfo(None, prebuilt="cgtb_op_elwise_binary", closure_triples=[
            ("op", ctypes.c_int, BINARY_OPCODE[self.opname]),
            ("scalar_x", ctypes.c_int, int(self.scalar_mask[0])),
            ("scalar_y", ctypes.c_int, int(self.scalar_mask[1]))])


class FusedElwise(Op):
    """A connected group of ElwiseUnary / ElwiseBinary nodes over one shape, evaluated by one kernel.

    Not part of the reference's Op set: the compiler forms these nodes after simplification and
    differentiation (compilation.fuse_elementwise), the reference launches one generated loop per Op
    (cgt/core.py:1160-1378). ``program`` is a list of (arity, opcode, a, b) over registers: registers
    0..n_in-1 are the inputs, register n_in+j is the result of operation j. ``in_kinds`` gives each
    input's form (0 f4 tensor, 1 i1 tensor, 2 f4 scalar, 3 i8 scalar, 4 f4 tensor broadcast along its
    singleton axes: the operand of a folded Repeat). ``out_regs`` / ``out_dtypes`` name the registers that
    leave the group. With several outputs the node is tuple-valued."""
    available_impls = ("native_gpu",)
    return_type = "byref"
    MAX_IN, MAX_OPS, MAX_OUT = 16, 32, 12

    def __init__(self, program, in_kinds, out_regs, out_dtypes, ndim, shape_input, descr="", views=None, static_shape=None):
        """views: {input index: (first column, row length of the input matrix)} for the inputs of kind 7, which are
        [R, row length] matrices whose columns [first, first + W) the chain reads (the index space is [R, W] then);
        static_shape: the result's extents when no input has the result's shape (shape_input None)."""
        assert 1 <= len(in_kinds) <= self.MAX_IN and 1 <= len(program) <= self.MAX_OPS and 1 <= len(out_regs) <= self.MAX_OUT
        self.program = [tuple(p) for p in program]
        self.in_kinds = list(in_kinds)
        self.out_regs = list(out_regs)
        self.out_dtypes = list(out_dtypes)
        self.ndim = ndim
        self.shape_input = shape_input
        self.descr = descr
        self.views = dict(views or {})
        self.static_shape = tuple(int(d) for d in static_shape) if static_shape is not None else None
        assert sorted(self.views) == [k for (k, kind) in enumerate(self.in_kinds) if kind == 7]
        assert not self.views or (self.static_shape is not None and len(self.static_shape) == 2)
        assert shape_input is not None or self.static_shape is not None

    def get_diff(self, num_inputs):
        return [False] * num_inputs

    def shp_apply(self, inputs):
        if self.shape_input is not None:
            shp = cgt.shape(inputs[self.shape_input])
        else:
            shp = [cgt.constant(np.array(d, "i8")) for d in self.static_shape]
        return shp if len(self.out_regs) == 1 else tuple(list(shp) for _ in self.out_regs)

    def typ_apply(self, input_types):
        typs = [TensorType(dt, self.ndim) for dt in self.out_dtypes]
        return typs[0] if len(typs) == 1 else TupleType(*typs)

    def get_native_compile_info(self, input_types, devtype):
        def arr(vals, n):
            vals = list(vals) + [0] * (n - len(vals))
            return (ctypes.c_int * n)(*vals)
        def larr(vals):
            vals = list(vals) + [0] * (self.MAX_IN - len(vals))
            return (ctypes.c_long * self.MAX_IN)(*vals)
        code = {"f4": 11, "i1": 1}
        return NativeCompileInfo(None, prebuilt="cgtb_op_fused_elwise", closure_triples=[
            ("n_in", ctypes.c_int, len(self.in_kinds)),
            ("n_ops", ctypes.c_int, len(self.program)),
            ("n_out", ctypes.c_int, len(self.out_regs)),
            ("in_kind", ctypes.c_int * self.MAX_IN, arr(self.in_kinds, self.MAX_IN)),
            ("op_arity", ctypes.c_int * self.MAX_OPS, arr([p[0] for p in self.program], self.MAX_OPS)),
            ("op_code", ctypes.c_int * self.MAX_OPS, arr([p[1] for p in self.program], self.MAX_OPS)),
            ("op_a", ctypes.c_int * self.MAX_OPS, arr([p[2] for p in self.program], self.MAX_OPS)),
            ("op_b", ctypes.c_int * self.MAX_OPS, arr([p[3] for p in self.program], self.MAX_OPS)),
            ("out_reg", ctypes.c_int * self.MAX_OUT, arr(self.out_regs, self.MAX_OUT)),
            ("out_dtype", ctypes.c_int * self.MAX_OUT, arr([code[d] for d in self.out_dtypes], self.MAX_OUT)),
            ("launcher", ctypes.c_void_p, self._launcher()),
            ("view_width", ctypes.c_long, self.static_shape[1] if self.views else 0),
            ("view_pitch", ctypes.c_long * self.MAX_IN, larr([self.views.get(k, (0, 0))[1] for k in range(len(self.in_kinds))])),
            ("view_off", ctypes.c_long * self.MAX_IN, larr([self.views.get(k, (0, 0))[0] for k in range(len(self.in_kinds))]))])

    def _launcher(self):
        from . import codegen
        return codegen.fused_launcher(self)

    def __repr__(self):
        return "FusedElwise{%s}" % self.descr


class MultiFusedElwise(Op):
    """k FusedElwise instructions with one and the same single-output program, issued as one launch.

    Not part of the reference's Op set and never a graph node: the compiler forms it on the instruction list
    (compilation.merge_parameter_updates) from the k update instructions of a training step, which are k tiny launches
    of the same chain (p - lr * g). Its callable reads the k operand lists back to back, then the result arrays of
    tensors 1..k-1; the instruction's own write location is tensor 0's result."""
    available_impls = ("native_gpu",)
    return_type = "byref"

    def __init__(self, fused, k):
        assert isinstance(fused, FusedElwise) and len(fused.out_regs) == 1 and k >= 2
        self.fused = fused
        self.k = int(k)

    def get_native_compile_info(self, input_types, devtype):
        triples = list(self.fused.get_native_compile_info(input_types, devtype).closure_triples)
        triples = [t for t in triples if t[0] not in ("launcher", "view_width", "view_pitch", "view_off")]
        triples += [("launcher", ctypes.c_void_p, None), ("view_width", ctypes.c_long, 0), ("k", ctypes.c_int, self.k)]
        return NativeCompileInfo(None, prebuilt="cgtb_op_multi_fused_elwise", closure_triples=triples)

    def __repr__(self):
        return "MultiFusedElwise{%d x %s}" % (self.k, self.fused.descr)


class ScatterCols(Op):
    """(y_0, ..., y_{k-1}) -> [R, C] matrix of zeros with y_j ([R, width_j]) in columns [offset_j, offset_j + width_j).

    Not part of the reference's Op set: compilation.fuse_slice_sums forms it from a sum of IncSli(zeros, ...) over
    disjoint column ranges, which is how the gradient of several column slices of one matrix arrives after
    differentiation (GetSli.pullback, cgt/core.py:1786-1790): k zero fills, k slice increments and k-1 additions
    become one launch with the same values."""
    available_impls = ("native_gpu",)
    return_type = "byref"

    def __init__(self, offsets, widths, C):
        assert 1 <= len(offsets) <= 8 and len(offsets) == len(widths)
        self.offsets = [int(o) for o in offsets]
        self.widths = [int(w) for w in widths]
        self.C = int(C)

    def get_diff(self, num_inputs):
        return [False] * num_inputs

    def shp_apply(self, inputs):
        return [cgt.size(inputs[0], 0), cgt.constant(np.array(self.C, "i8"))]

    def typ_apply(self, input_types):
        return TensorType("f4", 2)

    def get_native_compile_info(self, input_types, devtype):
        def arr(vals):
            vals = list(vals) + [0] * (8 - len(vals))
            return (ctypes.c_long * 8)(*vals)
        return NativeCompileInfo(None, prebuilt="cgtb_op_scatter_cols", closure_triples=[
            ("k", ctypes.c_int, len(self.offsets)), ("C", ctypes.c_long, self.C),
            ("off", ctypes.c_long * 8, arr(self.offsets)), ("width", ctypes.c_long * 8, arr(self.widths))])

    def __repr__(self):
        return "ScatterCols{%s of %d}" % (",".join("%d:%d" % (o, o + w) for (o, w) in zip(self.offsets, self.widths)), self.C)


class FusedRows(Op):
    """Elementwise operations and sums along axis 1 over an [R, C] matrix (C <= 128) evaluated by one kernel, one warp per
    row: a softmax, its logarithm and its pullback are such chains, and as separate launches on a [batch, classes] matrix
    each costs far more in launch latency than in bytes.

    Not part of the reference's Op set: compilation.fuse_elementwise(rows=True) forms these nodes. ``program`` as in
    FusedElwise plus (3, 0, a, 0): the sum of register a over the row, and (4, 0, a, b): the sum of the elements of a
    where register b is not zero (MaskedRowSum). ``in_kinds``: 0 an [R, C] array, 5 an [R, 1]
    array, 6 a [1, C] array, 2 / 3 scalars, 8 an int64 [R] array of column numbers read as OneHotRows of it. ``out_cols[j]``: output j is [R, 1] rather than [R, C]. ``shape_input``: an
    input whose axis 0 gives R."""
    available_impls = ("native_gpu",)
    return_type = "byref"
    MAX_C = 128

    def __init__(self, program, in_kinds, out_regs, out_cols, C, shape_input, descr=""):
        F = FusedElwise
        assert 1 <= len(in_kinds) <= F.MAX_IN and 1 <= len(program) <= F.MAX_OPS and 1 <= len(out_regs) <= F.MAX_OUT
        self.program = [tuple(p) for p in program]
        self.in_kinds = list(in_kinds)
        self.out_regs = list(out_regs)
        self.out_cols = [int(bool(c)) for c in out_cols]
        self.C = int(C)
        self.shape_input = shape_input
        self.descr = descr

    def get_diff(self, num_inputs):
        return [False] * num_inputs

    def shp_apply(self, inputs):
        R = cgt.size(inputs[self.shape_input], 0)
        shps = [[R, cgt.constant(np.array(1 if col else self.C, "i8"))] for col in self.out_cols]
        return shps[0] if len(shps) == 1 else tuple(shps)

    def typ_apply(self, input_types):
        typs = [TensorType("f4", 2) for _ in self.out_regs]
        return typs[0] if len(typs) == 1 else TupleType(*typs)

    def get_native_compile_info(self, input_types, devtype):
        F = FusedElwise

        def arr(vals, n):
            vals = list(vals) + [0] * (n - len(vals))
            return (ctypes.c_int * n)(*vals)
        return NativeCompileInfo(None, prebuilt="cgtb_op_fused_rows", closure_triples=[
            ("n_in", ctypes.c_int, len(self.in_kinds)),
            ("n_ops", ctypes.c_int, len(self.program)),
            ("n_out", ctypes.c_int, len(self.out_regs)),
            ("in_kind", ctypes.c_int * F.MAX_IN, arr(self.in_kinds, F.MAX_IN)),
            ("op_arity", ctypes.c_int * F.MAX_OPS, arr([p[0] for p in self.program], F.MAX_OPS)),
            ("op_code", ctypes.c_int * F.MAX_OPS, arr([p[1] for p in self.program], F.MAX_OPS)),
            ("op_a", ctypes.c_int * F.MAX_OPS, arr([p[2] for p in self.program], F.MAX_OPS)),
            ("op_b", ctypes.c_int * F.MAX_OPS, arr([p[3] for p in self.program], F.MAX_OPS)),
            ("out_reg", ctypes.c_int * F.MAX_OUT, arr(self.out_regs, F.MAX_OUT)),
            ("out_col", ctypes.c_int * F.MAX_OUT, arr(self.out_cols, F.MAX_OUT)),
            ("launcher", ctypes.c_void_p, self._launcher()),
            ("C", ctypes.c_int, self.C)])

    def _launcher(self):
        from . import codegen
        return codegen.rows_launcher(self)

    def __repr__(self):
        return "FusedRows{%s}" % self.descr


def elwise_binary(opname, x, y):
    (x, y) = map(as_node, (x, y))
    scalar_mask = ((x.ndim == 0), (y.ndim == 0))
    op = ElwiseBinary(opname, scalar_mask)
    if scalar_mask == (False, False):
        assert x.ndim == y.ndim
    return Result(op, [x, y])


# ================================================================
# Ops: shape manipulation
# ================================================================

class Size(Op):
    """One element of a tensor's shape, as a host int64 scalar (cgt/core.py:1391-1430)."""
    return_type = "byval"
    available_impls = ("python", "native_cpu", "native_gpu")

    def __init__(self, axis):
        self.axis = axis

    def get_diff(self, _):
        return [False]

    def __str__(self):
        return "Size{%i}" % self.axis

    __repr__ = __str__

    def get_py_func(self, input_types):
        def f(reads):
            return np.array(reads[0].shape[self.axis], "i8")
        return f

    def pullback(self, inputs, output, goutput):
        raise NonDifferentiable

    def shp_apply(self, _inputs):
        return []

    def typ_apply(self, _):
        return TensorType("i8", 0)

    def host_inputs(self, n):
        return ()

    def get_replacement(self, inputs, _analysis):
        x = inputs[0]
        if x.is_input():
            fixed_shape = x.get_fixed_shape()
            if fixed_shape[self.axis] is not None:
                return cgt.constant(np.array(fixed_shape[self.axis], "i8"))

    def get_native_compile_info(self, input_types, devtype):
        return NativeCompileInfo(None, prebuilt="cgtb_op_size", closure_triples=[("ax", ctypes.c_int, self.axis)])


class Reshape(Op):
    """(x, shape...) -> view of x with a new shape; no data movement (cgt/core.py:1432-1465)."""
    available_impls = ("python", "native_cpu", "native_gpu")
    return_type = "byval"

    def get_diff(self, num_inputs):
        return [True] + [False] * (num_inputs - 1)

    def get_py_func(self, input_types):
        def f(reads):
            out = np.asarray(reads[0]).reshape([int(r) for r in reads[1:]])
            return np.ascontiguousarray(out) if out.ndim else out
        return f

    def pullback(self, inputs, _out, gout):
        return [cgt.reshape(gout, cgt.shape(inputs[0]))] + [None] * (len(inputs) - 1)

    def shp_apply(self, inputs):
        return list(inputs[1:])

    def typ_apply(self, input_types):
        return TensorType(input_types[0].dtype, len(input_types) - 1)

    def host_inputs(self, n):
        return tuple(range(1, n))

    def get_native_compile_info(self, input_types, devtype):
        return NativeCompileInfo(None, prebuilt="cgtb_op_reshape",
                                 closure_triples=[("ndim", ctypes.c_int, len(input_types) - 1)])


class OneHotRows(Op):
    """(idx int64 [R]) -> float32 [R, C] with a one in column idx[r] of row r, zeros elsewhere.

    Not part of the reference's Op set. compilation.fuse_flat_index_rows writes x[arange(R), idx] on an [R, C] matrix
    (GetFlatIndices on arange(R)*C + idx, cgt/core.py:1781-1812) as Sum{1}(x * OneHotRows(idx)) and its gradient
    (IncFlatIndices on zeros, cgt/core.py:1814-1860) as OneHotRows(idx) * g, so that both join the row chain around them
    (a softmax cross-entropy and its pullback become one FusedRows launch, which reads idx itself: input kind 8); a
    OneHotRows node left outside such a chain is written by its own kernel."""
    available_impls = ("python", "native_gpu")
    return_type = "byref"

    def __init__(self, C):
        self.C = int(C)

    def get_diff(self, num_inputs):
        return [False] * num_inputs

    def get_py_func(self, input_types):
        def f(reads, write):
            idx = np.asarray(reads[0]).astype("i8").reshape(-1)
            write[...] = (np.arange(self.C, dtype="i8")[None, :] == idx[:, None]).astype("f4")
        return f

    def shp_apply(self, inputs):
        return [cgt.size(inputs[0], 0), cgt.constant(np.array(self.C, "i8"))]

    def typ_apply(self, input_types):
        return TensorType("f4", 2)

    def get_native_compile_info(self, input_types, devtype):
        return NativeCompileInfo(None, prebuilt="cgtb_op_onehot_rows", closure_triples=[("C", ctypes.c_long, self.C)])

    def __repr__(self):
        return "OneHotRows{%d}" % self.C


class MaskedRowSum(Op):
    """(x f4 [R, C], m f4 [R, C]) -> [R, 1]: the sum of each row's elements of x where m is not zero. With
    m = OneHotRows(idx) it is x[r, idx[r]] itself: the element is selected, not multiplied by one and added to zero
    products, so an infinite element elsewhere in the row (a log-probability of -inf) stays out of the result as it
    does with the reference's GetFlatIndices (cgt/core.py:1781-1812).

    Not part of the reference's Op set: compilation.fuse_flat_index_rows forms it; in a FusedRows program it is the
    entry (4, 0, a, b)."""
    available_impls = ("python", "native_gpu")
    return_type = "byref"

    def get_diff(self, num_inputs):
        return [False] * num_inputs

    def get_py_func(self, input_types):
        def f(reads, write):
            (x, m) = (np.asarray(reads[0]), np.asarray(reads[1]))
            write[...] = np.where(m != 0, x, np.float32(0)).sum(axis=1, keepdims=True, dtype="f4")
        return f

    def shp_apply(self, inputs):
        return [cgt.size(inputs[0], 0), cgt.constant(np.array(1, "i8"))]

    def typ_apply(self, input_types):
        return TensorType("f4", 2)

    def get_native_compile_info(self, input_types, devtype):
        return NativeCompileInfo(None, prebuilt="cgtb_op_masked_row_sum", closure_triples=[])

    def __repr__(self):
        return "MaskedRowSum"


class LeadingSlice(Op):
    """(x, start, stop) -> view of x[start:stop] along axis 0; no data movement: the rows of a C-contiguous array are
    contiguous, so the slice is the same memory at an offset. The compiler (compilation.view_leading_slices) puts it in
    place of GetSli{0} with step 1 (cgt/core.py:1767-1812), which copies: x[t] of a [T, batch, features] sequence is
    taken once per time step of an unrolled recurrent network. The view retains its source."""
    available_impls = ("python", "native_cpu", "native_gpu")
    return_type = "byval"

    def get_diff(self, num_inputs):
        return [False] * num_inputs

    def get_py_func(self, input_types):
        def f(reads):
            return np.ascontiguousarray(np.asarray(reads[0])[int(reads[1]):int(reads[2])])
        return f

    def shp_apply(self, inputs):
        s = cgt.shape(inputs[0])
        s[0] = inputs[2] - inputs[1]
        return s

    def typ_apply(self, input_types):
        return input_types[0]

    def host_inputs(self, n):
        return (1, 2)

    def get_native_compile_info(self, input_types, devtype):
        return NativeCompileInfo(None, prebuilt="cgtb_op_leading_slice", closure_triples=[])

    def __repr__(self):
        return "LeadingSlice"


class Concatenate(Op):
    """np.concatenate along one axis (cgt/core.py:1467-1509)."""
    available_impls = ("python", "native_cpu", "native_gpu")

    def __init__(self, axis):
        self.axis = axis

    def get_diff(self, num_inputs):
        return [True] * num_inputs

    def get_py_func(self, input_types):
        def f(reads, write):
            write[...] = np.concatenate(reads, axis=self.axis)
        return f

    def pullback(self, inputs, _output, gout):
        start = 0
        out = []
        for x in inputs:
            end = start + cgt.size(x, self.axis)
            out.append(Result(GetSli(self.axis), [gout, start, end, 1]))
            start = end
        return out

    def shp_apply(self, inputs):
        out = cgt.shape(inputs[0])
        out[self.axis] = cgt.add_multi([cgt.size(x, self.axis) for x in inputs])
        return out

    def typ_apply(self, input_types):
        return TensorType(_promote_multi([x.dtype for x in input_types]), input_types[0].ndim)

    def get_native_compile_info(self, input_types, devtype):
        assert len(set(t.dtype for t in input_types)) == 1, "Concatenate inputs must share a dtype"
        return NativeCompileInfo(None, prebuilt="cgtb_op_concatenate", closure_triples=[
            ("axis", ctypes.c_int, self.axis), ("n_in", ctypes.c_int, len(input_types))])


def _axes_mask(axes):
    m = 0
    for a in axes:
        m |= 1 << int(a)
    return m


class Repeat(Op):
    """(x, reps...) -> x repeated along singleton `axes`; how broadcast() materialises operands
    (cgt/core.py:1511-1557)."""
    available_impls = ("python", "native_cpu", "native_gpu")

    def __init__(self, axes):
        self.axes = list(axes)

    def get_diff(self, num_inputs):
        return [True] + [False] * (num_inputs - 1)

    def get_py_func(self, input_types):
        def f(reads, write):
            arr = np.asarray(reads[0])
            assert all(arr.shape[i] == 1 for i in self.axes)
            for (ax, numrep) in utils.safezip(self.axes, reads[1:]):
                arr = np.repeat(arr, int(numrep), ax)
            np.copyto(write, arr)
        return f

    def get_replacement(self, parents, analysis):
        if parents[0] in analysis["node2sv"]:
            value = analysis["node2sv"][parents[0]]
            shp = self.shp_apply(parents)
            return Result(Fill(value), shp)

    def pullback(self, inputs, output, goutput):
        return [cgt.sum(goutput, self.axes, keepdims=True)] + [None] * (len(inputs) - 1)

    def shp_apply(self, inputs):
        out = cgt.shape(inputs[0])
        for (ax, rep) in utils.safezip(self.axes, inputs[1:]):
            out[ax] = rep
        return out

    def typ_apply(self, input_types):
        assert all(x.dtype == "i8" for x in input_types[1:])
        return input_types[0]

    def host_inputs(self, n):
        return tuple(range(1, n))

    def get_native_compile_info(self, input_types, devtype):
        return NativeCompileInfo(None, prebuilt="cgtb_op_repeat",
                                 closure_triples=[("axes_mask", ctypes.c_int, _axes_mask(self.axes))])


class Transpose(Op):
    """Physical axis permutation (cgt/core.py:1559-1594)."""
    available_impls = ("python", "native_cpu", "native_gpu")

    def __init__(self, axes):
        self.axes = [int(a) for a in axes]

    def get_diff(self, _):
        return [True]

    def get_py_func(self, input_types):
        def f(reads, write):
            np.copyto(write, np.asarray(reads[0]).transpose(self.axes))
        return f

    def pullback(self, inputs, output, goutput):
        return [cgt.transpose(goutput, utils.invert_perm(self.axes))]

    def shp_apply(self, inputs):
        inshape = cgt.shape(inputs[0])
        return [inshape[ax] for ax in self.axes]

    def typ_apply(self, input_types):
        return input_types[0]

    def __str__(self):
        return "Transpose{%s}" % ",".join(map(str, self.axes))

    __repr__ = __str__

    def get_native_compile_info(self, input_types, devtype):
        perm = 0
        for (i, a) in enumerate(self.axes):
            perm |= a << (4 * i)
        return NativeCompileInfo(None, prebuilt="cgtb_op_transpose", closure_triples=[("perm", ctypes.c_long, perm)])


class Transport(Op):
    """Copy between devices, inserted by the compiler on every cross-device edge (cgt/core.py:1596-1612)."""
    available_impls = ("native_cpu", "native_gpu")

    def __init__(self, dev):
        self.dev = dev

    def get_hash(self):
        return ("Transport%r" % (self.dev,)).encode()

    def typ_apply(self, input_types):
        return input_types[0]

    def shp_apply(self, inputs):
        return cgt.shape(inputs[0])

    def get_native_compile_info(self, _inputs, _devtype):
        from . import runtime
        return NativeCompileInfo(None, prebuilt="cgtb_op_transport", flags=runtime.INSTR_TRANSPORT)


# ================================================================
# Ops: reductions
# ================================================================

class Sum(Op):
    """Sum over `axes`, keepdims (cgt/core.py:1687-1709)."""
    available_impls = ("python", "native_cpu", "native_gpu")
    kind = 0

    def __init__(self, axes):
        self.axes = tuple(int(a) for a in axes)

    def get_diff(self, _):
        return [True]

    def __str__(self):
        return "Sum{%s}" % (",".join(map(str, self.axes)))

    __repr__ = __str__

    def get_py_func(self, input_types):
        def f(reads, write):
            np.asarray(reads[0]).sum(axis=self.axes or None, out=write, keepdims=True)
        return f

    def pullback(self, inputs, output, goutput):
        return [Result(Repeat(self.axes), [goutput] + [cgt.size(inputs[0], ax) for ax in self.axes])]

    def shp_apply(self, inputs):
        x = inputs[0]
        s = cgt.shape(x)
        return [(cgt.constant(np.array(1, "i8")) if i in self.axes else s[i]) for i in range(x.ndim)]

    def typ_apply(self, input_types):
        return input_types[0]

    def get_native_compile_info(self, input_types, devtype):
        return NativeCompileInfo(None, prebuilt="cgtb_op_reduce", closure_triples=[
            ("kind", ctypes.c_int, self.kind), ("axes_mask", ctypes.c_int, _axes_mask(self.axes))])


class Max(Op):
    """Max over `axes`, keepdims (cgt/core.py:1711-1738)."""
    available_impls = ("python", "native_cpu", "native_gpu")
    kind = 1

    def __init__(self, axes):
        self.axes = tuple(int(a) for a in axes)

    def get_diff(self, _):
        return [True]

    def __str__(self):
        return "Max{%s}" % (",".join(map(str, self.axes)))

    __repr__ = __str__

    def get_py_func(self, input_types):
        def f(reads, write):
            np.asarray(reads[0]).max(axis=self.axes or None, keepdims=True, out=write)
        return f

    def pullback(self, inputs, output, goutput):
        x = inputs[0]
        inputpat = "x" * x.ndim
        singpat = "".join(["1" if i in self.axes else "x" for i in range(x.ndim)])
        bcpat = singpat + "," + inputpat
        return [cgt.broadcast("*", goutput, cgt.broadcast("==", output, x, bcpat), bcpat)]

    def shp_apply(self, inputs):
        x = inputs[0]
        s = cgt.shape(x)
        return [(cgt.constant(np.array(1, "i8")) if i in self.axes else s[i]) for i in range(x.ndim)]

    def typ_apply(self, input_types):
        return input_types[0]

    def get_native_compile_info(self, input_types, devtype):
        return NativeCompileInfo(None, prebuilt="cgtb_op_reduce", closure_triples=[
            ("kind", ctypes.c_int, self.kind), ("axes_mask", ctypes.c_int, _axes_mask(self.axes))])


# ================================================================
# Ops: slicing and flat indexing
# ================================================================

class GetSli(Op):
    """(x, start, stop, step) -> x[..., start:stop:step, ...] along `axis` (cgt/core.py:1767-1812)."""
    available_impls = ("python", "native_cpu", "native_gpu")

    def __init__(self, axis):
        self.axis = axis

    def get_diff(self, _):
        return [True, False, False, False]

    def get_py_func(self, input_types):
        def f(reads, write):
            x, start, stop, step = reads
            start, stop, step = int(start), int(stop), int(step)
            if step < 0 and stop == -1:
                stop = None
            slices = [slice(None)] * np.ndim(x)
            slices[self.axis] = slice(start, stop, step)
            write[...] = np.asarray(x)[tuple(slices)]
        return f

    def pullback(self, inputs, output, goutput):
        z = cgt.zeros_like(inputs[0])
        z.op.tag = id(output)
        return [Result(IncSli(self.axis), [z] + list(inputs[1:]) + [goutput])] + [None] * 3

    def shp_apply(self, inputs):
        arr, start, stop, step = inputs
        s = cgt.shape(arr)
        s[self.axis] = cgt.ceil_divide(stop - start, step)
        return s

    def typ_apply(self, input_types):
        assert _list_is_valid_sli(input_types[1:])
        return input_types[0]

    def host_inputs(self, n):
        return (1, 2, 3)

    def get_native_compile_info(self, input_types, devtype):
        return NativeCompileInfo(None, prebuilt="cgtb_op_getsli", closure_triples=[("axis", ctypes.c_int, self.axis)])


class IncSli(Op):
    """(x, start, stop, step, y) -> x with x[slice] += y; writes into x's memory (cgt/core.py:1814-1861)."""
    available_impls = ("python", "native_cpu", "native_gpu")
    writes_to_input = 0

    def __init__(self, axis):
        self.axis = axis

    def get_diff(self, _):
        return [True, False, False, False, True]

    def get_py_func(self, input_types):
        def f(reads, write):
            x, start, stop, step, y = reads
            start, stop, step = int(start), int(stop), int(step)
            if step < 0 and stop == -1:
                stop = None
            slices = [slice(None)] * np.ndim(x)
            slices[self.axis] = slice(start, stop, step)
            if write is not x:
                np.copyto(write, x)
            write[tuple(slices)] += y
        return f

    def pullback(self, inputs, output, goutput):
        _x, start, stop, step, _y = inputs
        return [goutput, None, None, None, Result(GetSli(self.axis), [goutput, start, stop, step])]

    def shp_apply(self, inputs):
        return cgt.shape(inputs[0])

    def typ_apply(self, input_types):
        return input_types[0]

    def host_inputs(self, n):
        return (1, 2, 3)

    def get_native_compile_info(self, input_types, devtype):
        return NativeCompileInfo(None, prebuilt="cgtb_op_incsli", closure_triples=[("axis", ctypes.c_int, self.axis)])


class GetFlatIndices(Op):
    """(x, k) -> x.flat[k] (cgt/core.py:1960-1987)."""
    available_impls = ("python", "native_cpu", "native_gpu")

    def get_diff(self, _):
        return [True, False]

    def get_py_func(self, input_types):
        def f(reads, write):
            np.copyto(write, np.asarray(reads[0]).flat[np.asarray(reads[1])])
        return f

    def pullback(self, inputs, output, goutput):
        x, inds = inputs
        ginput = cgt.zeros_like(x)
        return [Result(IncFlatIndices(), [ginput, inds, goutput]), None]

    def shp_apply(self, inputs):
        return cgt.shape(inputs[1])

    def typ_apply(self, inputs):
        assert inputs[1].ndim == 1 and dtype_kind(inputs[1].dtype) == "i"
        return TensorType(inputs[0].dtype, 1)

    def get_native_compile_info(self, input_types, devtype):
        return NativeCompileInfo(None, prebuilt="cgtb_op_getflat")


class IncFlatIndices(Op):
    """(x, k, y) -> x with x.flat[k[i]] += y[i] in index order, so duplicate indices accumulate
    (cgt/core.py:1989-2023); writes into x's memory."""
    available_impls = ("python", "native_cpu", "native_gpu")
    writes_to_input = 0

    def get_diff(self, _):
        return [True, False, True]

    def get_py_func(self, input_types):
        def f(reads, write):
            x, inds, y = reads
            if write is not x:
                np.copyto(write, x)
            for (i, ind) in enumerate(inds):
                write.flat[ind] += y[i]
        return f

    def pullback(self, inputs, output, goutput):
        x, inds, y = inputs
        return [goutput, None, Result(GetFlatIndices(), [goutput, inds])]

    def shp_apply(self, inputs):
        return cgt.shape(inputs[0])

    def typ_apply(self, input_types):
        return input_types[0]

    def get_native_compile_info(self, input_types, devtype):
        return NativeCompileInfo(None, prebuilt="cgtb_op_incflat")


# ================================================================
# Ops: linear algebra
# ================================================================

class Mul22(Op):
    """Matrix product with optional transposes (cgt/core.py:2129-2229); row-major, alpha 1, beta 0."""
    available_impls = ("python", "native_cpu", "native_gpu")

    def __init__(self, tA, tB):
        self.tA = bool(tA)
        self.tB = bool(tB)

    def get_py_func(self, input_types):
        def f(reads, write):
            x, y = reads
            if self.tA: x = x.T
            if self.tB: y = y.T
            np.dot(x, y, out=write)
        return f

    def pullback(self, inputs, output, goutput):
        A, B = inputs
        GC = goutput
        if (self.tA, self.tB) == (False, False):
            return [Result(Mul22(False, True), [GC, B]), Result(Mul22(True, False), [A, GC])]
        elif (self.tA, self.tB) == (False, True):
            return [Result(Mul22(False, False), [GC, B]), Result(Mul22(True, False), [GC, A])]
        elif (self.tA, self.tB) == (True, False):
            return [Result(Mul22(False, True), [B, GC]), Result(Mul22(False, False), [A, GC])]
        else:
            return [Result(Mul22(True, True), [B, GC]), Result(Mul22(True, True), [GC, A])]

    def shp_apply(self, inputs):
        return [cgt.size(inputs[0], 1 if self.tA else 0), cgt.size(inputs[1], 0 if self.tB else 1)]

    def typ_apply(self, input_types):
        assert input_types[0].dtype == cgt.floatX and input_types[1].dtype == cgt.floatX
        return input_types[0]

    def get_closure(self):
        return [("tA", ctypes.c_bool, self.tA), ("tB", ctypes.c_bool, self.tB), ("handle", ctypes.c_void_p, 0)]

    def get_native_compile_info(self, input_types, devtype):
        return NativeCompileInfo(None, prebuilt="cgtb_op_mul22", closure_triples=self.get_closure())

    def __repr__(self):
        return "Mul22{%s,%s}" % ("T" if self.tA else "N", "T" if self.tB else "N")

    __str__ = __repr__


class Mul22BiasAdd(Op):
    """(A, B, bias [1,N], addend [M,N], addend_bias [1,N]) -> (addend + addend_bias) + (op(A).op(B) + bias).

    Not part of the reference's Op set. compilation.fuse_product_sums forms it from the sum of two affine
    pre-activations, (x.W + b) + (h.U + c) (nn.Affine twice, cgt/nn.py:190-215, as an unrolled recurrent cell has it once
    per layer and time step): the three additions run in the output stage of the product h.U, in the association of
    the separate Ops, so the result has their bits. Only products that Mul22 gives to its FMA-tile kernel."""
    available_impls = ("native_gpu",)

    def __init__(self, tA, tB):
        self.tA = bool(tA)
        self.tB = bool(tB)

    def get_diff(self, num_inputs):
        return [False] * num_inputs

    def shp_apply(self, inputs):
        return [cgt.size(inputs[0], 1 if self.tA else 0), cgt.size(inputs[1], 0 if self.tB else 1)]

    def typ_apply(self, input_types):
        return TensorType("f4", 2)

    def get_native_compile_info(self, input_types, devtype):
        return NativeCompileInfo(None, prebuilt="cgtb_op_mul22_bias_add",
                                 closure_triples=[("tA", ctypes.c_bool, self.tA), ("tB", ctypes.c_bool, self.tB), ("handle", ctypes.c_void_p, 0)])

    def __repr__(self):
        return "Mul22BiasAdd{%s,%s}" % ("T" if self.tA else "N", "T" if self.tB else "N")


class BatchedMul22(Op):
    """Per-batch matrix product over the leading axis (cgt/core.py:2231-2288)."""
    available_impls = ("python", "native_cpu", "native_gpu")

    def __init__(self, tA, tB):
        self.tA = bool(tA)
        self.tB = bool(tB)

    def get_py_func(self, input_types):
        def f(reads, z):
            x, y = reads
            for (xmat, ymat, zmat) in zip(x, y, z):
                if self.tA: xmat = xmat.T
                if self.tB: ymat = ymat.T
                np.dot(xmat, ymat, out=zmat)
        return f

    def pullback(self, inputs, output, goutput):
        A, B = inputs
        GC = goutput
        if (self.tA, self.tB) == (False, False):
            return [Result(BatchedMul22(False, True), [GC, B]), Result(BatchedMul22(True, False), [A, GC])]
        elif (self.tA, self.tB) == (False, True):
            return [Result(BatchedMul22(False, False), [GC, B]), Result(BatchedMul22(True, False), [GC, A])]
        elif (self.tA, self.tB) == (True, False):
            return [Result(BatchedMul22(False, True), [B, GC]), Result(BatchedMul22(False, False), [A, GC])]
        else:
            return [Result(BatchedMul22(True, True), [B, GC]), Result(BatchedMul22(True, True), [GC, A])]

    def shp_apply(self, inputs):
        return [cgt.size(inputs[0], 0), cgt.size(inputs[0], 2 if self.tA else 1), cgt.size(inputs[1], 1 if self.tB else 2)]

    def typ_apply(self, input_types):
        return input_types[0]

    def get_native_compile_info(self, input_types, devtype):
        return NativeCompileInfo(None, prebuilt="cgtb_op_batched_mul22",
                                 closure_triples=[("tA", ctypes.c_bool, self.tA), ("tB", ctypes.c_bool, self.tB)])

    def __repr__(self):
        return "BatchedMul22{%s,%s}" % ("T" if self.tA else "N", "T" if self.tB else "N")


# ================================================================
# Ops: tuples
# ================================================================

class TupleIndex(Op):
    available_impls = ("python", "native_cpu", "native_gpu")
    return_type = "byval"

    def __init__(self, idx):
        self.idx = idx

    def get_py_func(self, input_types):
        def f(reads):
            return reads[0][self.idx]
        return f

    def shp_apply(self, inputs):
        return cgt.shape(inputs[0])[self.idx]

    def typ_apply(self, input_types):
        intype = input_types[0]
        assert isinstance(intype, TupleType)
        return intype[self.idx]

    def get_native_compile_info(self, input_types, devtype):
        return NativeCompileInfo(None, prebuilt="cgtb_op_tuple_index", closure_triples=[("idx", ctypes.c_int, self.idx)])

    def __repr__(self):
        return "TupleIndex{%d}" % self.idx


class MakeTuple(Op):
    available_impls = ("python",)
    return_type = "byval"

    def get_py_func(self, input_types):
        def f(inputs):
            return tuple(inputs)
        return f

    def shp_apply(self, inputs):
        return tuple(cgt.shape(x) for x in inputs)

    def typ_apply(self, input_types):
        assert all(isinstance(t, TensorType) for t in input_types), "Can only create tuples of tensors"
        return TupleType(*input_types)


def unpack(tup):
    return [Result(TupleIndex(i), [tup]) for i in range(len(tup.typ))]


# ================================================================
# Graph optimisation (cgt/core.py:2538-2711): CSE, constant propagation, size propagation,
# op-specific identities. Iterative (explicit stack) so deep unrolled graphs do not overflow.
# ================================================================

def init_analysis():
    return {"node2hash": {}, "hash2node": {}, "node2shape": {}, "node2sv": {}, "repl": {}}


def analyze(outputs):
    analysis = init_analysis()
    for node in topsorted(outputs):
        do_analysis(node, analysis)
    return analysis


def simplify_and_analyze(outputs):
    assert isinstance(outputs, list)
    analysis = init_analysis()
    repl = {}
    for output in outputs:
        update_simplify_map(output, analysis, repl)
    return [repl[node] for node in outputs], analysis, repl


def _process_top(stack, analysis, repl):
    (orig, node) = stack.pop()
    if node.is_input():
        return (orig, node)
    for par in node.parents:
        if par not in repl:
            stack.append((orig, node))
            stack.append((par, par))
            return None
    newparents = [repl[p] for p in node.parents]
    newnode = node.clone(newparents)
    newnewnode = maybe_replace(newnode, analysis, repl)
    if newnewnode is None:
        return (orig, newnode)
    assert newnewnode.typ == orig.typ, "simplification changed the type of %s: %s -> %s" % (orig, orig.typ, newnewnode.typ)
    if newnewnode in repl:
        return (orig, newnewnode)
    stack.append((orig, newnewnode))
    return None


def update_simplify_map(node, analysis, repl):
    stack = [(node, node)]
    while stack:
        maybe_pair = _process_top(stack, analysis, repl)
        if maybe_pair:
            (orig, node) = maybe_pair
            do_analysis(node, analysis)
            repl[orig] = node
            repl[node] = node


def do_analysis(node, analysis):
    node2hash = analysis["node2hash"]
    node2shape = analysis["node2shape"]
    node2sv = analysis["node2sv"]
    h = node.get_hash(node2hash)
    node2hash[node] = h
    analysis["hash2node"][h] = node
    if node.is_input():
        node2shape[node] = cgt.shape(node)
    elif isinstance(node.op, TupleIndex):
        node2shape[node] = node2shape[node.parents[0]][node.op.idx]
    else:
        node2shape[node] = node.op.shp_apply(node.parents)
    assert isinstance(node.typ, TupleType) or len(node2shape[node]) == node.ndim
    if not node.is_input():
        op = node.op
        pars = node.parents
        if isinstance(op, Fill):
            node2sv[node] = op.value
        elif isinstance(op, ConstantTensor) and utils.is_singleton(op.value):
            node2sv[node] = op.value.flat[0]
        elif isinstance(op, Repeat) and pars[0] in node2sv:
            node2sv[node] = node2sv[pars[0]]
        elif isinstance(op, (ElwiseUnary, ElwiseBinary)) and all(p in node2sv for p in pars):
            out = np.empty((), node.dtype)
            if isinstance(op, ElwiseUnary):
                op.info.pyfunc(node2sv[pars[0]], out=out)
            else:
                op.info.pyfunc(node2sv[pars[0]], node2sv[pars[1]], out=out)
            node2sv[node] = out[()]


_MAX_FOLDED_ELEMENTS = 4096


def maybe_replace(node, analysis, repl):
    if node.is_input():
        return
    if isinstance(node.op, Constant):
        return
    node2hash = analysis["node2hash"]
    h = node.get_hash(node2hash)
    if h in analysis["hash2node"]:  # common subexpression
        newnode = analysis["hash2node"][h]
        assert newnode in repl and newnode.op.__class__ == node.op.__class__
        return newnode
    parents = node.parents
    # constant propagation: only when every parent is a Constant. A Fill already is a constant in
    # compact form, and large results stay symbolic (a Repeat of a constant becomes a Fill below)
    # instead of being embedded as big host arrays.
    if len(parents) > 0 and all(isinstance(par.op, Constant) for par in parents) and not isinstance(node.op, Fill):
        try:
            val = py_numeric_apply(node, [p.op.value for p in parents])
            if isinstance(val, np.ndarray) and val.size <= _MAX_FOLDED_ELEMENTS:
                return cgt.constant(val)
        except MethodNotDefined:
            pass
    if isinstance(node.op, Size):
        s = analysis["node2shape"][parents[0]][node.op.axis]
        if not (isinstance(s.op, Size) and s.parents[0] is node.parents[0]):
            return s
    return node.op.get_replacement(parents, analysis)


def simplify(xs):
    assert isinstance(xs, list)
    return simplify_and_analyze(xs)[0]


def simplify1(x):
    return simplify([x])[0]


# ================================================================
# Graph traversal
# ================================================================

def topsorted(outputs):
    """Topological order by iterative depth-first search, parents before children."""
    assert isinstance(outputs, (list, tuple))
    marks = {}
    out = []
    stack = []
    for x in outputs:
        stack.append((x, 0))
        while stack:
            (i, jidx) = stack.pop()
            if jidx == 0:
                m = marks.get(i, 0)
                if m == 0:
                    marks[i] = 1
                elif m == 1:
                    raise ValueError("not a dag")
                else:
                    continue
            ps = i.parents
            if jidx == len(ps):
                marks[i] = 2
                out.append(i)
            else:
                stack.append((i, jidx + 1))
                stack.append((ps[jidx], 0))
    return out


def count_nodes(outputs):
    if isinstance(outputs, Node):
        outputs = [outputs]
    return len(list(topsorted(outputs)))


def clone(nodes, replace=None):
    if isinstance(nodes, Node):
        return _clone_list([nodes], replace)[0]
    return _clone_list(list(nodes), replace)


def _clone_list(nodes, replace):
    assert isinstance(nodes, list)
    if replace is None:
        replace = {}
    else:
        replace = {k: (v if isinstance(v, Node) else as_node(v)) for (k, v) in replace.items()}
    for node in topsorted(nodes):
        if node in replace:
            pass
        elif node.is_input():
            replace[node] = node
        else:
            replace[node] = node.clone([replace[p] for p in node.parents])
    return [replace[node] for node in nodes]


def alloc_from_shp(shp, typ):
    if isinstance(shp, tuple):
        return tuple([alloc_from_shp(shpel, typel) for (shpel, typel) in utils.safezip(shp, typ)])
    return np.empty([int(s) for s in shp], typ.dtype)


def get_numeric_shape_fun(node):
    args = [make_argument(p.typ) for p in node.parents]
    syshape = node.op.shp_apply(args)
    if isinstance(syshape, list):
        istuple = False
        sizes = None
    elif isinstance(syshape, tuple):
        istuple = True
        sizes = [len(s) for s in syshape]
        syshape = [el for s in syshape for el in s]
    else:
        raise ValueError("shape should be a list or tuple of lists. got %s" % (syshape,))
    nodes = topsorted(syshape)

    def fn(vals):
        node2val = {n: v for (n, v) in utils.safezip(args, vals)}
        for n in nodes:
            if not n.is_argument():
                node2val[n] = py_numeric_apply(n, [node2val[p] for p in n.parents])
        nushape = [node2val[n] for n in syshape]
        if istuple:
            out, start = [], 0
            for sz in sizes:
                out.append(nushape[start:start + sz])
                start += sz
            return tuple(out)
        return nushape
    return fn


def py_numeric_apply(node, vals):
    """Evaluate one node on numpy values with the Op's Python function (compile-time folding)."""
    if "python" not in node.op.available_impls:
        raise MethodNotDefined("Op %r has no Python implementation" % node.op)
    callable_ = node.op.get_py_callable([par.typ for par in node.parents])
    if node.op.return_type == "byval":
        return callable_.call(vals)
    shp = get_numeric_shape_fun(node)(vals)
    out = alloc_from_shp(shp, node.typ)
    callable_.call(vals, out)
    return out


class NonDifferentiable(Exception):
    pass


class Disconnected(Exception):
    pass


class Todo(Exception):
    pass


class ShapeError(Exception):
    pass


class AllocationError(Exception):
    pass


class MethodNotDefined(Exception):
    pass


class Unreachable(Exception):
    pass


# ================================================================
# Configuration (cgt/core.py:2948-3033; keys of cgtrc_spec.ini plus the GPU-backend ones).
# Dict-backed; overridden by the CGT_FLAGS environment variable (k=v,k=v).
# ================================================================

_DEFAULTS = dict(
    debug=False, precision="single", backend="native", cache_dir="~/.cgt_b200_cache", enable_inplace_opt=True,
    enable_simplification=True, parallel=False, num_threads=1, force_python_impl=False, debug_cpp=False, verbose=False,
    # additions for this backend
    devtype="gpu", device_index=0, use_cuda_graphs=True, fuse_elementwise=True, jit_fused_elementwise=True, fuse_conv_dgrad=True, fuse_conv_output=True, fuse_conv_grad_input=True, fuse_conv_implicit=True, fuse_conv_direct=True, fuse_flat_index_rows=True, hoist_filter_splits=True, split_gate_columns=True, fuse_product_sums=True, merge_parameter_updates=True, fuse_rows=True, fuse_slice_sums=True, fuse_slice_views=True, batch_summed_products=True,
    pad_conv_columns=True, profile=False,
)

_CONFIG = None


def get_config(force_reload=False):
    global _CONFIG
    if _CONFIG is None or force_reload:
        _CONFIG = _load_config()
    return _CONFIG


def _parse_value(old, s):
    if isinstance(old, bool):
        if s.lower() in ("true", "1", "yes", "on"): return True
        if s.lower() in ("false", "0", "no", "off"): return False
        raise ValueError("not a boolean: %s" % s)
    if isinstance(old, int): return int(s)
    if isinstance(old, float): return float(s)
    return s


def _load_config():
    config = dict(_DEFAULTS)
    envflags = os.getenv("CGT_FLAGS")
    if envflags:
        for pair in envflags.split(","):
            lhs, rhs = pair.split("=")
            assert lhs in config, "Unrecognized config option %s provided" % lhs
            config[lhs] = _parse_value(config[lhs], rhs)
    local_rank = os.getenv("LOCAL_RANK")
    if local_rank is not None and "device_index" not in (envflags or ""):
        config["device_index"] = int(local_rank)
    config["default_device"] = Device(config["devtype"], int(config["device_index"]))
    cgt.set_precision(config["precision"])
    return config


def reset_config():
    get_config(True)


def update_config(**kws):
    config = get_config()
    for (name, val) in kws.items():
        if name not in config:
            raise ValueError("%s is not a valid config option" % name)
        config[name] = val
    if "precision" in kws:
        cgt.set_precision(config["precision"])


class scoped_update_config(object):
    """``with scoped_update_config(precision='double'): ...`` restores the old values on exit."""

    def __init__(self, **kw):
        self.kw = kw
        config = get_config()
        self.prevsettings = {}
        for k in kw:
            if k not in config:
                raise ValueError("%s is not a valid config option" % k)
            self.prevsettings[k] = config[k]

    def __enter__(self):
        config = get_config()
        config.update(self.kw)
        cgt.set_precision(config["precision"])

    def __exit__(self, *args):
        config = get_config()
        config.update(self.prevsettings)
        cgt.set_precision(config["precision"])
