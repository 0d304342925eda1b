"""TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Evaluates a cgt_b200 expression graph on the host with the oracle kernels: the "reference CPU
backend" stand-in used by the parity tests, the smoke check and the benchmark's CPU baseline.

It takes the same simplified graph the GPU compiler takes (``compilation.simplify_for_execution``), so
the op sequence is identical, and runs each node with the CPU restatement (``impl="port"``) or, for
im2col / col2im / pooling / LRN, the reference's own headers (``impl="ref"``). GEMMs go to OpenBLAS
through numpy. Shared variables are copied in at construction and live in this object; the GPU-side
values are never touched.
"""
import numpy as np

from cgt_b200 import compilation, core
from cgt_b200.nn_ops import cross_channel_lrn as lrn_ops
from cgt_b200.nn_ops import im2col as im2col_ops
from cgt_b200.nn_ops import max_pool_2d as pool_ops

from . import oracle as O


class OracleFunction(object):
    def __init__(self, inputs, outputs, updates=None, givens=None, impl="port", wide_sums=False):
        """wide_sums=True: Sum and Mul22 accumulate in float64 and round once (not what the reference does: an
        adjudicator for float32 results whose difference comes from the order of a long summation)."""
        self.wide_sums = wide_sums
        self.single = isinstance(outputs, core.Node)
        outs = [outputs] if self.single else list(outputs)
        updates = compilation._check_updates(updates)
        self.inputs = inputs
        self.impl = impl
        self.outputs, self.update_srcs, self.update_targs, _ = compilation.simplify_for_execution(outs, updates, givens or [])
        self.nodes = core.topsorted(self.outputs + self.update_targs)
        self.values = {}
        for node in self.nodes:
            if node.is_data():
                self.values[node.op] = node.op.get_value().copy()
        for src in self.update_srcs:
            if src.op not in self.values:
                self.values[src.op] = src.op.get_value().copy()

    def get_value(self, shared_node):
        return self.values[shared_node.op]

    def _kimpl(self, geometry_ok=True):
        return self.impl if (self.impl == "ref" and O.have_ref() and geometry_ok) else "port"

    def __call__(self, *args):
        assert len(args) == len(self.inputs)
        val = {}
        for (node, a) in zip(self.inputs, args):
            val[node] = core.as_valid_array(a, node.dtype)
        for node in self.nodes:
            if node in val:
                continue
            if node.is_argument():
                raise ValueError("argument %r was not supplied" % node)
            val[node] = self._eval(node, [val[p] for p in node.parents])
        outs = [_copy(val[n]) for n in self.outputs]
        for (src, targ) in zip(self.update_srcs, self.update_targs):
            self.values[src.op] = np.array(val[targ], copy=True)
        return outs[0] if self.single else outs

    def _eval(self, node, p):
        op = node.op
        if isinstance(op, core.InMemoryData):
            return self.values[op]
        if isinstance(op, core.ConstantTensor):
            return op.value
        if isinstance(op, core.Fill):
            return O.fill(op.value.item(), [int(s) for s in p], node.dtype)
        if isinstance(op, core.Arange):
            return O.arange(int(p[0]), int(p[1]), int(p[2]))
        if isinstance(op, core.ElwiseUnary):
            name = op.opname if op.opname in O.UNARY else ("cast" if op.opname.startswith("cast_to_") else None)
            if name is None:
                raise NotImplementedError("oracle has no expression for unary op %s" % op.opname)
            return O.unary(name, p[0], node.dtype)
        if isinstance(op, core.ElwiseBinary):
            return O.binary(op.opname, p[0], p[1], node.dtype)
        if isinstance(op, core.Size):
            return np.array(np.shape(p[0])[op.axis], "i8")
        if isinstance(op, core.Reshape):
            return np.asarray(p[0]).reshape([int(s) for s in p[1:]])
        if isinstance(op, core.Concatenate):
            return O.concatenate(p, op.axis)
        if isinstance(op, core.Repeat):
            return O.repeat(p[0], op.axes, [int(r) for r in p[1:]])
        if isinstance(op, core.Transpose):
            return O.transpose(p[0], op.axes)
        if isinstance(op, core.Sum):
            if self.wide_sums and np.asarray(p[0]).dtype == np.float32:
                return np.asarray(p[0], "f8").sum(axis=tuple(op.axes), keepdims=True).astype("f4")
            return O.reduce("sum", p[0], op.axes)
        if isinstance(op, core.Max):
            return O.reduce("max", p[0], op.axes)
        if isinstance(op, core.GetSli):
            return O.getsli(p[0], op.axis, int(p[1]), int(p[2]), int(p[3]))
        if isinstance(op, core.IncSli):
            return O.incsli(p[0], op.axis, int(p[1]), int(p[2]), int(p[3]), p[4])
        if isinstance(op, core.GetFlatIndices):
            return O.getflat(p[0], p[1])
        if isinstance(op, core.IncFlatIndices):
            return O.incflat(p[0], p[1], p[2])
        if isinstance(op, core.Mul22):
            if self.wide_sums and np.asarray(p[0]).dtype == np.float32:
                a, b = np.asarray(p[0], "f8"), np.asarray(p[1], "f8")
                return ((a.T if op.tA else a) @ (b.T if op.tB else b)).astype("f4")
            return O.mul22(p[0], p[1], op.tA, op.tB)
        if isinstance(op, core.BatchedMul22):
            return O.batched_mul22(p[0], p[1], op.tA, op.tB)
        if isinstance(op, core.TupleIndex):
            return p[0][op.idx]
        if isinstance(op, core.MakeTuple):
            return tuple(p)
        if isinstance(op, core.Transport):
            return p[0]
        if isinstance(op, im2col_ops.Im2Col):
            i = op.info
            return self._geo(O.im2col, p[0], i)
        if isinstance(op, im2col_ops.Col2Im):
            i = op.info
            shape = tuple(int(s) for s in p[1:])
            return self._geo(O.col2im, p[0], i, shape)
        if isinstance(op, pool_ops.MaxPool):
            i = op.info
            return O.max_pool(p[0], (i.kernel_h, i.kernel_w), (i.pad_h, i.pad_w), (i.stride_h, i.stride_w), impl=self._kimpl())
        if isinstance(op, pool_ops.MaxPoolPullback):
            # the reference's scatter writes out of bounds through a mask of -1 (an all-NaN window,
            # include/pooling.h:96-97): such inputs only go to the guarded restatement
            ok = bool((np.asarray(p[2]) >= 0).all())
            return O.max_pool_pullback(np.shape(p[0]), p[2], p[3], impl=self._kimpl(ok))
        if isinstance(op, lrn_ops.CrossChannelLRNForward):
            i = op.info
            return O.lrn_forward(p[0], i.localsize, i.alpha, i.beta, impl=self._kimpl())
        if isinstance(op, lrn_ops.CrossChannelLRNBackward):
            i = op.info
            return O.lrn_backward(p[0], p[1], p[2], p[3], i.localsize, i.alpha, i.beta, impl=self._kimpl())
        ev = getattr(op, "oracle_eval", None)
        if ev is not None:
            return ev(p)
        raise NotImplementedError("oracle cannot evaluate %r" % op)

    def _geo(self, fn, x, info, *extra):
        args = list(extra) + [(info.kernel_h, info.kernel_w), (info.pad_h, info.pad_w), (info.stride_h, info.stride_w)]
        if self.impl == "ref" and O.have_ref():
            try:
                return fn(x, *args, impl="ref")
            except RuntimeError:
                pass  # geometry not instantiated in the shim: the restatement covers it
        return fn(x, *args, impl="port")


def _copy(x):
    if isinstance(x, tuple):
        return tuple(np.array(e, copy=True) for e in x)
    return np.array(x, copy=True)


def function(inputs, outputs, updates=None, givens=None, impl="port", wide_sums=False):
    return OracleFunction(inputs, outputs, updates=updates, givens=givens, impl=impl, wide_sums=wide_sums)
