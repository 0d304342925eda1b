"""Cross-channel local response normalisation (counterpart of cgt/nn_ops/cross_channel_lrn.py).

Forward returns the tuple (top, scale) with scale = 1 + (alpha/n) * sum over the channel window of
x^2 and top = x * scale^(-beta); backward consumes (x, top, scale, gtop).
"""
import ctypes
from collections import namedtuple

from .. import core

LRNInfo = namedtuple("LRNInfo", ["localsize", "alpha", "beta"])


def make_closure(info):
    return [("localsize", ctypes.c_int, int(info.localsize)), ("alpha", ctypes.c_double, float(info.alpha)),
            ("beta", ctypes.c_double, float(info.beta))]


class CrossChannelLRNForward(core.Op):
    available_impls = ("native_gpu",)

    def __init__(self, info):
        assert isinstance(info, LRNInfo)
        self.info = info

    def get_native_compile_info(self, input_types, devtype):
        return core.NativeCompileInfo(None, prebuilt="cgtb_op_lrn_forward", closure_triples=make_closure(self.info))

    def shp_apply(self, inputs):
        return (core.cgt.shape(inputs[0]), core.cgt.shape(inputs[0]))

    def typ_apply(self, input_types):
        return core.TupleType(input_types[0], input_types[0])

    def pullback(self, inputs, output, gout):
        top, scaling = core.unpack(output)
        gtop, _ = gout
        return [core.Result(CrossChannelLRNBackward(self.info), [inputs[0], top, scaling, gtop])]

    def __repr__(self):
        return "LRNForward{%s}" % (tuple(self.info),)


class CrossChannelLRNBackward(core.Op):
    available_impls = ("native_gpu",)

    def __init__(self, info):
        self.info = info

    def get_diff(self, n):
        return [False, False, False, True]

    def get_native_compile_info(self, input_types, devtype):
        return core.NativeCompileInfo(None, prebuilt="cgtb_op_lrn_backward", closure_triples=make_closure(self.info))

    def shp_apply(self, inputs):
        return core.cgt.shape(inputs[0])

    def typ_apply(self, input_types):
        return core.TensorType(input_types[0].dtype, 4)

    def __repr__(self):
        return "LRNBackward{%s}" % (tuple(self.info),)


def cross_channel_lrn(X, localsize, alpha, beta):
    assert X.ndim == 4
    return core.Result(CrossChannelLRNForward(LRNInfo(localsize, alpha, beta)), [X])[0]
