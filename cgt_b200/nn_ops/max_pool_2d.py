"""MaxPool / MaxPoolPullback Ops (counterpart of the reference's cgt/nn_ops/max_pool_2d.py).

MaxPool returns a tuple (pooled values, int32 argmax mask). The pooled extent is
``iceil((H + 2*pad - k) / stride)`` -- the reference's formula, without the ``+ 1`` of Caffe.
"""
from collections import namedtuple

from .. import core
from .im2col import info2closure

PoolInfo = namedtuple("PoolInfo", ["kernel_h", "kernel_w", "pad_h", "pad_w", "stride_h", "stride_w"])


class MaxPool(core.Op):
    available_impls = ("native_cpu", "native_gpu")

    def __init__(self, info):
        assert info.stride_h > 0 and info.stride_w > 0
        self.info = info

    def get_diff(self, _):
        return [True]

    def pullback(self, inputs, y, gy):
        pool, mask = core.unpack(y)
        gpool, _gmask = gy
        return [core.Result(MaxPoolPullback(self.info), [inputs[0], pool, mask, gpool])]

    def shp_apply(self, inputs):
        cgt = core.cgt
        info = self.info
        batch_size, channels, height, width = cgt.shape(inputs[0])
        pooled_height = cgt.ceil_divide(height + 2 * info.pad_h - info.kernel_h, info.stride_h)
        pooled_width = cgt.ceil_divide(width + 2 * info.pad_w - info.kernel_w, info.stride_w)
        outshape = [batch_size, channels, pooled_height, pooled_width]
        return (outshape, outshape)

    def typ_apply(self, inputs):
        return core.TupleType(core.TensorType(inputs[0].dtype, 4), core.TensorType("i4", 4))

    def get_native_compile_info(self, input_types, devtype):
        return core.NativeCompileInfo(None, prebuilt="cgtb_op_max_pool", closure_triples=info2closure(self.info))

    def __repr__(self):
        return "MaxPool{%s}" % (tuple(self.info),)


class MaxPoolPullback(core.Op):
    """(x, pooled, mask, gpooled) -> gx; x and pooled only supply shapes."""
    available_impls = ("native_cpu", "native_gpu")

    def __init__(self, info):
        self.info = info

    def get_diff(self, n):
        return [False, False, False, True]

    def shp_apply(self, inputs):
        return core.cgt.shape(inputs[0])

    def typ_apply(self, inputs):
        return core.TensorType(inputs[0].dtype, 4)

    def get_native_compile_info(self, input_types, devtype):
        return core.NativeCompileInfo(None, prebuilt="cgtb_op_max_pool_pullback", closure_triples=info2closure(self.info))

    def __repr__(self):
        return "MaxPoolPullback{%s}" % (tuple(self.info),)
