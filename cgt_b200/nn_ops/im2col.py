"""Im2Col / Col2Im Ops (counterpart of the reference's cgt/nn_ops/im2col.py).

Column layout is channels-last, ``[B, Ho, Wo, C*kh*kw]`` with column channel ``(c_im*kh + i)*kw + j``,
so ``Mul22(F,T)(col.reshape(B*Ho*Wo, Z), W.reshape(L, Z))`` is the cross-correlation.
"""
import ctypes

import numpy as np
from collections import namedtuple

from .. import core

Im2ColInfo = namedtuple("Im2ColInfo", ["kernel_h", "kernel_w", "pad_h", "pad_w", "stride_h", "stride_w"])


def im2col(x, kernelshape, pad, stride):
    assert stride[0] > 0 and stride[1] > 0
    assert kernelshape[0] > 0 and kernelshape[1] > 0
    kernelshape, pad, stride = map(tuple, (kernelshape, pad, stride))
    return core.Result(Im2Col(Im2ColInfo(*(kernelshape + pad + stride))), [x])


def info2closure(info):
    """Field order of the reference's conv_closure struct (include/pooling.h:7-14)."""
    return [(name, ctypes.c_int, int(getattr(info, name)))
            for name in ("kernel_h", "kernel_w", "pad_h", "pad_w", "stride_h", "stride_w")]


class Im2Col(core.Op):
    available_impls = ("native_cpu", "native_gpu")

    def __init__(self, info, pitch=0):
        """pitch > 0 (set only by compilation.pad_conv_columns, after differentiation): column rows are `pitch`
        entries apart instead of C*kh*kw, the extra entries zero."""
        assert info.stride_h > 0 and info.stride_w > 0
        self.info = info
        self.pitch = int(pitch)

    def get_diff(self, _):
        return [True]

    def pullback(self, inputs, _y, gy):
        assert not self.pitch, "padded column rows are introduced after differentiation"
        return [core.Result(Col2Im(self.info), [gy] + core.cgt.shape(inputs[0]))]

    def shp_apply(self, inputs):
        info = self.info
        batch_size, channels, height, width = core.cgt.shape(inputs[0])
        height_out = (height + 2 * info.pad_h - info.kernel_h) // info.stride_h + 1
        width_out = (width + 2 * info.pad_w - info.kernel_w) // info.stride_w + 1
        rowlen = core.cgt.constant(self.pitch) if self.pitch else channels * info.kernel_w * info.kernel_h
        return [batch_size, height_out, width_out, rowlen]

    def typ_apply(self, inputs):
        assert inputs[0].ndim == 4
        return core.TensorType(inputs[0].dtype, 4)

    def get_native_compile_info(self, input_types, devtype):
        return core.NativeCompileInfo(None, prebuilt="cgtb_op_im2col", closure_triples=info2closure(self.info))

    def __repr__(self):
        return "Im2Col{%s}" % (tuple(self.info),) + ("/pitch%d" % self.pitch if self.pitch else "")


class Col2Im(core.Op):
    """(col, B, C, H, W) -> image gradient; the adjoint of Im2Col."""
    available_impls = ("native_cpu", "native_gpu")

    def __init__(self, info):
        self.info = info

    def get_diff(self, n):
        return [True] + [False] * (n - 1)

    def pullback(self, inputs, _y, gy):
        return [core.Result(Im2Col(self.info), [gy])] + [None] * (len(inputs) - 1)

    def shp_apply(self, inputs):
        return list(inputs[1:])

    def typ_apply(self, inputs):
        return core.TensorType(inputs[0].dtype, 4)

    def host_inputs(self, n):
        return (1, 2, 3, 4)

    def get_native_compile_info(self, input_types, devtype):
        return core.NativeCompileInfo(None, prebuilt="cgtb_op_col2im", closure_triples=info2closure(self.info))

    def __repr__(self):
        return "Col2Im{%s}" % (tuple(self.info),)


class ConvDgrad(core.Op):
    """(dy NHWC [B,Ho,Wo,Cin], filters, B, C, H, W) -> dx NCHW [B,C,H,W]: the data gradient of a stride-1 convolution
    in one kernel. The filters are the layer's bank [Cin,C,kh,kw] as stored (w_bank=True, what the compiler passes)
    or a copy rearranged to [C,kh,kw,Cin].

    Not part of the reference's Op set. The compiler substitutes it (compilation.fuse_conv_dgrad) for the
    pair that Im2Col.pullback produces, Col2Im(Mul22(dy, W)) (cgt/nn_ops/im2col.py, cgt/nn.py conv2d), when
    the extents allow; the column matrix is then neither written nor read."""
    available_impls = ("native_gpu",)

    def __init__(self, info, w_bank=False, pre=False):
        assert info.stride_h == 1 and info.stride_w == 1
        self.info = info
        self.w_bank = bool(w_bank)
        self.pre = bool(pre)    # a seventh input: the bank's [w_hi | w_lo] copy from SplitFilterBanks

    def get_diff(self, n):
        return [False] * n

    def shp_apply(self, inputs):
        return list(inputs[2:6])

    def typ_apply(self, inputs):
        return core.TensorType("f4", 4)

    def host_inputs(self, n):
        return (2, 3, 4, 5)

    def get_native_compile_info(self, input_types, devtype):
        return core.NativeCompileInfo(None, prebuilt="cgtb_op_conv_dgrad",
                                      closure_triples=info2closure(self.info) + [("w_bank", ctypes.c_int, int(self.w_bank)),
                                                                                ("pre", ctypes.c_int, int(self.pre))])

    def __repr__(self):
        return "ConvDgrad{%s}" % (tuple(self.info),)


class ConvBiasRelu(core.Op):
    """(col [M,K], W [C,K], bias [1,C,1,1], B, C, H, W) -> tuple(mask i1, relu f4), both NCHW [B,C,H,W]:
    the output stage of a convolution layer, Mul22 -> Transpose{0,3,1,2} -> + bias -> relu, in one call.

    Not part of the reference's Op set. The compiler substitutes it (compilation.fuse_conv_output) for the
    sequence that nn.conv2d / SpatialConvolution / rectify spell out (cgt/nn.py:87-100, 228-233, 44-45); the
    values are bit-identical to that sequence."""
    available_impls = ("native_gpu",)

    def get_diff(self, n):
        return [False] * n

    def shp_apply(self, inputs):
        shp = list(inputs[3:])
        return (shp, list(shp))

    def typ_apply(self, inputs):
        return core.TupleType(core.TensorType("i1", 4), core.TensorType("f4", 4))

    def host_inputs(self, n):
        return tuple(range(3, n))

    def get_native_compile_info(self, input_types, devtype):
        return core.NativeCompileInfo(None, prebuilt="cgtb_op_conv_bias_relu")

    def __repr__(self):
        return "ConvBiasRelu"


class ReluGradNHWC(core.Op):
    """(mask i1 NCHW, g f4 NCHW) -> tuple(mask*g as NHWC [B,H,W,C], Sum{0,2,3}(mask*g) as [1,C,1,1]): the input
    stage of a convolution layer's backward pass in one call.

    Not part of the reference's Op set. The compiler substitutes it (compilation.fuse_conv_grad_input) for the relu
    pullback (ElwiseBinary *), its Transpose{0,2,3,1} and the bias gradient's Sum{0,2,3} that differentiating
    nn.rectify / conv2d / SpatialConvolution yields (cgt/nn.py:44-45, 87-100, 228-233). The transposed product has the
    bits of the Op sequence; the bias gradient is summed in a different fixed order."""
    available_impls = ("native_gpu",)

    def get_diff(self, n):
        return [False] * n

    def shp_apply(self, inputs):
        (b, c, h, w) = core.cgt.shape(inputs[1])
        one = core.cgt.constant(1)
        return ([b, h, w, c], [one, c, one, one])

    def typ_apply(self, inputs):
        return core.TupleType(core.TensorType("f4", 4), core.TensorType("f4", 4))

    def get_native_compile_info(self, input_types, devtype):
        return core.NativeCompileInfo(None, prebuilt="cgtb_op_relu_grad_nhwc")

    def __repr__(self):
        return "ReluGradNHWC"


class ConvWgrad(core.Op):
    """(dy [M,C], col [M,pitch]) -> dy^T . col[:, :K] as [C,K]: the filter gradient of a convolution whose column
    matrix has padded rows.

    Not part of the reference's Op set. The compiler substitutes it (compilation.pad_conv_columns) for the
    Mul22{T,N}(dy, col) that differentiating nn.conv2d yields (cgt/nn.py:93-100, cgt/core.py:2195-2222) when it
    widens the rows of that column matrix to a multiple of four entries."""
    available_impls = ("native_gpu",)

    def __init__(self, k):
        self.k = int(k)

    def get_diff(self, n):
        return [False] * n

    def shp_apply(self, inputs):
        return [core.cgt.size(inputs[0], 1), core.cgt.constant(self.k)]

    def typ_apply(self, inputs):
        return core.TensorType("f4", 2)

    def get_native_compile_info(self, input_types, devtype):
        return core.NativeCompileInfo(None, prebuilt="cgtb_op_conv_wgrad")

    def __repr__(self):
        return "ConvWgrad{%d}" % self.k


class ConvDirectFwd(core.Op):
    """(x NCHW [B,Cin,H,W], W [Cout, Cin*kh*kw], bias [1,Cout,1,1], B, Cout, H, W) -> tuple(mask i1, relu f4), both NCHW:
    the forward pass of a stride-1 "same" convolution layer on very few input channels, computed directly from the image.

    Not part of the reference's Op set. The compiler substitutes it (compilation.fuse_conv_direct) for
    Im2Col -> ConvBiasRelu (cgt/nn.py:87-100, 228-233, 44-45) when the layer has 3 input channels, 5 x 5 filters and 32
    filters on images 32 pixels wide: the column matrix of such a layer is 25 times its input. Float32 tolerance against
    the column-matrix path (the sums run tap by tap in FMA arithmetic)."""
    available_impls = ("native_gpu",)

    def __init__(self, info):
        self.info = info

    def get_diff(self, n):
        return [False] * n

    def shp_apply(self, inputs):
        shp = list(inputs[3:])
        return (shp, list(shp))

    def typ_apply(self, inputs):
        return core.TupleType(core.TensorType("i1", 4), core.TensorType("f4", 4))

    def host_inputs(self, n):
        return tuple(range(3, n))

    def get_native_compile_info(self, input_types, devtype):
        return core.NativeCompileInfo(None, prebuilt="cgtb_op_conv_direct_fwd", closure_triples=info2closure(self.info))

    def __repr__(self):
        return "ConvDirectFwd{%s}" % (tuple(self.info),)


class ConvDirectWgrad(core.Op):
    """(x NCHW [B,Cin,H,W], dy channels-last with B*H*W*Cout elements) -> [Cout, Cin*kh*kw]: the filter gradient of the same
    layer, directly from the image (compilation.fuse_conv_direct puts it in place of the Mul22{T,N} / ConvWgrad on the
    column matrix). Partial results per block of image rows, added in block order."""
    available_impls = ("native_gpu",)

    def __init__(self, info, cout):
        self.info = info
        self.cout = int(cout)

    def get_diff(self, n):
        return [False] * n

    def shp_apply(self, inputs):
        info = self.info
        return [core.cgt.constant(self.cout), core.cgt.size(inputs[0], 1) * (info.kernel_h * info.kernel_w)]

    def typ_apply(self, inputs):
        return core.TensorType("f4", 2)

    def get_native_compile_info(self, input_types, devtype):
        return core.NativeCompileInfo(None, prebuilt="cgtb_op_conv_direct_wgrad",
                                      closure_triples=info2closure(self.info) + [("cout", ctypes.c_int, self.cout)])

    def __repr__(self):
        return "ConvDirectWgrad{%s}" % (tuple(self.info),)


class ConvDirectWgradRelu(core.Op):
    """(x NCHW [B,Cin,H,W], relu mask i1 NCHW [B,Cout,H,W], g f4 NCHW) -> tuple(filter gradient [Cout, Cin*kh*kw], bias
    gradient [1,Cout,1,1]): ConvDirectWgrad fed by the layer's backward inputs. compilation.fuse_conv_direct puts it in
    place of ReluGradNHWC + ConvDirectWgrad when the channels-last gradient has no other reader (a first layer has no
    data gradient), so that gradient is never written; the kernel forms mask * g while it stages its tile."""
    available_impls = ("native_gpu",)

    def __init__(self, info, cout):
        self.info = info
        self.cout = int(cout)

    def get_diff(self, n):
        return [False] * n

    def shp_apply(self, inputs):
        info = self.info
        one = core.cgt.constant(1)
        c = core.cgt.constant(self.cout)
        return ([c, core.cgt.size(inputs[0], 1) * (info.kernel_h * info.kernel_w)], [one, c, one, one])

    def typ_apply(self, inputs):
        return core.TupleType(core.TensorType("f4", 2), core.TensorType("f4", 4))

    def get_native_compile_info(self, input_types, devtype):
        return core.NativeCompileInfo(None, prebuilt="cgtb_op_conv_direct_wgrad_relu",
                                      closure_triples=info2closure(self.info) + [("cout", ctypes.c_int, self.cout)])

    def __repr__(self):
        return "ConvDirectWgradRelu{%s}" % (tuple(self.info),)


class ConvFwdBiasRelu(core.Op):
    """(x NHWC [B,H,W,Cin], filters, bias [1,Cout,1,1], B, Cout, Ho, Wo) -> tuple(mask i1, relu f4), both NCHW
    [B,Cout,Ho,Wo]: the forward pass of a stride-1 convolution layer in one kernel. The filters are the layer's bank
    [Cout,Cin,kh,kw] as stored (w_bank=True, what the compiler passes) or a copy rearranged to [Cout,kh,kw,Cin].

    Not part of the reference's Op set. The compiler substitutes it (compilation.fuse_conv_implicit) for
    ConvBiasRelu(Reshape(Im2Col(x)), ...), i.e. for the sequence that nn.conv2d / SpatialConvolution / rectify spell
    out (cgt/nn.py:87-100, 228-233, 44-45; include/im2col.h:6-28), when the extents allow; the column matrix is then
    neither written nor read. The sum over a patch runs in (tap, channel) order instead of (channel, tap): float32
    tolerance against the Op sequence."""
    available_impls = ("native_gpu",)

    def __init__(self, info, w_bank=False, pre=False):
        assert info.stride_h == 1 and info.stride_w == 1
        self.info = info
        self.w_bank = bool(w_bank)
        self.pre = bool(pre)    # an eighth input: the bank's [w_hi | w_lo] copy from SplitFilterBanks

    def get_diff(self, n):
        return [False] * n

    def shp_apply(self, inputs):
        shp = list(inputs[3:7])
        return (shp, list(shp))

    def typ_apply(self, inputs):
        return core.TupleType(core.TensorType("i1", 4), core.TensorType("f4", 4))

    def host_inputs(self, n):
        return (3, 4, 5, 6)

    def get_native_compile_info(self, input_types, devtype):
        return core.NativeCompileInfo(None, prebuilt="cgtb_op_conv_fwd_bias_relu",
                                      closure_triples=info2closure(self.info) + [("w_bank", ctypes.c_int, int(self.w_bank)),
                                                                                ("pre", ctypes.c_int, int(self.pre))])

    def __repr__(self):
        return "ConvFwdBiasRelu{%s}" % (tuple(self.info),)


class SplitFilterBanks(core.Op):
    """(filter banks...) -> tuple of float32 [2, n_out, taps * n_src] arrays, one per job: the K-major [w_hi | w_lo] copy
    that ConvFwdBiasRelu (layout 1) or ConvDgrad (layout 2) of a layer needs of its bank, all made by ONE launch.
    jobs: (input index, n_out, n_src, taps, layout). The convolution calls otherwise make that copy themselves, one
    small launch each; the banks change only with the parameter update, so the compiler
    (compilation.hoist_filter_splits) makes all copies of a step here, ahead of its first convolution. Same bits."""
    available_impls = ("native_gpu",)
    MAX_JOBS = 8

    def __init__(self, jobs):
        assert 1 <= len(jobs) <= self.MAX_JOBS
        self.jobs = [tuple(int(v) for v in job) for job in jobs]

    def get_diff(self, n):
        return [False] * n

    def shp_apply(self, inputs):
        c = lambda v: core.cgt.constant(np.array(v, "i8"))
        return tuple([c(2), c(n_out), c(taps * n_src)] for (_src, n_out, n_src, taps, _layout) in self.jobs)

    def typ_apply(self, inputs):
        return core.TupleType(*[core.TensorType("f4", 3) for _ in self.jobs])

    def get_native_compile_info(self, input_types, devtype):
        def arr(k):
            vals = [job[k] for job in self.jobs] + [0] * (self.MAX_JOBS - len(self.jobs))
            return (ctypes.c_int * self.MAX_JOBS)(*vals)
        return core.NativeCompileInfo(None, prebuilt="cgtb_op_split_filter_banks", closure_triples=[
            ("njobs", ctypes.c_int, len(self.jobs)), ("src", ctypes.c_int * self.MAX_JOBS, arr(0)),
            ("n_out", ctypes.c_int * self.MAX_JOBS, arr(1)), ("n_src", ctypes.c_int * self.MAX_JOBS, arr(2)),
            ("taps", ctypes.c_int * self.MAX_JOBS, arr(3)), ("layout", ctypes.c_int * self.MAX_JOBS, arr(4))])

    def __repr__(self):
        return "SplitFilterBanks{%d}" % len(self.jobs)


class ConvWgradImplicit(core.Op):
    """(x NHWC [B,H,W,Cin], dy NHWC [B,Ho,Wo,Cout]) -> filter gradient [Cout, Cin*kh*kw] of a stride-1 convolution.

    Not part of the reference's Op set. The compiler substitutes it (compilation.fuse_conv_implicit) for
    Mul22{T,N}(dy, Reshape(Im2Col(x))), which differentiating nn.conv2d yields (cgt/nn.py:93-100,
    cgt/core.py:2162-2175), together with ConvFwdBiasRelu, so that the column matrix disappears from the step."""
    available_impls = ("native_gpu",)

    def __init__(self, info):
        assert info.stride_h == 1 and info.stride_w == 1
        self.info = info

    def get_diff(self, n):
        return [False] * n

    def shp_apply(self, inputs):
        cin = core.cgt.size(inputs[0], 3)
        return [core.cgt.size(inputs[1], 3), cin * (self.info.kernel_h * self.info.kernel_w)]

    def typ_apply(self, inputs):
        return core.TensorType("f4", 2)

    def get_native_compile_info(self, input_types, devtype):
        return core.NativeCompileInfo(None, prebuilt="cgtb_op_conv_wgrad_implicit", closure_triples=info2closure(self.info))

    def __repr__(self):
        return "ConvWgradImplicit{%s}" % (tuple(self.info),)
