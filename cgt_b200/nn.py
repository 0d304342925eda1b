"""Neural-network helpers expressed as graph ops (counterpart of the reference's cgt/nn.py):
layers, initialisers and optimisers. On this backend ``conv2d`` and ``max_pool_2d`` always use the
im2col + Mul22 and MaxPool Ops (the formulation of the reference's CPU backend, cgt/nn.py:93-100,
110-111), executed on the GPU.
"""
from collections import namedtuple

import numpy as np

from . import core
from .nn_ops.im2col import im2col
from .nn_ops.cross_channel_lrn import cross_channel_lrn  # noqa: F401  (re-exported)
from .nn_ops.max_pool_2d import MaxPool, PoolInfo


def _cgt():
    return core.cgt


def is_parameter(node):
    return node.is_data() and node.props.get("is_parameter", False)


def get_parameters(loss):
    return [node for node in core.topsorted([loss]) if is_parameter(node)]


def parameter(val, name=None, device=None):
    out = _cgt().shared(val, name=name, device=device, fixed_shape_mask="all")
    out.props["is_parameter"] = True
    return out


# ---------------------------------------------------------------- math
def rectify(x):
    """x * (x >= 0): an int8 mask times x (cgt/nn.py:44-45)."""
    return x * (x >= 0)


def _nu_softplus(x, out=None):
    x = np.asarray(x)
    absx = np.abs(x)
    r = (absx + x) / 2 + np.log(1 + np.exp(-absx))
    if out is None:
        return r
    out[...] = r


def softplus(x):
    op = core.ElwiseUnary("softplus", core.UnaryInfo(
        "SoftPlus", _nu_softplus, True, "f", lambda x, g, gy: gy / (_cgt().exp(-x) + 1.0),
        "(x > 0) ? (x + log(exp(-x) + 1)) : log(1+exp(x))"))
    return core.Result(op, [x])


def softmax(x, axis=1):
    """exp(x) / sum(exp(x)) with no max-shift, as the reference computes it (cgt/nn.py:55-59)."""
    cgt = _cgt()
    out = cgt.exp(x)
    return cgt.broadcast("/", out, out.sum(axis=axis, keepdims=True), "xx,x1")


def logsoftmax(x, axis=1):
    return _cgt().log(softmax(x, axis=axis))


def binary_crossentropy(x, y):
    cgt = _cgt()
    return -(y * cgt.log(x) + (1 - y) * cgt.log(1 - x))


# ---------------------------------------------------------------- image ops
def conv2d(x_BKRC, f_LKrc, kernelshape, pad=(0, 0), stride=(1, 1)):
    """Cross-correlation as Im2Col -> Mul22(F,T) -> reshape -> Transpose{0,3,1,2} (cgt/nn.py:93-100)."""
    L, K, r, c = f_LKrc.shape
    col_BmnZ = im2col(x_BKRC, kernelshape, pad, stride)
    f_LZ = f_LKrc.reshape([L, K * r * c])
    B, m, n, Z = col_BmnZ.shape
    col_Bmn_Z = col_BmnZ.reshape([B * m * n, Z])
    col_Bmn_L = core.Result(core.Mul22(False, True), [col_Bmn_Z, f_LZ])
    return col_Bmn_L.reshape([B, m, n, L]).transpose([0, 3, 1, 2])


def max_pool_2d(x, kernelshape, pad=(0, 0), stride=(1, 1)):
    kernel_h, kernel_w = kernelshape
    pad_h, pad_w = pad
    stride_h, stride_w = stride
    info = PoolInfo(kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w)
    return core.Result(MaxPool(info), [x])[0]


# ---------------------------------------------------------------- initialisers
IIDGaussian = namedtuple("IIDGaussian", ["mean", "std"])
IIDGaussian.__new__.__defaults__ = (0, 1)
IIDUniform = namedtuple("IIDUniform", ["low", "high"])
Constant = namedtuple("Constant", ["constant"])
XavierNormal = namedtuple("XavierNormal", ["scale"])
XavierUniform = namedtuple("XavierUniform", ["scale"])
XavierNormal.__new__.__defaults__ = (1,)
XavierUniform.__new__.__defaults__ = (1,)
HeNormal = namedtuple("HeNormal", ["scale"])
HeUniform = namedtuple("HeUniform", ["scale"])


def init_array(init, shape):
    """Draws from the global numpy RNG, like the reference (cgt/nn.py:130-158)."""
    floatX = _cgt().floatX
    if isinstance(init, IIDGaussian):
        return (np.random.randn(*shape) * init.std + init.mean).astype(floatX)
    elif isinstance(init, IIDUniform):
        return (np.random.rand(*shape) * (init.high - init.low) + init.low).astype(floatX)
    elif isinstance(init, Constant):
        return init.constant * np.ones(shape, floatX)
    elif isinstance(init, XavierNormal):
        return (np.random.randn(*shape) * get_xavier_weight(init, shape)).astype(floatX)
    elif isinstance(init, XavierUniform):
        std = get_xavier_weight(init, shape)
        high, low = -np.sqrt(3) * std, np.sqrt(3) * std
        return (np.random.rand(*shape) * (high - low) + low).astype(floatX)
    elif isinstance(init, HeNormal):
        return (np.random.randn(*shape) * get_he_weight(init, shape)).astype(floatX)
    elif isinstance(init, HeUniform):
        std = get_he_weight(init, shape)
        low, high = -np.sqrt(3) * std, np.sqrt(3) * std
        return (np.random.rand(*shape) * (high - low) + low).astype(floatX)
    raise ValueError("Invalid initializer %s" % (init,))


def get_xavier_weight(init, shape):
    if len(shape) < 2:
        raise RuntimeError("Shape length must at least 2")
    n1, n2 = shape[:2]
    field_size = np.prod(shape[2:])
    return init.scale * np.sqrt(2.0 / ((n1 + n2) * field_size))


def get_he_weight(init, shape):
    """std = scale * sqrt(1 / fan_in); fan_in = shape[0] for matrices, prod(shape[1:]) otherwise."""
    if len(shape) == 2:
        fan_in = shape[0]
    elif len(shape) > 2:
        fan_in = np.prod(shape[1:])
    else:
        raise RuntimeError("This initializer does not work with shapes of length less than two")
    return init.scale * np.sqrt(1.0 / fan_in)


# ---------------------------------------------------------------- layers
class Affine(object):
    """x.dot(W) + b with b stored as [1, n] and broadcast by Repeat (cgt/nn.py:198-213)."""

    def __init__(self, input_size, output_size, name=None, weight_init=Constant(0), bias_init=Constant(0)):
        input_size, output_size = int(input_size), int(output_size)
        name = "unnamed" if name is None else name
        self.weight = parameter(init_array(weight_init, (input_size, output_size)), name=name + ".W")
        self.bias = parameter(init_array(bias_init, (1, output_size)), name=name + ".b")

    def __call__(self, x):
        return _cgt().broadcast("+", x.dot(self.weight), self.bias, "xx,1x")


class SpatialConvolution(object):
    def __init__(self, input_channels, output_channels, kernelshape, pad, stride=(1, 1), name=None,
                 weight_init=Constant(0), bias_init=Constant(0)):
        input_channels, output_channels = int(input_channels), int(output_channels)
        self.kernelshape = tuple(map(int, kernelshape))
        self.pad = tuple(map(int, pad))
        self.stride = tuple(map(int, stride))
        name = "unnamed" if name is None else name
        self.weight = parameter(init_array(weight_init, (output_channels, input_channels) + self.kernelshape),
                                name=name + ".W")
        self.bias = parameter(init_array(bias_init, (1, output_channels, 1, 1)), name=name + ".b")

    def __call__(self, x):
        tmp = conv2d(x, self.weight, self.kernelshape, self.pad, self.stride)
        return _cgt().broadcast("+", tmp, self.bias, "xxxx,1x11")


# ---------------------------------------------------------------- optimisers (update lists for cgt.function)
def sgd(cost, params, learning_rate):
    """param := param - learning_rate * grad"""
    grads = _cgt().grad(cost, params)
    return [(param, param - learning_rate * grad) for (param, grad) in zip(params, grads)]


def _zeros_like_param(param):
    assert isinstance(param.op, core.GetData)
    return _cgt().shared(np.zeros(param.op.get_shape(), dtype=param.dtype), fixed_shape_mask="all")


def momentum(cost, params, learning_rate, mu=0.9):
    updates = []
    grads = _cgt().grad(cost, params)
    for param, grad in zip(params, grads):
        velocity = _zeros_like_param(param)
        new_velocity = mu * velocity - learning_rate * grad
        updates.append((velocity, new_velocity))
        updates.append((param, param + new_velocity))
    return updates


def nesterov_momentum(cost, params, learning_rate, mu=0.9):
    updates = []
    grads = _cgt().grad(cost, params)
    for param, grad in zip(params, grads):
        velocity = _zeros_like_param(param)
        new_velocity = mu * velocity - learning_rate * grad
        updates.append((velocity, new_velocity))
        updates.append((param, param - mu * velocity + (mu + 1) * new_velocity))
    return updates


def adagrad(cost, params, learning_rate=1.0, epsilon=1e-6):
    cgt = _cgt()
    updates = []
    grads = cgt.grad(cost, params)
    for param, grad in zip(params, grads):
        accu = _zeros_like_param(param)
        accu_new = accu + grad ** 2
        updates.append((accu, accu_new))
        updates.append((param, param - (learning_rate * grad) / cgt.sqrt(accu_new + epsilon)))
    return updates


def rmsprop(cost, params, learning_rate=1.0, rho=0.9, epsilon=1e-6):
    cgt = _cgt()
    updates = []
    grads = cgt.grad(cost, params)
    for param, grad in zip(params, grads):
        accu = _zeros_like_param(param)
        accu_new = rho * accu + (1 - rho) * grad ** 2
        updates.append((accu, accu_new))
        updates.append((param, param - (learning_rate * grad / cgt.sqrt(accu_new + epsilon))))
    return updates


def adadelta(cost, params, learning_rate=1.0, rho=0.95, epsilon=1e-6):
    cgt = _cgt()
    updates = []
    grads = cgt.grad(cost, params)
    for param, grad in zip(params, grads):
        accu = _zeros_like_param(param)
        delta_accu = _zeros_like_param(param)
        accu_new = rho * accu + (1 - rho) * grad ** 2
        updates.append((accu, accu_new))
        update = grad * cgt.sqrt(delta_accu + epsilon) / cgt.sqrt(accu_new + epsilon)
        updates.append((param, param - learning_rate * update))
        delta_accu_new = rho * delta_accu + (1 - rho) * update ** 2
        updates.append((delta_accu, delta_accu_new))
    return updates


def adam(cost, params, learning_rate=0.001, beta1=0.9, beta2=0.999, epsilon=1e-8):
    """Adam built from elementwise graph ops. The reference holds only a golden-value key for it
    (cgt/tests/test_optimizers.py:20) and no implementation; the VAE configuration needs one.
    The step counter is a shared scalar-like [1] array so the bias corrections stay on the device."""
    cgt = _cgt()
    updates = []
    grads = cgt.grad(cost, params)
    t_prev = cgt.shared(np.zeros((1,), dtype=cgt.floatX), fixed_shape_mask="all")
    t = t_prev + 1
    updates.append((t_prev, t))
    b1t = cgt.exp(t * float(np.log(beta1)))   # beta1 ** t
    b2t = cgt.exp(t * float(np.log(beta2)))
    a_t = learning_rate * cgt.sqrt(1 - b2t) / (1 - b1t)   # shape [1]
    for param, grad in zip(params, grads):
        m_prev = _zeros_like_param(param)
        v_prev = _zeros_like_param(param)
        m_t = beta1 * m_prev + (1 - beta1) * grad
        v_t = beta2 * v_prev + (1 - beta2) * cgt.square(grad)
        pat = "1" * param.ndim + "," + "x" * param.ndim
        a_full = a_t.reshape([1] * param.ndim)
        step = cgt.broadcast("*", a_full, m_t / (cgt.sqrt(v_t) + epsilon), pat)
        updates.append((m_prev, m_t))
        updates.append((v_prev, v_t))
        updates.append((param, param - step))
    return updates
