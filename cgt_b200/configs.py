"""The five benchmark configurations, built through the public API exactly as a user script would.

Each ``build_*`` returns a ``Config`` with the argument nodes, the scalar loss, the parameter list
and the update list; ``Config.compile()`` makes the training-step function (forward + ``cgt.grad``
backward + parameter update) and ``Config.batch(seed)`` draws one synthetic batch of the right
shapes and value ranges. The shapes come from the reference's demo scripts (examples/demo_mnist.py,
demo_cifar.py, demo_char_rnn.py, demo_variational_autoencoder.py); the data are seeded random
tensors, not dataset records.
"""
import numpy as np

from . import core, nn
from .distributions import categorical


def _cgt():
    return core.cgt


class Config(object):
    def __init__(self, name, inputs, loss, params, updates, batch_fn, examples_per_step, extra_outputs=()):
        self.name = name
        self.inputs = inputs
        self.loss = loss
        self.params = params
        self.updates = updates
        self.batch_fn = batch_fn
        self.examples_per_step = examples_per_step
        self.extra_outputs = list(extra_outputs)

    def compile(self):
        return _cgt().function(self.inputs, [self.loss] + self.extra_outputs, updates=self.updates)

    def batch(self, seed=0):
        return self.batch_fn(np.random.RandomState(seed))

    def state_variables(self):
        """Every shared variable of the training step (parameters, optimizer slots, step counters): what a
        checkpoint has to hold."""
        from . import checkpoint
        return checkpoint.state_variables(self.updates, [self.loss] + self.extra_outputs, self.params)


class _seeded(object):
    """Weight initialisers draw from numpy's global RNG (as the reference's do); seed it locally."""

    def __init__(self, seed):
        self.seed = seed

    def __enter__(self):
        self.state = np.random.get_state()
        np.random.seed(self.seed)

    def __exit__(self, *a):
        np.random.set_state(self.state)


def _sgd(loss, params, lr, grad_hook):
    """nn.sgd with an optional transformation of the gradient list (data-parallel averaging)."""
    grads = _cgt().grad(loss, params)
    if grad_hook is not None:
        grads = grad_hook(grads)
    return [(p, p - lr * g) for (p, g) in zip(params, grads)]


def _softmax_ce(logits, y, batch):
    cgt = _cgt()
    logprobs = nn.logsoftmax(logits)
    return -logprobs[cgt.arange(batch), y].mean()


# ------------------------------------------------------------------------------------------------
# C1: MLP 784 -> 256 tanh -> 256 tanh -> 10 softmax
# ------------------------------------------------------------------------------------------------
def build_mlp(batch=128, seed=1, lr=0.1, grad_hook=None):
    cgt = _cgt()
    X = cgt.matrix("X", fixed_shape=(batch, 784))
    y = cgt.vector("y", dtype="i8", fixed_shape=(batch,))
    with _seeded(seed):
        l1 = nn.Affine(784, 256, name="fc1", weight_init=nn.IIDGaussian(std=0.01))
        l2 = nn.Affine(256, 256, name="fc2", weight_init=nn.IIDGaussian(std=0.01))
        l3 = nn.Affine(256, 10, name="fc3", weight_init=nn.IIDGaussian(std=0.01))
    h = cgt.tanh(l1(X))
    h = cgt.tanh(l2(h))
    loss = _softmax_ce(l3(h), y, batch)
    params = nn.get_parameters(loss)
    updates = _sgd(loss, params, lr, grad_hook)

    def batch_fn(rs):
        return [rs.rand(batch, 784).astype("f4"), rs.randint(0, 10, size=batch).astype("i8")]
    return Config("mlp", [X, y], loss, params, updates, batch_fn, batch)


# ------------------------------------------------------------------------------------------------
# C2: CIFAR-shape convnet (the headline configuration)
# ------------------------------------------------------------------------------------------------
def build_cifar(batch=128, seed=1, lr=0.005, grad_hook=None):
    cgt = _cgt()
    X = cgt.tensor4("X", fixed_shape=(batch, 3, 32, 32))
    y = cgt.vector("y", dtype="i8", fixed_shape=(batch,))
    he = nn.HeNormal(scale=float(np.sqrt(2.0)))
    with _seeded(seed):
        conv1 = nn.SpatialConvolution(3, 32, kernelshape=(5, 5), pad=(2, 2), name="conv1", weight_init=he)
        conv2 = nn.SpatialConvolution(32, 32, kernelshape=(5, 5), pad=(2, 2), name="conv2", weight_init=he)
        conv3 = nn.SpatialConvolution(32, 64, kernelshape=(5, 5), pad=(2, 2), name="conv3", weight_init=he)
    h = nn.rectify(conv1(X))
    h = nn.max_pool_2d(h, kernelshape=(3, 3), stride=(2, 2))
    h = nn.cross_channel_lrn(h, 5, 1e-4, 0.75)
    h = nn.rectify(conv2(h))
    h = nn.max_pool_2d(h, kernelshape=(3, 3), stride=(2, 2))
    h = nn.rectify(conv3(h))
    h = nn.max_pool_2d(h, kernelshape=(3, 3), stride=(2, 2))
    d0, d1, d2, d3 = h.shape
    flat = h.reshape([d0, d1 * d2 * d3])
    nfeats = cgt.infer_shape(flat)[1]
    with _seeded(seed + 100):
        ip = nn.Affine(nfeats, 10, name="ip", weight_init=nn.HeNormal(scale=1.0))
    loss = _softmax_ce(ip(flat), y, batch)
    params = nn.get_parameters(loss)
    updates = _sgd(loss, params, lr, grad_hook)

    def batch_fn(rs):
        return [rs.randn(batch, 3, 32, 32).astype("f4"), rs.randint(0, 10, size=batch).astype("i8")]
    return Config("cifar", [X, y], loss, params, updates, batch_fn, batch)


# ------------------------------------------------------------------------------------------------
# C5: wide conv stack (128 examples per GPU)
# ------------------------------------------------------------------------------------------------
def build_wide(batch=128, seed=1, lr=0.0005, grad_hook=None):
    cgt = _cgt()
    X = cgt.tensor4("X", fixed_shape=(batch, 3, 64, 64))
    y = cgt.vector("y", dtype="i8", fixed_shape=(batch,))
    he = nn.HeNormal(scale=float(np.sqrt(2.0)))
    with _seeded(seed):
        conv1 = nn.SpatialConvolution(3, 96, kernelshape=(11, 11), pad=(2, 2), stride=(4, 4), name="conv1", weight_init=he)
        conv2 = nn.SpatialConvolution(96, 256, kernelshape=(5, 5), pad=(2, 2), name="conv2", weight_init=he)
    h = nn.rectify(conv1(X))
    h = nn.cross_channel_lrn(h, 5, 1e-4, 0.75)
    h = nn.max_pool_2d(h, kernelshape=(3, 3), stride=(2, 2))
    h = nn.rectify(conv2(h))
    h = nn.max_pool_2d(h, kernelshape=(3, 3), stride=(2, 2))
    d0, d1, d2, d3 = h.shape
    flat = h.reshape([d0, d1 * d2 * d3])
    nfeats = cgt.infer_shape(flat)[1]
    with _seeded(seed + 100):
        fc1 = nn.Affine(nfeats, 4096, name="fc1", weight_init=he)
        fc2 = nn.Affine(4096, 100, name="fc2", weight_init=nn.HeNormal(scale=1.0))
    h = nn.rectify(fc1(flat))
    loss = _softmax_ce(fc2(h), y, batch)
    params = nn.get_parameters(loss)
    updates = _sgd(loss, params, lr, grad_hook)

    def batch_fn(rs):
        return [rs.randn(batch, 3, 64, 64).astype("f4"), rs.randint(0, 100, size=batch).astype("i8")]
    return Config("wide", [X, y], loss, params, updates, batch_fn, batch)


# ------------------------------------------------------------------------------------------------
# C3: two-layer char-level LSTM, unrolled, with gradient clipping at a global norm
# ------------------------------------------------------------------------------------------------
def build_lstm(vocab=65, hidden=128, n_layers=2, seq_len=50, batch=64, seed=1, lr=0.1, clip=5.0):
    cgt = _cgt()
    x_tnk = cgt.tensor3("x", fixed_shape=(seq_len, batch, vocab))
    targ_tnk = cgt.tensor3("targ", fixed_shape=(seq_len, batch, vocab))
    uni = nn.IIDUniform(-0.08, 0.08)
    with _seeded(seed):
        layers = []
        for i in range(n_layers):
            size_x = vocab if i == 0 else hidden
            layers.append((nn.Affine(size_x, 4 * hidden, name="l%d.x2h" % i, weight_init=uni),
                           nn.Affine(hidden, 4 * hidden, name="l%d.h2h" % i, weight_init=uni)))
        pred = nn.Affine(hidden, vocab, name="pred", weight_init=uni)
    hs = [cgt.zeros((batch, hidden)) for _ in range(n_layers)]
    cs = [cgt.zeros((batch, hidden)) for _ in range(n_layers)]
    loss = 0
    for t in range(seq_len):
        x = x_tnk[t]
        for i in range(n_layers):
            x2h, h2h = layers[i]
            input_sums = x2h(x) + h2h(hs[i])
            sigmoid_chunk = cgt.sigmoid(input_sums[:, 0:3 * hidden])
            in_gate = sigmoid_chunk[:, 0:hidden]
            forget_gate = sigmoid_chunk[:, hidden:2 * hidden]
            out_gate = sigmoid_chunk[:, 2 * hidden:3 * hidden]
            in_transform = cgt.tanh(input_sums[:, 3 * hidden:4 * hidden])
            cs[i] = forget_gate * cs[i] + in_gate * in_transform
            hs[i] = out_gate * cgt.tanh(cs[i])
            x = hs[i]
        logprobs = nn.logsoftmax(pred(x))
        loss = loss - (logprobs * targ_tnk[t]).sum()
    loss = loss / (seq_len * batch)
    params = nn.get_parameters(loss)
    grads = cgt.grad(loss, params)
    # global-norm clipping with comparison masks (there is no min/clip Op): the factor is a host scalar
    sqnorm = cgt.add_multi([cgt.square(g).sum() for g in grads])
    gnorm = cgt.sqrt(sqnorm)
    factor = (gnorm > clip) * (clip / gnorm) + (gnorm <= clip)
    updates = [(p, p - lr * (g * factor)) for (p, g) in zip(params, grads)]

    def batch_fn(rs):
        def onehot():
            idx = rs.randint(0, vocab, size=(seq_len, batch))
            out = np.zeros((seq_len, batch, vocab), "f4")
            out[np.arange(seq_len)[:, None], np.arange(batch)[None, :], idx] = 1
            return out
        return [onehot(), onehot()]
    return Config("lstm", [x_tnk, targ_tnk], loss, params, updates, batch_fn, batch, extra_outputs=[gnorm])


# ------------------------------------------------------------------------------------------------
# C4: variational autoencoder 784 -> 500 softplus -> (mu, logvar) 20 -> 500 softplus -> 784 sigmoid
# ------------------------------------------------------------------------------------------------
def build_vae(batch=100, xdim=784, hdim=500, zdim=20, seed=1, lr=0.001):
    cgt = _cgt()
    x = cgt.matrix("x", fixed_shape=(batch, xdim))
    eps = cgt.matrix("eps", fixed_shape=(batch, zdim))
    g = nn.IIDGaussian(std=0.01)
    with _seeded(seed):
        enc_h = nn.Affine(xdim, hdim, name="enc_h", weight_init=g)
        enc_mu = nn.Affine(hdim, zdim, name="enc_mu", weight_init=g)
        enc_lv = nn.Affine(hdim, zdim, name="enc_logvar", weight_init=g)
        dec_h = nn.Affine(zdim, hdim, name="dec_h", weight_init=g)
        dec_o = nn.Affine(hdim, xdim, name="dec_out", weight_init=g)
    h = nn.softplus(enc_h(x))
    mu = enc_mu(h)
    logvar = enc_lv(h)
    sigma = cgt.sqrt(cgt.exp(logvar))
    z = mu + sigma * eps
    out = cgt.sigmoid(dec_o(nn.softplus(dec_h(z))))
    recon = cgt.sum(nn.binary_crossentropy(out, x))
    kl = -0.5 * cgt.sum(1 + logvar - cgt.square(mu) - cgt.exp(logvar))
    loss = (recon + kl) / batch
    params = nn.get_parameters(loss)
    updates = nn.adam(loss, params, learning_rate=lr)

    def batch_fn(rs):
        return [(rs.rand(batch, xdim) < 0.13).astype("f4"), rs.randn(batch, zdim).astype("f4")]
    return Config("vae", [x, eps], loss, params, updates, batch_fn, batch)


BUILDERS = {"mlp": build_mlp, "cifar": build_cifar, "lstm": build_lstm, "vae": build_vae, "wide": build_wide}
