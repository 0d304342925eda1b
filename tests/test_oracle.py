"""CPU tests of the oracle itself (no GPU): the restatement in oracle/cgt_oracle.cpp is pinned against

  * the golden vectors in tests/golden/, produced by the reference's own headers (make_golden.py);
  * the reference's own code when oracle/_ref is built (bit-for-bit, random cases);
  * the checks the reference's test-suite makes for this path: conv against scipy
    (cgt/tests/test_conv.py:14-33), im2col/col2im adjointness and pooling / LRN gradients against
    finite differences (cgt/tests/test_imgproc.py:40-97), duplicate-index accumulation
    (cgt/tests/test_inc_subtensor.py:53-71), and the C expression quirks of the elementwise tables.
"""
import glob
import os.path as osp

import numpy as np
import pytest

from oracle import oracle as O

GOLDEN = osp.join(osp.dirname(osp.abspath(__file__)), "golden")


def _geom(a):
    g = [int(v) for v in a]
    return (g[0], g[1]), (g[2], g[3]), (g[4], g[5])


@pytest.mark.parametrize("path", sorted(glob.glob(osp.join(GOLDEN, "im2col_*.npz"))))
def test_golden_im2col(path):
    d = np.load(path)
    k, p, s = _geom(d["geom"])
    assert np.array_equal(O.im2col(d["x"], k, p, s), d["col"])
    assert np.array_equal(O.col2im(d["g"], d["x"].shape, k, p, s), d["im"])


@pytest.mark.parametrize("path", sorted(glob.glob(osp.join(GOLDEN, "pool_*.npz"))))
def test_golden_pool(path):
    d = np.load(path)
    k, p, s = _geom(d["geom"])
    top, mask = O.max_pool(d["x"], k, p, s)
    assert np.array_equal(mask, d["mask"]) and mask.dtype == np.int32
    assert np.array_equal(top, d["top"])
    assert np.array_equal(O.max_pool_pullback(d["x"].shape, mask, d["g"]), d["gx"])


@pytest.mark.parametrize("path", sorted(glob.glob(osp.join(GOLDEN, "lrn_*.npz"))))
def test_golden_lrn(path):
    d = np.load(path)
    size, alpha, beta = int(d["params"][0]), float(d["params"][1]), float(d["params"][2])
    top, scale = O.lrn_forward(d["x"], size, alpha, beta)
    assert np.array_equal(scale, d["scale"]) and np.array_equal(top, d["top"])
    assert np.array_equal(O.lrn_backward(d["x"], top, scale, d["g"], size, alpha, beta), d["gx"])


def test_golden_files_present():
    assert len(glob.glob(osp.join(GOLDEN, "*.npz"))) >= 12


@pytest.mark.skipif(not O.have_ref(), reason="oracle/_ref is built only where the reference tree is present")
@pytest.mark.parametrize("dtype", ["f4", "f8"])
def test_port_matches_reference_code(dtype):
    rs = np.random.RandomState(0)
    x = rs.randn(3, 4, 9, 11).astype(dtype)
    for geo in [((5, 5), (2, 2), (1, 1)), ((3, 3), (1, 1), (2, 2)), ((4, 7), (3, 6), (1, 1)), ((2, 3), (1, 0), (2, 1)),
                ((11, 11), (2, 2), (4, 4))]:
        if x.shape[2] + 2 * geo[1][0] < geo[0][0]:
            continue
        a = O.im2col(x, *geo)
        assert np.array_equal(a, O.im2col(x, *geo, impl="ref"))
        g = rs.randn(*a.shape).astype(dtype)
        assert np.array_equal(O.col2im(g, x.shape, *geo), O.col2im(g, x.shape, *geo, impl="ref"))
    for geo in [((3, 3), (0, 0), (2, 2)), ((4, 4), (0, 0), (1, 1)), ((3, 3), (1, 1), (2, 2)), ((2, 2), (0, 0), (2, 2))]:
        for xx in (x, np.round(x)):
            t, m = O.max_pool(xx, *geo)
            t2, m2 = O.max_pool(xx, *geo, impl="ref")
            assert np.array_equal(t, t2) and np.array_equal(m, m2)
            g = rs.randn(*t.shape).astype(dtype)
            assert np.array_equal(O.max_pool_pullback(x.shape, m, g), O.max_pool_pullback(x.shape, m, g, impl="ref"))
    x = rs.randn(4, 8, 6, 5).astype(dtype)
    for (n, a, b) in [(5, 1e-4, 0.75), (4, .1, .5), (3, 0.5, 1.0), (8, 1.0, 0.75)]:
        t, s = O.lrn_forward(x, n, a, b)
        t2, s2 = O.lrn_forward(x, n, a, b, impl="ref")
        assert np.array_equal(t, t2) and np.array_equal(s, s2)
        g = rs.randn(*x.shape).astype(dtype)
        assert np.array_equal(O.lrn_backward(x, t, s, g, n, a, b), O.lrn_backward(x, t, s, g, n, a, b, impl="ref"))


def test_conv_against_scipy():
    """Im2Col + Mul22(F,T) + reshape/transpose is a cross-correlation (reference test_conv.py)."""
    import scipy.signal
    rs = np.random.RandomState(0)
    x = rs.randn(2, 2, 5, 17)
    filt = rs.randn(3, 2, 4, 7)
    fr, fc = filt.shape[2:]
    want = np.zeros((2, 3, x.shape[2] + fr - 1, x.shape[3] + fc - 1))
    for b in range(2):
        for ic in range(2):
            for oc in range(3):
                want[b, oc] += scipy.signal.convolve2d(x[b, ic], filt[oc, ic][::-1, ::-1], mode="full")
    for (dt, atol) in (("f8", 1e-6), ("f4", 1e-3)):
        col = O.im2col(x.astype(dt), (fr, fc), (fr - 1, fc - 1), (1, 1))
        B, m, n, Z = col.shape
        out = O.mul22(col.reshape(B * m * n, Z), filt.astype(dt).reshape(3, -1), False, True)
        out = O.transpose(out.reshape(B, m, n, 3), [0, 3, 1, 2])
        np.testing.assert_allclose(out, want, atol=atol)


def test_im2col_col2im_adjoint():
    rs = np.random.RandomState(1)
    for (kernel, pad, stride) in [((4, 4), (0, 0), (1, 1)), ((3, 3), (1, 1), (2, 2)), ((3, 3), (1, 1), (3, 3))]:
        x = rs.randn(2, 1, 28, 28)
        col = O.im2col(x, kernel, pad, stride)
        g = rs.randn(*col.shape)
        assert abs((col * g).sum() - (x * O.col2im(g, x.shape, kernel, pad, stride)).sum()) < 1e-9


def _numgrad(f, x, eps):
    g = np.zeros_like(x)
    flat, gf = x.ravel(), g.ravel()
    for i in range(flat.size):
        old = flat[i]
        flat[i] = old + eps
        fp = f(x)
        flat[i] = old - eps
        fm = f(x)
        flat[i] = old
        gf[i] = (fp - fm) / (2 * eps)
    return g


def test_pool_gradient():
    np.random.seed(0)
    x = np.random.randn(2, 3, 5, 7)
    geo = ((4, 4), (0, 0), (1, 1))
    top, mask = O.max_pool(x, *geo)
    assert top.shape == (2, 3, 1, 3)  # iceil((5-4)/1), iceil((7-4)/1): no "+1"
    h = np.random.randn(*top.shape)
    gana = O.max_pool_pullback(x.shape, mask, h)
    gnum = _numgrad(lambda v: (O.max_pool(v, *geo)[0] * h).sum(), x, 1e-6)
    assert np.allclose(gnum, gana)


def test_lrn_gradient_and_window_asymmetry():
    rs = np.random.RandomState(0)
    x = rs.randn(2, 8, 3, 3)
    a = rs.rand(*x.shape)
    for (size, alpha, beta) in [(4, .1, .5), (5, 1e-2, .75)]:
        top, scale = O.lrn_forward(x, size, alpha, beta)
        gana = O.lrn_backward(x, top, scale, a, size, alpha, beta)
        gnum = _numgrad(lambda v: (O.lrn_forward(v, size, alpha, beta)[0] * a).sum(), x, 1e-6)
        assert np.allclose(gnum, gana, atol=1e-7)
    # even window: forward covers [c-1, c+2] (pre=(n-1)/2=1, post=2)
    x = np.zeros((1, 8, 1, 1))
    x[0, 5] = 1.0
    _, scale = O.lrn_forward(x, 4, 4.0, 1.0)
    assert [c for c in range(8) if scale[0, c, 0, 0] != 1.0] == [3, 4, 5, 6]


def test_elementwise_expression_quirks():
    f = np.float32
    assert O.unary("sign", f([0.0, 2.0, -3.0]), "f4").tolist() == [-1.0, 1.0, -1.0]  # 2*(x>0)-1: sign(0) == -1
    assert O.unary("iceil", f([0.5, -2.5, 3.0]), "i8").tolist() == [1, -2, 3]
    assert O.unary("ifloor", f([0.5, -2.5]), "i8").tolist() == [0, -3]
    # sigmoid: exp in float, the division in double, narrowed once
    x = f([0.3, -1.7, 5.0])
    want = (1.0 / (1.0 + np.exp(-x).astype(np.float32).astype(np.float64))).astype(np.float32)
    assert np.array_equal(O.unary("sigmoid", x, "f4"), want)
    # "/" is (x+0.0)/y: integer operands divide in double
    assert O.binary("/", np.int64([1, 7]), np.int64([2, 2]), "f4").tolist() == [0.5, 3.5]
    assert O.binary(">=", f([0.0, -0.0, -1e-30]), np.int64(0), "i1").tolist() == [1, 1, 0]
    # relu as x * (x >= 0): relu(-inf) is NaN
    m = O.binary(">=", f([-np.inf, 1.0]), np.int64(0), "i1")
    with np.errstate(invalid="ignore"):
        r = O.binary("*", f([-np.inf, 1.0]), m, "f4")
    assert np.isnan(r[0]) and r[1] == 1.0
    sp = O.unary("softplus", f([-50.0, 0.0, 50.0]), "f4")
    # log(1+exp(x)) in float: exp(-50) vanishes against 1, exactly as the reference expression does
    np.testing.assert_allclose(sp, [0.0, np.log(2.0), 50.0], rtol=1e-6)


def test_reductions_and_movement():
    rs = np.random.RandomState(2)
    x = rs.randn(3, 4, 5).astype("f4")
    for axes in ([0], [1], [2], [0, 2], [0, 1, 2]):
        np.testing.assert_allclose(O.reduce("sum", x, axes), x.sum(axis=tuple(axes), keepdims=True), rtol=1e-5, atol=1e-6)
        assert np.array_equal(O.reduce("max", x, axes), x.max(axis=tuple(axes), keepdims=True))
    # sequential float32 order: the output is the accumulator, input walked in row-major order
    v = np.float32([1e8, 1.0, -1e8, 1.0])
    assert O.reduce("sum", v, [0])[0] == np.float32(np.float32(np.float32(np.float32(1e8) + 1) - np.float32(1e8)) + 1)
    assert np.array_equal(O.transpose(x, [2, 0, 1]), x.transpose(2, 0, 1))
    assert np.array_equal(O.repeat(x[:, :1], [1], [6]), np.repeat(x[:, :1], 6, 1))
    assert np.array_equal(O.getsli(x, 1, 3, -1, -1), x[:, ::-1])
    assert np.array_equal(O.getsli(x, 2, 1, 5, 2), x[:, :, 1:5:2])
    y = O.incsli(x, 1, 1, 3, 1, np.ones((3, 2, 5), "f4"))
    z = x.copy()
    z[:, 1:3] += 1
    assert np.array_equal(y, z)
    assert np.array_equal(O.concatenate([x, x[:, :2]], 1), np.concatenate([x, x[:, :2]], 1))
    assert np.array_equal(O.arange(2, 11, 3), np.arange(2, 11, 3))
    assert O.fill(3, (2,), "i8").tolist() == [3, 3]


def test_flat_indices_duplicates():
    """Duplicate indices accumulate (reference test_inc_subtensor.py:53-71)."""
    x = np.zeros(5, "i8")
    out = O.incflat(x, np.int64([1, 1, 3, 1]), np.int64([1, 2, 3, 4]))
    assert out.tolist() == [0, 7, 0, 3, 0]
    xf = np.arange(12, dtype="f4").reshape(3, 4)
    assert O.getflat(xf, np.int64([0, 5, 11])).tolist() == [0.0, 5.0, 11.0]


def test_shapes():
    assert O.conv_out_size(32, 5, 2, 1) == 32 and O.conv_out_size(64, 11, 2, 4) == 15
    assert [O.pool_out_size(s, 3, 0, 2) for s in (32, 15, 6)] == [15, 6, 2]  # CIFAR chain 32 -> 15 -> 6 -> 2


def test_sgd_closed_form():
    """Reference golden values for sgd on scale*x^2 from x=1, lr 0.1, 10 steps
    (cgt/tests/test_optimizers.py:8-21): (1 - 0.2*scale)^10."""
    for (scale, want) in zip([0.1, 0.2, 0.3], [0.81707280688755, 0.6648326359915, 0.5386151140949]):
        assert abs((1 - 0.2 * scale) ** 10 - want) < 1e-12
