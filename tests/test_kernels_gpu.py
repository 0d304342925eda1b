"""GPU parity: every kernel of the C ABI against the CPU oracle on the same seeded inputs.

Integer / index outputs (pool argmax mask, comparisons, casts to int, gathers) must be bit-exact.
Float outputs of order-dependent sums that the kernels reproduce in the reference's order (pool
pullback, col2im) must be bit-exact too. Other float outputs: rtol 1e-4, atol 1e-5.
"""
import ctypes

import numpy as np
import pytest

from cgt_b200 import runtime
from oracle import oracle as O
from tests.gpu_util import Dev, call, code, ints, longs

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-4, 1e-5

GEOMS = [
    # (x shape, kernel, pad, stride)
    ((2, 2, 5, 17), (4, 7), (3, 6), (1, 1)),     # reference test_conv.py
    ((2, 1, 28, 28), (4, 4), (0, 0), (1, 1)),    # reference test_imgproc.py test_im2col
    ((2, 1, 28, 28), (3, 3), (1, 1), (2, 2)),
    ((2, 1, 28, 28), (3, 3), (1, 1), (3, 3)),
    ((3, 3, 32, 32), (5, 5), (2, 2), (1, 1)),    # CIFAR conv1 geometry
    ((2, 32, 15, 15), (5, 5), (2, 2), (1, 1)),   # CIFAR conv2 geometry
    ((2, 3, 64, 64), (11, 11), (2, 2), (4, 4)),  # wide conv1 geometry
    ((1, 2, 7, 9), (2, 3), (1, 0), (2, 1)),      # ragged
    ((1, 1, 3, 3), (3, 3), (0, 0), (1, 1)),      # single output pixel
]


@pytest.mark.parametrize("shape,kernel,pad,stride", GEOMS)
@pytest.mark.parametrize("dtype", ["f4", "f8"])
def test_im2col_col2im(rt, shape, kernel, pad, stride, dtype):
    rs = np.random.RandomState(0)
    x = rs.randn(*shape).astype(dtype)
    want = O.im2col(x, kernel, pad, stride)
    dx, dcol = Dev(x), Dev(shape=want.shape, dtype=dtype)
    B, C, H, W = shape
    call("cgtb_im2col", code(dtype), dx.ptr, B, C, H, W, kernel[0], kernel[1], pad[0], pad[1], stride[0], stride[1], dcol.ptr)
    assert np.array_equal(dcol.get(), want)  # a copy with zero fill: exact
    g = rs.randn(*want.shape).astype(dtype)
    want_im = O.col2im(g, shape, kernel, pad, stride)
    dg, dim = Dev(g), Dev(shape=shape, dtype=dtype)
    call("cgtb_col2im", code(dtype), dg.ptr, B, C, H, W, kernel[0], kernel[1], pad[0], pad[1], stride[0], stride[1], dim.ptr)
    assert np.array_equal(dim.get(), want_im)  # same accumulation order as the CPU loop: exact


@pytest.mark.parametrize("shape,kernel,pad,stride,pitch", [
    ((3, 3, 32, 32), (5, 5), (2, 2), (1, 1), 76),     # CIFAR conv1: rows of 75 widened to 16-byte multiples
    ((2, 3, 64, 64), (11, 11), (2, 2), (4, 4), 364),  # wide conv1: 363 -> 364
    ((2, 3, 9, 11), (3, 3), (1, 1), (2, 2), 28),
    ((2, 3, 9, 11), (3, 3), (1, 1), (2, 2), 33),      # a pitch that is not a multiple of four: scalar stores
    ((1, 2, 7, 9), (2, 3), (1, 0), (2, 1), 12),       # pitch == row length
])
@pytest.mark.parametrize("dtype", ["f4", "f8"])
def test_im2col_padded_rows(rt, shape, kernel, pad, stride, pitch, dtype):
    """cgtb_im2col_ld: the column rows lie `pitch` entries apart, the entries beyond C*kh*kw are zero."""
    rs = np.random.RandomState(2)
    x = rs.randn(*shape).astype(dtype)
    ref = O.im2col(x, kernel, pad, stride)
    want = np.zeros(ref.shape[:3] + (pitch,), dtype)
    want[..., :ref.shape[3]] = ref
    dx, dcol = Dev(x), Dev(np.full(want.shape, 7, dtype))
    B, C, H, W = shape
    L = runtime.lib()
    L.cgtb_im2col_ld.restype = ctypes.c_int
    L.cgtb_im2col_ld.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_long] + [ctypes.c_int] * 9 + [ctypes.c_long, ctypes.c_void_p]
    call("cgtb_im2col_ld", code(dtype), dx.ptr, B, C, H, W, kernel[0], kernel[1], pad[0], pad[1], stride[0], stride[1], pitch, dcol.ptr)
    assert np.array_equal(dcol.get(), want)
    assert L.cgtb_im2col_ld(code(dtype), dx.ptr, B, C, H, W, kernel[0], kernel[1], pad[0], pad[1], stride[0], stride[1],
                            ref.shape[3] - 1, dcol.ptr) != 0  # a pitch below the row length is refused


POOLS = [
    ((2, 3, 5, 7), (4, 4), (0, 0), (1, 1)),      # reference test_imgproc.py test_pool
    ((4, 32, 32, 32), (3, 3), (0, 0), (2, 2)),   # CIFAR pool1
    ((4, 32, 15, 15), (3, 3), (0, 0), (2, 2)),
    ((4, 64, 6, 6), (3, 3), (0, 0), (2, 2)),
    ((2, 3, 9, 11), (3, 3), (1, 1), (2, 2)),     # padded
    ((2, 2, 8, 8), (2, 2), (0, 0), (2, 2)),      # non-overlapping
    ((2, 3, 12, 12), (3, 3), (1, 1), (2, 2)),    # padded, row length a multiple of four (four pixels per thread)
    ((2, 3, 8, 4), (2, 2), (1, 1), (2, 2)),
    ((1, 1, 6, 6), (3, 2), (1, 0), (1, 2)),
]


@pytest.mark.parametrize("shape,kernel,pad,stride", POOLS)
@pytest.mark.parametrize("dtype", ["f4", "f8"])
@pytest.mark.parametrize("ties", [False, True])
def test_max_pool(rt, shape, kernel, pad, stride, dtype, ties):
    rs = np.random.RandomState(1)
    x = rs.randn(*shape).astype(dtype)
    if ties:  # many equal values: the first maximum in scan order must win
        x = np.round(x).astype(dtype)
    top, mask = O.max_pool(x, kernel, pad, stride)
    B, C, H, W = shape
    PH, PW = top.shape[2:]
    dx, dtop, dmask = Dev(x), Dev(shape=top.shape, dtype=dtype), Dev(shape=mask.shape, dtype="i4")
    call("cgtb_max_pool", code(dtype), dx.ptr, B, C, H, W, kernel[0], kernel[1], pad[0], pad[1], stride[0], stride[1], PH, PW,
         dtop.ptr, dmask.ptr)
    assert np.array_equal(dmask.get(), mask)
    assert np.array_equal(dtop.get(), top)
    g = rs.randn(*top.shape).astype(dtype)
    want = O.max_pool_pullback(shape, mask, g)
    dg, dgx = Dev(g), Dev(shape=shape, dtype=dtype)
    call("cgtb_max_pool_pullback", code(dtype), dmask.ptr, dg.ptr, B, C, PH, PW, H, W, kernel[0], kernel[1], pad[0], pad[1],
         stride[0], stride[1], dgx.ptr)
    assert np.array_equal(dgx.get(), want)


def test_max_pool_nan_window(rt):
    """A window of NaNs keeps (-FLT_MAX, -1); the pullback must not scatter through the -1."""
    x = np.full((1, 1, 4, 4), np.nan, "f4")
    top, mask = O.max_pool(x, (2, 2), (0, 0), (2, 2))
    dx, dtop, dmask = Dev(x), Dev(shape=top.shape, dtype="f4"), Dev(shape=mask.shape, dtype="i4")
    call("cgtb_max_pool", code("f4"), dx.ptr, 1, 1, 4, 4, 2, 2, 0, 0, 2, 2, 2, 2, dtop.ptr, dmask.ptr)
    assert np.array_equal(dmask.get(), mask) and (mask == -1).all()
    assert np.array_equal(dtop.get(), top)
    dg, dgx = Dev(np.ones_like(top)), Dev(shape=x.shape, dtype="f4")
    call("cgtb_max_pool_pullback", code("f4"), dmask.ptr, dg.ptr, 1, 1, 2, 2, 4, 4, 2, 2, 0, 0, 2, 2, dgx.ptr)
    assert np.array_equal(dgx.get(), np.zeros_like(x))


LRNS = [
    ((4, 8, 16, 16), 4, 0.1, 0.5),       # reference test_imgproc.py test_lrn
    ((4, 32, 15, 15), 5, 1e-4, 0.75),    # CIFAR
    ((2, 96, 15, 15), 5, 1e-4, 0.75),    # wide
    ((2, 5, 3, 3), 5, 1.0, 0.75),        # channels == localsize
    ((2, 7, 2, 3), 3, 0.5, 1.0),
    ((3, 40, 9, 9), 5, 1e-2, 0.75),      # more channels than one pass of the staged kernel covers (odd plane size)
    ((2, 130, 8, 8), 7, 1e-2, 0.75),     # the same with 128-bit accesses
    ((130, 32, 6, 6), 5, 1e-4, 0.75),    # plane smaller than a pixel tile
]


@pytest.mark.parametrize("shape,size,alpha,beta", LRNS)
@pytest.mark.parametrize("dtype", ["f4", "f8"])
def test_lrn(rt, shape, size, alpha, beta, dtype):
    rs = np.random.RandomState(2)
    x = rs.randn(*shape).astype(dtype)
    top, scale = O.lrn_forward(x, size, alpha, beta)
    N, C, H, W = shape
    dx, dtop, dscale = Dev(x), Dev(shape=shape, dtype=dtype), Dev(shape=shape, dtype=dtype)
    call("cgtb_lrn_forward", code(dtype), dx.ptr, N, C, H, W, size, alpha, beta, dtop.ptr, dscale.ptr)
    np.testing.assert_allclose(dscale.get(), scale, rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(dtop.get(), top, rtol=RTOL, atol=ATOL)
    g = rs.randn(*shape).astype(dtype)
    want = O.lrn_backward(x, top, scale, g, size, alpha, beta)
    dt, ds, dg, dgx = Dev(top), Dev(scale), Dev(g), Dev(shape=shape, dtype=dtype)
    call("cgtb_lrn_backward", code(dtype), dx.ptr, dt.ptr, ds.ptr, dg.ptr, N, C, H, W, size, alpha, beta, dgx.ptr)
    np.testing.assert_allclose(dgx.get(), want, rtol=RTOL, atol=ATOL)


UNARY_CASES = [
    ("abs", "f4", "f4"), ("ceil", "f4", "i8"), ("cos", "f4", "f4"), ("exp", "f4", "f4"), ("iceil", "f4", "i8"),
    ("ifloor", "f4", "i8"), ("log", "f4", "f4"), ("neg", "f4", "f4"), ("sign", "f4", "f4"), ("sin", "f4", "f4"),
    ("square", "f4", "f4"), ("sqrt", "f4", "f4"), ("tanh", "f4", "f4"), ("sigmoid", "f4", "f4"), ("softplus", "f4", "f4"),
    ("cast", "i1", "f4"), ("cast", "i8", "f4"), ("cast", "f4", "i8"), ("cast", "f4", "f8"), ("cast", "i4", "i8"),
    ("neg", "i8", "i8"), ("square", "i8", "i8"), ("exp", "f8", "f8"), ("sigmoid", "f8", "f8"), ("sign", "i8", "i8"),
]


@pytest.mark.parametrize("op,dt_in,dt_out", UNARY_CASES)
@pytest.mark.parametrize("n", [1, 5, 1000, 40003])
def test_unary(rt, op, dt_in, dt_out, n):
    rs = np.random.RandomState(3)
    if np.dtype(dt_in).kind == "f":
        x = (rs.randn(n) * 3).astype(dt_in)
        if op in ("log", "sqrt"):
            x = np.abs(x) + 0.01
        x[:1] = 0  # sign(0) == -1 and friends
    else:
        x = rs.randint(-100, 100, size=n).astype(dt_in)
    want = O.unary(op, x, dt_out)
    dx, dout = Dev(x), Dev(shape=(n,), dtype=dt_out)
    call("cgtb_unary", O.UNARY[op], code(dt_in), code(dt_out), n, dx.ptr, dout.ptr)
    got = dout.get()
    if np.dtype(dt_out).kind == "i" or op in ("abs", "neg", "sign", "square", "cast", "ceil", "sqrt"):
        assert np.array_equal(got, want)
    else:
        np.testing.assert_allclose(got, want, rtol=RTOL, atol=ATOL)


BINARY_CASES = [
    ("*", "f4", "f4", "f4"), ("+", "f4", "f4", "f4"), ("-", "f4", "f4", "f4"), ("/", "f4", "f4", "f4"),
    ("<", "f4", "f4", "i1"), (">", "f4", "f4", "i1"), ("<=", "f4", "f4", "i1"), (">=", "f4", "f4", "i1"),
    ("**", "f4", "f4", "f4"), ("==", "f4", "f4", "i1"), ("!=", "f4", "f4", "i1"),
    ("*", "f4", "i1", "f4"), ("*", "i8", "i8", "i8"), ("+", "i8", "i8", "i8"), ("/", "i8", "i8", "f4"),
    (">=", "f4", "i8", "i1"), ("/", "f4", "i8", "f4"), ("*", "f8", "f8", "f8"), ("-", "i8", "f4", "f4"),
    ("**", "f4", "i8", "f4"), ("==", "i8", "i8", "i1"),
]


@pytest.mark.parametrize("op,dtx,dty,dto", BINARY_CASES)
@pytest.mark.parametrize("mode", ["tt", "ts", "st"])
@pytest.mark.parametrize("n", [1, 7, 4099])
def test_binary(rt, op, dtx, dty, dto, mode, n):
    rs = np.random.RandomState(4)

    def draw(dt, size):
        if np.dtype(dt).kind == "f":
            v = np.asarray(rs.randn(*size) * 2)
            if op == "**":
                v = np.abs(v) + 0.1
            return v.astype(dt)
        v = np.asarray(rs.randint(-5, 6, size=size))
        if op in ("/", "**"):
            v = np.abs(v) + 1
        return v.astype(dt)
    x = draw(dtx, () if mode == "st" else (n,))
    y = draw(dty, () if mode == "ts" else (n,))
    if op in ("==", "!=", ">=", "<=") and mode == "tt":
        y[::3] = x[::3].astype(dty)  # make equality happen
    want = O.binary(op, x, y, dto)
    dx, dy, dout = Dev(x), Dev(y), Dev(shape=(n,), dtype=dto)
    call("cgtb_binary", O.BINARY[op], code(dtx), code(dty), code(dto), n, dx.ptr, dy.ptr, dout.ptr, int(mode == "st"),
         int(mode == "ts"))
    got = dout.get()
    if np.dtype(dto).kind == "i" or op in ("*", "+", "-", "/"):
        assert np.array_equal(got, want)  # IEEE basic operations: exact
    else:
        np.testing.assert_allclose(got, want, rtol=RTOL, atol=ATOL)


REDUCE_CASES = [
    ((128, 10), [1]), ((128, 10), [0]), ((128,), [0]), ((8, 32, 9, 9), [0, 2, 3]), ((100, 784), [1]), ((100, 20), [0, 1]),
    ((3, 1, 5), [1]), ((2, 3, 4, 5), [1, 3]), ((64, 2048), [0, 1]), ((5, 70000), [1]), ((1,), [0]),
]


@pytest.mark.parametrize("shape,axes", REDUCE_CASES)
@pytest.mark.parametrize("kind", ["sum", "max"])
@pytest.mark.parametrize("dtype", ["f4", "f8", "i8"])
def test_reduce(rt, shape, axes, kind, dtype):
    rs = np.random.RandomState(5)
    x = rs.randn(*shape).astype(dtype) if dtype != "i8" else rs.randint(-50, 50, size=shape).astype("i8")
    want = O.reduce(kind, x, axes)
    dx, dout = Dev(x), Dev(shape=want.shape, dtype=dtype)
    red = [1 if i in axes else 0 for i in range(len(shape))]
    call("cgtb_reduce", {"sum": 0, "max": 1}[kind], code(dtype), len(shape), longs(shape), ints(red), dx.ptr, dout.ptr)
    got = dout.get()
    if kind == "max" or dtype == "i8":
        assert np.array_equal(got, want)
    else:
        # a parallel sum cannot follow the sequential fp32 order; both are compared with float64
        exact = x.astype("f8").sum(axis=tuple(axes), keepdims=True)
        n = x.size / max(want.size, 1)
        tol = 1e-4 * np.abs(exact) + 1e-5 * max(1.0, np.sqrt(n))
        assert (np.abs(got - exact) <= tol).all()
        assert np.abs(got - exact).max() <= 2 * np.abs(want - exact).max() + 1e-5 * max(1.0, np.sqrt(n))


def test_repeat_transpose_slices(rt):
    rs = np.random.RandomState(6)
    for dtype in ("f4", "i8", "i1", "f8"):
        # Repeat: bias [1,L,1,1] -> [B,L,m,n] and [1,n] -> [B,n]
        for (shape, axes, reps) in [((1, 5, 1, 1), [0, 2, 3], [3, 4, 6]), ((1, 7), [0], [9]), ((3, 1), [1], [5]), ((1, 1), [0, 1], [2, 3])]:
            x = (rs.randn(*shape) * 10).astype(dtype)
            want = O.repeat(x, axes, reps)
            dx, dout = Dev(x), Dev(shape=want.shape, dtype=dtype)
            call("cgtb_repeat", code(dtype), len(shape), longs(want.shape), ints([1 if i in axes else 0 for i in range(len(shape))]),
                 dx.ptr, dout.ptr)
            assert np.array_equal(dout.get(), want)
        for (shape, axes) in [((4, 6, 5, 3), [0, 3, 1, 2]), ((4, 3, 6, 5), [0, 2, 3, 1]), ((7, 9), [1, 0]), ((2, 3, 4), [2, 0, 1]),
                              ((2, 3, 4), [1, 0, 2]), ((33, 65), [1, 0]), ((3, 1, 4), [2, 1, 0]), ((5, 4), [0, 1])]:
            x = (rs.randn(*shape) * 10).astype(dtype)
            want = O.transpose(x, axes)
            dx, dout = Dev(x), Dev(shape=want.shape, dtype=dtype)
            call("cgtb_transpose", code(dtype), len(shape), longs(shape), ints(axes), dx.ptr, dout.ptr)
            assert np.array_equal(dout.get(), want), (shape, axes)
        x = (rs.randn(6, 10, 4) * 10).astype(dtype)
        for (axis, start, stop, step) in [(1, 0, 10, 1), (1, 2, 9, 3), (0, 5, -1, -1), (2, 1, 3, 1), (0, 3, 4, 1)]:
            want = O.getsli(x, axis, start, stop, step)
            outer, n_in, inner = O._split(x.shape, axis)
            dx, dout = Dev(x), Dev(shape=want.shape, dtype=dtype)
            call("cgtb_getsli", code(dtype), outer, n_in, inner, start, step, want.shape[axis], dx.ptr, dout.ptr)
            assert np.array_equal(dout.get(), want)
            inc = (rs.randn(*want.shape) * 10).astype(dtype)
            want2 = O.incsli(x, axis, start, stop, step, inc)
            dinc, dout2 = Dev(inc), Dev(shape=x.shape, dtype=dtype)
            call("cgtb_incsli", code(dtype), outer, n_in, inner, start, step, want.shape[axis], dx.ptr, dinc.ptr, dout2.ptr)
            assert np.array_equal(dout2.get(), want2)
        parts = [(rs.randn(3, k, 2) * 10).astype(dtype) for k in (1, 4, 2)]
        want = O.concatenate(parts, 1)
        dout = Dev(shape=want.shape, dtype=dtype)
        pos = 0
        for p in parts:
            dp = Dev(p)
            call("cgtb_concat_part", code(dtype), 3, p.shape[1], want.shape[1], 2, pos, dp.ptr, dout.ptr)
            pos += p.shape[1]
        assert np.array_equal(dout.get(), want)


def test_flat_indices(rt):
    rs = np.random.RandomState(7)
    for dtype in ("f4", "i8", "f8"):
        x = (rs.randn(128, 10) * 10).astype(dtype)
        k = (np.arange(128) * 10 + rs.randint(0, 10, size=128)).astype("i8")
        want = O.getflat(x, k)
        dx, dk, dout = Dev(x), Dev(k), Dev(shape=(128,), dtype=dtype)
        call("cgtb_getflat", code(dtype), 128, dx.ptr, dk.ptr, dout.ptr)
        assert np.array_equal(dout.get(), want)
        # duplicates accumulate, in index order (reference test_inc_subtensor.py:53-71)
        kdup = rs.randint(0, 20, size=300).astype("i8")
        p = (rs.randn(300) * 10).astype(dtype)
        base = (rs.randn(40) * 10).astype(dtype)
        want = O.incflat(base, kdup, p)
        db, dk2, dp, dout2 = Dev(base), Dev(kdup), Dev(p), Dev(shape=(40,), dtype=dtype)
        call("cgtb_incflat", code(dtype), 40, 300, db.ptr, dk2.ptr, dp.ptr, dout2.ptr)
        assert np.array_equal(dout2.get(), want)
    want = O.fill(2.5, (3, 4), "f4")
    dout = Dev(shape=(3, 4), dtype="f4")
    call("cgtb_fill", code("f4"), 12, ctypes.c_double(2.5), 0, dout.ptr)
    assert np.array_equal(dout.get(), want)
    dout = Dev(shape=(5,), dtype="i8")
    call("cgtb_fill", code("i8"), 5, ctypes.c_double(0), 7, dout.ptr)
    assert np.array_equal(dout.get(), np.full(5, 7, "i8"))


GEMM_SHAPES = [
    # (M, N, K)  -- reference test shapes, config shapes scaled to run in seconds, ragged edges
    (3, 5, 4), (128, 10, 256), (128, 256, 784), (1024, 32, 75), (900, 32, 800), (32, 75, 4096), (64, 800, 1152),
    (450, 800, 32), (1, 1, 1), (65, 63, 17), (100, 20, 500), (64, 512, 65), (129, 257, 130),
    # the unrolled LSTM's products (hidden 128, batch 64)
    (64, 512, 128), (128, 512, 64), (64, 128, 512),
]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
@pytest.mark.parametrize("tA,tB", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("impl", [1, 0, 6])
def test_sgemm(rt, M, N, K, tA, tB, impl):
    """impl 0: the dispatcher's choice; 1: the generic FMA kernel; 6: the 16 x 16 FMA-tile kernel for products below the
    tensor-core kernels' break-even size."""
    if impl == 6 and M * N * K > (1 << 25):
        pytest.skip("beyond the FMA-tile kernel's size limit")
    rs = np.random.RandomState(8)
    A = rs.randn(*((K, M) if tA else (M, K))).astype("f4")
    B = rs.randn(*((N, K) if tB else (K, N))).astype("f4")
    want = O.mul22(A, B, tA, tB)
    dA, dB, dC = Dev(A), Dev(B), Dev(shape=(M, N), dtype="f4")
    call("cgtb_sgemm", tA, tB, M, N, K, dA.ptr, A.shape[1], dB.ptr, B.shape[1], dC.ptr, N, impl)
    got = dC.get()
    exact = (A.T if tA else A).astype("f8") @ (B.T if tB else B).astype("f8")
    # fp32 semantics: the error against float64 must be of the size of OpenBLAS's own fp32 error
    scale = np.sqrt(K)
    assert np.abs(got - exact).max() <= 4 * np.abs(want - exact).max() + 1e-5 * scale
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-5 * scale)


# every extent a multiple of 4 floats, so both tensor-core feeds (4: TMA, 3: registers) accept the operands;
# ragged against the 128 x UN x 32 tiling, one K block only, split-K (few tiles, long K), several column tiles
ALIGNED_GEMM_SHAPES = [(128, 12, 256), (900, 32, 800), (32, 76, 4096), (64, 800, 1152), (452, 800, 32), (132, 260, 132),
                       (2000, 128, 96), (128, 512, 784), (36, 36, 40), (4000, 16, 64)]


@pytest.mark.parametrize("M,N,K", ALIGNED_GEMM_SHAPES)
@pytest.mark.parametrize("tA,tB", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("impl", [4, 3])
def test_sgemm_tensor_core_feeds(rt, M, N, K, tA, tB, impl):
    rs = np.random.RandomState(18)
    A = rs.randn(*((K, M) if tA else (M, K))).astype("f4")
    B = rs.randn(*((N, K) if tB else (K, N))).astype("f4")
    A[0, 0] = np.float32(1e20)  # large magnitudes survive the hi/lo split
    if M > 2:
        A[(0, 1) if tA else (1, 0)] = np.float32(-3e36)  # beyond the fast split's range: the guarded path
    want = O.mul22(A, B, tA, tB)
    dA, dB, dC = Dev(A), Dev(B), Dev(np.full((M, N), np.nan, "f4"))
    call("cgtb_sgemm", tA, tB, M, N, K, dA.ptr, A.shape[1], dB.ptr, B.shape[1], dC.ptr, N, impl)
    got = dC.get()
    exact = (A.T if tA else A).astype("f8") @ (B.T if tB else B).astype("f8")
    big = np.abs(exact) > 1e15
    np.testing.assert_allclose(got[big], exact[big], rtol=1e-5)
    scale = np.sqrt(K)
    assert np.abs(got - exact)[~big].max() <= 4 * np.abs(want - exact)[~big].max() + 1e-5 * scale
    np.testing.assert_allclose(got[~big], want[~big], rtol=1e-4, atol=1e-5 * scale)


@pytest.mark.parametrize("impl", [4, 3, 0])
def test_sgemm_batched_strided(rt, impl):
    rs = np.random.RandomState(19)
    P, M, N, K = 3, 200, 48, 160
    A, B = rs.randn(P, M, K).astype("f4"), rs.randn(P, K, N).astype("f4")
    want = O.batched_mul22(A, B)
    dA, dB, dC = Dev(A), Dev(B), Dev(shape=(P, M, N), dtype="f4")
    call("cgtb_sgemm_batched", 0, 0, P, M, N, K, dA.ptr, K, M * K, dB.ptr, N, K * N, dC.ptr, N, M * N, impl)
    np.testing.assert_allclose(dC.get(), want, rtol=1e-4, atol=1e-4)
    # a view into wider storage: leading dimensions larger than the extents
    A2, B2 = rs.randn(M, K + 8).astype("f4"), rs.randn(N, K + 4).astype("f4")
    dA2, dB2, dC2 = Dev(A2), Dev(B2), Dev(shape=(M, N), dtype="f4")
    call("cgtb_sgemm", 0, 1, M, N, K, dA2.ptr, K + 8, dB2.ptr, K + 4, dC2.ptr, N, impl)
    np.testing.assert_allclose(dC2.get(), A2[:, :K].astype("f8") @ B2[:, :K].astype("f8").T, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("impl", [4, 3])
def test_sgemm_non_finite_inputs_stay_non_finite(rt, impl):
    rs = np.random.RandomState(20)
    M, N, K = 256, 32, 64
    A, B = rs.randn(M, K).astype("f4"), rs.randn(N, K).astype("f4")
    A[3, 5], A[7, 9], A[200, 63] = np.inf, np.nan, -np.inf
    A[9, 1] = np.float32(np.frombuffer(np.uint32(0x7F800001).tobytes(), "f4")[0])  # NaN with only low mantissa bits set
    dA, dB, dC = Dev(A), Dev(B), Dev(shape=(M, N), dtype="f4")
    call("cgtb_sgemm", 0, 1, M, N, K, dA.ptr, K, dB.ptr, K, dC.ptr, N, impl)
    got = dC.get()
    bad = np.zeros(M, bool)
    bad[[3, 7, 9, 200]] = True
    assert not np.isfinite(got[bad]).any()
    assert np.isnan(got[7]).all() and np.isnan(got[9]).all()
    np.testing.assert_allclose(got[~bad], (A[~bad].astype("f8") @ B.astype("f8").T), rtol=1e-4, atol=1e-4)


def test_sgemm_unaligned_is_refused_by_tma_feed(rt):
    A, B = np.ones((64, 75), "f4"), np.ones((75, 32), "f4")
    dA, dB, dC = Dev(A), Dev(B), Dev(shape=(64, 32), dtype="f4")
    rc = runtime.lib().cgtb_sgemm(0, 0, 64, 32, 75, dA.ptr, 75, dB.ptr, 32, dC.ptr, 32, 4)
    assert rc != 0 and "not eligible" in runtime.last_error()
    call("cgtb_sgemm", 0, 0, 64, 32, 75, dA.ptr, 75, dB.ptr, 32, dC.ptr, 32, 0)  # automatic choice falls back
    np.testing.assert_allclose(dC.get(), np.full((64, 32), 75.0, "f4"))


@pytest.mark.parametrize("M,N,K", [(128, 10, 256), (128, 256, 10), (256, 10, 128), (3, 5, 4), (1, 1, 1), (65, 63, 17), (7, 9, 2047)])
@pytest.mark.parametrize("tA,tB", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_sgemm_small_products(rt, M, N, K, tA, tB):
    rs = np.random.RandomState(21)
    A = rs.randn(*((K, M) if tA else (M, K))).astype("f4")
    B = rs.randn(*((N, K) if tB else (K, N))).astype("f4")
    want = O.mul22(A, B, tA, tB)
    dA, dB, dC = Dev(A), Dev(B), Dev(shape=(M, N), dtype="f4")
    call("cgtb_sgemm", tA, tB, M, N, K, dA.ptr, A.shape[1], dB.ptr, B.shape[1], dC.ptr, N, 5)
    got = dC.get()
    exact = (A.T if tA else A).astype("f8") @ (B.T if tB else B).astype("f8")
    assert np.abs(got - exact).max() <= 4 * np.abs(want - exact).max() + 1e-5 * np.sqrt(K)
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-5 * np.sqrt(K))


def test_sgemm_batched_and_dgemm(rt):
    rs = np.random.RandomState(9)
    A, B = rs.randn(2, 3, 5).astype("f4"), rs.randn(2, 5, 7).astype("f4")  # reference test_affine.py:364-375
    want = O.batched_mul22(A, B)
    dA, dB, dC = Dev(A), Dev(B), Dev(shape=(2, 3, 7), dtype="f4")
    call("cgtb_sgemm_batched", 0, 0, 2, 3, 7, 5, dA.ptr, 5, 15, dB.ptr, 7, 35, dC.ptr, 7, 21, 0)
    np.testing.assert_allclose(dC.get(), want, rtol=1e-4, atol=1e-5)
    A, B = rs.randn(40, 30), rs.randn(50, 30)
    dA, dB, dC = Dev(A), Dev(B), Dev(shape=(40, 50), dtype="f8")
    call("cgtb_dgemm", 0, 1, 40, 50, 30, dA.ptr, 30, dB.ptr, 30, dC.ptr, 50)
    np.testing.assert_allclose(dC.get(), A @ B.T, rtol=1e-12, atol=1e-12)


CONV_DGRADS = [
    # (B, C, H, W, Cin, k, pad): CIFAR conv2 and conv3 data gradients (scaled batch), bands that do not divide
    # the image, several small images per tile, a last tile with missing images, two K blocks per tap
    (8, 32, 15, 15, 32, 5, 2), (7, 32, 6, 6, 64, 5, 2), (3, 16, 20, 9, 32, 3, 1), (2, 48, 33, 128, 32, 3, 1),
    (5, 32, 4, 4, 32, 3, 0), (2, 128, 7, 5, 96, 1, 0),
]


@pytest.mark.parametrize("B,C,H,W,Cin,k,pad", CONV_DGRADS)
@pytest.mark.parametrize("bank", [False, True])
def test_conv_dgrad_matches_gemm_then_col2im(rt, B, C, H, W, Cin, k, pad, bank):
    """cgtb_conv_dgrad against the pair it replaces, evaluated by the CPU oracle: Mul22(dy, W) then Col2Im."""
    rs = np.random.RandomState(41)
    Ho, Wo = H + 2 * pad - k + 1, W + 2 * pad - k + 1
    dy = rs.randn(B, Ho, Wo, Cin).astype("f4")           # NHWC gradient of the convolution's output
    Wf = (rs.randn(Cin, C, k, k) * 0.2).astype("f4")     # filter bank [output channels of the conv, C, kh, kw]
    col = O.mul22(dy.reshape(B * Ho * Wo, Cin), Wf.reshape(Cin, C * k * k), 0, 0).reshape(B, Ho, Wo, C * k * k)
    want = O.col2im(col, (B, C, H, W), (k, k), (pad, pad), (1, 1))
    wr = Wf if bank else np.ascontiguousarray(Wf.transpose(1, 2, 3, 0))  # the bank as stored, or [C, kh, kw, Cin]
    ddy, dwr, ddx = Dev(dy), Dev(wr), Dev(np.full((B, C, H, W), np.nan, "f4"))
    call("cgtb_conv_dgrad_bank" if bank else "cgtb_conv_dgrad", ddy.ptr, B, Ho, Wo, Cin, dwr.ptr, C, H, W, k, k, pad, pad, ddx.ptr)
    got = ddx.get()
    exact = np.zeros((B, C, H, W))
    dy8, W8 = dy.astype("f8"), Wf.astype("f8")
    for i in range(k):
        for j in range(k):
            # dx[b,c,y,x] += sum_co dy[b, y+pad-i, x+pad-j, co] * W[co, c, i, j]
            ys, xs = np.arange(H) + pad - i, np.arange(W) + pad - j
            yv, xv = (ys >= 0) & (ys < Ho), (xs >= 0) & (xs < Wo)
            if not yv.any() or not xv.any():
                continue
            sub = dy8[:, ys[yv]][:, :, xs[xv]]                      # [B, ny, nx, Cin]
            exact[:, :, np.where(yv)[0][:, None], np.where(xv)[0][None, :]] += np.einsum("byxo,oc->bcyx", sub, W8[:, :, i, j])
    scale = np.sqrt(Cin * k * k)
    assert np.abs(got - exact).max() <= 4 * np.abs(want - exact).max() + 1e-5 * scale
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-5 * scale)


CONV_IMPLICIT = [
    # (B, Cin, H, W, Cout, k, pad): CIFAR conv2 / conv3 (scaled batch and batch 128), the wide net's conv2 (three K blocks
    # per tap, two column tiles), bands that do not divide the image, 1x1 and unpadded kernels, a last tile with missing images
    (8, 32, 15, 15, 32, 5, 2), (7, 32, 6, 6, 64, 5, 2), (128, 32, 15, 15, 32, 5, 2), (128, 32, 6, 6, 64, 5, 2),
    (6, 96, 6, 6, 256, 5, 2), (3, 32, 20, 9, 16, 3, 1), (2, 64, 7, 5, 48, 1, 0), (5, 32, 4, 4, 32, 3, 0), (300, 32, 3, 3, 16, 3, 1),
]


@pytest.mark.parametrize("B,Cin,H,W,Cout,k,pad", CONV_IMPLICIT)
@pytest.mark.parametrize("bank", [False, True])
def test_conv_fwd_bias_relu_matches_im2col_then_gemm(rt, B, Cin, H, W, Cout, k, pad, bank):
    """cgtb_conv_fwd_bias_relu against the sequence it replaces, evaluated by the CPU oracle: Im2Col, Mul22(col, W^T),
    NCHW, + bias, relu with its mask."""
    rs = np.random.RandomState(44)
    Ho, Wo = H + 2 * pad - k + 1, W + 2 * pad - k + 1
    x = rs.randn(B, Cin, H, W).astype("f4")
    Wf = (rs.randn(Cout, Cin, k, k) / np.sqrt(Cin * k * k)).astype("f4")
    bias = (0.1 * rs.randn(Cout)).astype("f4")
    col = O.im2col(x, (k, k), (pad, pad), (1, 1)).reshape(B * Ho * Wo, Cin * k * k)
    want_t = (O.mul22(col, Wf.reshape(Cout, -1), 0, 1) + bias).reshape(B, Ho * Wo, Cout).transpose(0, 2, 1)
    exact_t = (col.astype("f8") @ Wf.reshape(Cout, -1).astype("f8").T + bias.astype("f8")).reshape(B, Ho * Wo, Cout).transpose(0, 2, 1)
    xn = np.ascontiguousarray(x.transpose(0, 2, 3, 1))
    # the filter bank as the layer stores it, or a copy rearranged to [Cout, kh, kw, Cin]
    wr = Wf if bank else np.ascontiguousarray(Wf.transpose(0, 2, 3, 1))
    dx, dw, db = Dev(xn), Dev(wr), Dev(bias)
    y, mask = Dev(np.full((B, Cout, Ho * Wo), np.nan, "f4")), Dev(np.full((B, Cout, Ho * Wo), 7, "i1"))
    call("cgtb_conv_fwd_bias_relu_bank" if bank else "cgtb_conv_fwd_bias_relu", dx.ptr, B, H, W, Cin, dw.ptr, Cout, Ho, Wo, k, k, pad, pad, db.ptr, y.ptr, mask.ptr)
    got, gmask = y.get(), mask.get()
    assert set(np.unique(gmask)) <= {0, 1}
    K = Cin * k * k
    sure = np.abs(exact_t) > 1e-4 * np.sqrt(K)
    assert np.array_equal(gmask[sure], (exact_t >= 0)[sure].astype("i1"))
    on = gmask == 1
    scale = np.sqrt(K)
    assert np.abs(got[on] - exact_t[on]).max() <= 4 * np.abs(want_t[on] - exact_t[on]).max() + 1e-5 * scale
    np.testing.assert_allclose(got[on], want_t[on], rtol=1e-4, atol=1e-5 * scale)
    assert (got[~on] == 0).all()


@pytest.mark.parametrize("B,Cin,H,W,Cout,k,pad", [(8, 32, 15, 15, 32, 5, 2), (128, 32, 6, 6, 64, 5, 2), (6, 96, 6, 6, 256, 5, 2),
                                                  (3, 32, 20, 9, 16, 3, 1)])
def test_conv_with_filters_split_ahead(rt, B, Cin, H, W, Cout, k, pad):
    """cgtb_split_filter_banks makes the [w_hi | w_lo] copies of a layer's bank for the forward product and for the data
    gradient in one launch; cgtb_conv_fwd_bias_relu_pre / cgtb_conv_dgrad_pre given those copies return the bits of
    cgtb_conv_fwd_bias_relu_bank / cgtb_conv_dgrad_bank, which split on every call."""
    rs = np.random.RandomState(46)
    Ho, Wo = H + 2 * pad - k + 1, W + 2 * pad - k + 1
    xn = rs.randn(B, H, W, Cin).astype("f4")
    Wf = (rs.randn(Cout, Cin, k, k) / np.sqrt(Cin * k * k)).astype("f4")
    bias = (0.1 * rs.randn(Cout)).astype("f4")
    dyn = rs.randn(B, Ho, Wo, Cout).astype("f4")
    dx, dw, db, ddy = Dev(xn), Dev(Wf), Dev(bias), Dev(dyn)
    s_fwd, s_dg = Dev(np.full((2, Cout, k * k * Cin), np.nan, "f4")), Dev(np.full((2, Cin, k * k * Cout), np.nan, "f4"))
    banks = (ctypes.c_void_p * 2)(dw.ptr, dw.ptr)
    outs = (ctypes.c_void_p * 2)(s_fwd.ptr, s_dg.ptr)
    call("cgtb_split_filter_banks", 2, banks, ints((Cout, Cin)), ints((Cin, Cout)), ints((k * k, k * k)), ints((1, 2)), outs)
    hi, lo = s_fwd.get()
    want = Wf.transpose(0, 2, 3, 1).reshape(Cout, -1)      # K runs over (tap, input channel)
    assert np.abs(hi + lo - want).max() <= 2.0 ** -21 * np.abs(want).max()
    assert ((hi.view("u4") & 0x1FFF) == 0).all() and ((lo.view("u4") & 0x1FFF) == 0).all()
    y0, m0 = Dev(np.full((B, Cout, Ho * Wo), np.nan, "f4")), Dev(np.full((B, Cout, Ho * Wo), 7, "i1"))
    y1, m1 = Dev(np.full((B, Cout, Ho * Wo), np.nan, "f4")), Dev(np.full((B, Cout, Ho * Wo), 7, "i1"))
    call("cgtb_conv_fwd_bias_relu_bank", dx.ptr, B, H, W, Cin, dw.ptr, Cout, Ho, Wo, k, k, pad, pad, db.ptr, y0.ptr, m0.ptr)
    k0 = runtime.kernel_launches()
    call("cgtb_conv_fwd_bias_relu_pre", dx.ptr, B, H, W, Cin, dw.ptr, s_fwd.ptr, Cout, Ho, Wo, k, k, pad, pad, db.ptr, y1.ptr, m1.ptr)
    n_pre = runtime.kernel_launches() - k0
    assert np.array_equal(y0.get(), y1.get()) and np.array_equal(m0.get(), m1.get())
    if Cin <= 128 and Cout % 32 == 0:      # data gradient: at most 128 image channels, gradient channels in groups of 32
        g0, g1 = Dev(np.full((B, Cin, H * W), np.nan, "f4")), Dev(np.full((B, Cin, H * W), np.nan, "f4"))
        k0 = runtime.kernel_launches()
        call("cgtb_conv_dgrad_bank", ddy.ptr, B, Ho, Wo, Cout, dw.ptr, Cin, H, W, k, k, pad, pad, g0.ptr)
        n_bank = runtime.kernel_launches() - k0
        k0 = runtime.kernel_launches()
        call("cgtb_conv_dgrad_pre", ddy.ptr, B, Ho, Wo, Cout, dw.ptr, s_dg.ptr, Cin, H, W, k, k, pad, pad, g1.ptr)
        assert runtime.kernel_launches() - k0 == n_bank - 1
        assert np.array_equal(g0.get(), g1.get())
    assert n_pre == 1
    # more than eight jobs, or a layout that is neither, are refused
    rc = runtime.lib().cgtb_split_filter_banks(2, banks, ints((Cout, Cin)), ints((Cin, Cout)), ints((k * k, k * k)), ints((1, 3)), outs)
    assert rc != 0 and "layout" in runtime.last_error()


@pytest.mark.parametrize("B,Cin,H,W,Cout,k,pad", CONV_IMPLICIT + [(2, 32, 9, 32, 16, 3, 1), (3, 32, 5, 17, 32, 3, 1)])
def test_conv_wgrad_matches_gemm_on_im2col(rt, B, Cin, H, W, Cout, k, pad):
    """cgtb_conv_wgrad against the product it replaces, evaluated by the CPU oracle: Mul22{T,N}(dy, Im2Col(x))."""
    rs = np.random.RandomState(45)
    Ho, Wo = H + 2 * pad - k + 1, W + 2 * pad - k + 1
    x = rs.randn(B, Cin, H, W).astype("f4")
    dy = (rs.randn(B, Ho, Wo, Cout) * (rs.rand(B, Ho, Wo, Cout) > 0.5)).astype("f4")
    col = O.im2col(x, (k, k), (pad, pad), (1, 1)).reshape(B * Ho * Wo, Cin * k * k)
    want = O.mul22(dy.reshape(-1, Cout), col, 1, 0)
    exact = dy.reshape(-1, Cout).astype("f8").T @ col.astype("f8")
    xn = np.ascontiguousarray(x.transpose(0, 2, 3, 1))
    dxn, ddy, dwg = Dev(xn), Dev(dy), Dev(np.full((Cout, Cin * k * k), np.nan, "f4"))
    call("cgtb_conv_wgrad", dxn.ptr, B, H, W, Cin, ddy.ptr, Ho, Wo, Cout, k, k, pad, pad, dwg.ptr)
    got = dwg.get()
    scale = np.sqrt(B * Ho * Wo)
    assert np.abs(got - exact).max() <= 4 * np.abs(want - exact).max() + 1e-5 * scale
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-5 * scale)


@pytest.mark.parametrize("B,H", [(2, 32), (5, 8), (128, 32)])
def test_conv_direct_first_layer(rt, B, H):
    """The 3-channel first layer computed directly from the NCHW image: forward with bias, relu and mask against the
    reference's own path restated on the CPU (im2col_cpu -> sgemm -> + bias -> relu, cgt/nn.py:87-100, 44-45), and the
    filter gradient against Mul22{T,N}(dy, col) of the same column matrix, both adjudicated in float64."""
    rs = np.random.RandomState(B * 7 + H)
    Cin, W, Cout, k, pad = 3, 32, 32, 5, 2
    x = rs.randn(B, Cin, H, W).astype("f4")
    w = (rs.randn(Cout, Cin * k * k) * 0.1).astype("f4")
    bias = rs.randn(Cout).astype("f4")
    col = O.im2col(x, (k, k), (pad, pad), (1, 1)).reshape(B * H * W, Cin * k * k)
    exact = (col.astype("f8") @ w.astype("f8").T + bias.astype("f8")).reshape(B, H, W, Cout).transpose(0, 3, 1, 2)
    want32 = (O.mul22(col, w, False, True) + bias).reshape(B, H, W, Cout).transpose(0, 3, 1, 2)
    dx, dw_, db = Dev(x), Dev(w), Dev(bias)
    y, mask = Dev(shape=(B, Cout, H, W), dtype="f4"), Dev(shape=(B, Cout, H, W), dtype="i1")
    call("cgtb_conv_direct_fwd_bias_relu", dx.ptr, B, Cin, H, W, dw_.ptr, Cout, k, k, pad, pad, db.ptr, y.ptr, mask.ptr)
    got, gm = y.get(), mask.get()
    err = np.abs(got - np.maximum(exact, 0))
    assert err.max() <= 4 * np.abs(np.maximum(want32, 0) - np.maximum(exact, 0)).max() + 1e-5
    sure = np.abs(exact) > 1e-4     # the mask is (t >= 0): compare where rounding cannot flip the sign
    assert np.array_equal(gm[sure].astype(bool), exact[sure] >= 0)
    assert np.array_equal(got, np.where(gm.astype(bool), got, 0.0).astype("f4"))
    # filter gradient
    dy = rs.randn(B, H, W, Cout).astype("f4")
    exact_w = dy.reshape(-1, Cout).astype("f8").T @ col.astype("f8")
    want_w = O.mul22(dy.reshape(-1, Cout), col, True, False)
    ddy, out = Dev(dy), Dev(np.full((Cout, Cin * k * k), np.nan, "f4"))
    call("cgtb_conv_direct_wgrad", dx.ptr, B, Cin, H, W, ddy.ptr, Cout, k, k, pad, pad, out.ptr)
    got_w = out.get()
    scale = np.sqrt(B * H * W)
    assert np.abs(got_w - exact_w).max() <= 4 * np.abs(want_w - exact_w).max() + 1e-5 * scale
    # the same gradient from the layer's backward inputs: dy = mask * g (both NCHW), plus the bias gradient
    g = rs.randn(B, Cout, H, W).astype("f4")
    m = (rs.rand(B, Cout, H, W) < 0.5).astype("i1")
    dy2 = np.ascontiguousarray((g * m).transpose(0, 2, 3, 1))
    exact_w2 = dy2.reshape(-1, Cout).astype("f8").T @ col.astype("f8")
    want_w2 = O.mul22(dy2.reshape(-1, Cout), col, True, False)
    dg, dm, out2, outb = Dev(g), Dev(m), Dev(np.full((Cout, Cin * k * k), np.nan, "f4")), Dev(np.full((Cout,), np.nan, "f4"))
    call("cgtb_conv_direct_wgrad_relu", dx.ptr, B, Cin, H, W, dm.ptr, dg.ptr, Cout, k, k, pad, pad, out2.ptr, outb.ptr)
    assert np.abs(out2.get() - exact_w2).max() <= 4 * np.abs(want_w2 - exact_w2).max() + 1e-5 * scale
    exact_b = (g.astype("f8") * m).sum(axis=(0, 2, 3))
    want_b = (g * m).sum(axis=(0, 2, 3), dtype="f4")
    assert np.abs(outb.get() - exact_b).max() <= 4 * np.abs(want_b - exact_b).max() + 1e-5 * scale
    # given the product it forms, it adds in the order of the channels-last entry point (whose fold of fewer than 16
    # partial results adds them one after the other instead): identical bits
    ddy2 = Dev(dy2)
    call("cgtb_conv_direct_wgrad", dx.ptr, B, Cin, H, W, ddy2.ptr, Cout, k, k, pad, pad, out.ptr)
    if B * (H // 8) >= 16:
        assert np.array_equal(out.get(), out2.get())
    else:
        np.testing.assert_allclose(out.get(), out2.get(), rtol=1e-4, atol=1e-5 * scale)
    # an image that does not start on a 16-byte boundary is refused before any launch (its rows are read as 128-bit words)
    k0 = runtime.kernel_launches()
    rc = runtime.lib().cgtb_conv_direct_fwd_bias_relu(ctypes.c_void_p(dx.w.data + 4), B, Cin, H, W, dw_.ptr, Cout, k, k, pad, pad, db.ptr, y.ptr, mask.ptr)
    assert rc != 0 and "16-byte" in runtime.last_error() and runtime.kernel_launches() == k0
    # another layer is refused, not approximated
    rc = runtime.lib().cgtb_conv_direct_wgrad(dx.ptr, B, 4, H, W, ddy.ptr, Cout, k, k, pad, pad, out.ptr)
    assert rc != 0 and "not supported" in runtime.last_error()


def test_conv_implicit_refuses_unsupported_extents(rt):
    d = Dev(shape=(64,), dtype="f4")
    L = runtime.lib()
    assert L.cgtb_conv_fwd_bias_relu(d.ptr, 1, 4, 4, 3, d.ptr, 16, 4, 4, 3, 3, 1, 1, d.ptr, d.ptr, d.ptr) != 0
    assert "not supported" in runtime.last_error()
    assert L.cgtb_conv_wgrad(d.ptr, 1, 4, 40, 32, d.ptr, 4, 40, 16, 3, 3, 1, 1, d.ptr) != 0
    assert "not supported" in runtime.last_error()
    assert L.cgtb_conv_wgrad(d.ptr, 1, 4, 4, 32, d.ptr, 5, 4, 16, 3, 3, 1, 1, d.ptr) != 0
    assert "stride-1" in runtime.last_error()


@pytest.mark.parametrize("B,HW,C,K", [(4, 1024, 32, 75), (8, 225, 32, 800), (16, 36, 64, 800), (3, 10, 48, 40), (2, 7, 16, 5)])
def test_conv_bias_relu_matches_op_sequence(rt, B, HW, C, K):
    """cgtb_conv_bias_relu against the sequence it replaces, issued through the separate entry points:
    sgemm -> NHWC->NCHW transpose -> repeat bias -> add -> >= 0 -> multiply. Same bits."""
    rs = np.random.RandomState(51)
    M = B * HW
    col, w, bias = rs.randn(M, K).astype("f4"), (rs.randn(C, K) * 0.1).astype("f4"), rs.randn(C).astype("f4")
    dcol, dw, db = Dev(col), Dev(w), Dev(bias)
    y, mask = Dev(shape=(B, C, HW), dtype="f4"), Dev(shape=(B, C, HW), dtype="i1")
    L = runtime.lib()
    L.cgtb_conv_bias_relu.restype = ctypes.c_int
    L.cgtb_conv_bias_relu.argtypes = [ctypes.c_void_p, ctypes.c_long, ctypes.c_long, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p,
                                      ctypes.c_long, ctypes.c_void_p, ctypes.c_void_p]
    call("cgtb_conv_bias_relu", dcol.ptr, M, K, dw.ptr, C, db.ptr, HW, y.ptr, mask.ptr)
    g, gt, rep, t, m2, y2 = (Dev(shape=sh, dtype=dt) for (sh, dt) in [((M, C), "f4"), ((B, C, HW), "f4"), ((B, C, HW), "f4"),
                                                                       ((B, C, HW), "f4"), ((B, C, HW), "i1"), ((B, C, HW), "f4")])
    n = B * C * HW
    call("cgtb_sgemm", 0, 1, M, C, K, dcol.ptr, K, dw.ptr, K, g.ptr, C, 0)
    call("cgtb_transpose", code("f4"), 3, longs((B, HW, C)), ints((0, 2, 1)), g.ptr, gt.ptr)
    call("cgtb_repeat", code("f4"), 3, longs((B, C, HW)), ints([1, 0, 1]), db.ptr, rep.ptr)
    call("cgtb_binary", 1, code("f4"), code("f4"), code("f4"), n, gt.ptr, rep.ptr, t.ptr, 0, 0)
    zero = Dev(np.array(0, "i8"))
    call("cgtb_binary", 7, code("f4"), code("i8"), code("i1"), n, t.ptr, zero.ptr, m2.ptr, 0, 1)
    call("cgtb_binary", 0, code("f4"), code("i1"), code("f4"), n, t.ptr, m2.ptr, y2.ptr, 0, 0)
    assert np.array_equal(mask.get(), m2.get())
    assert np.array_equal(y.get(), y2.get())
    want = np.maximum((col.astype("f8") @ w.astype("f8").T + bias).reshape(B, HW, C).transpose(0, 2, 1), 0)
    np.testing.assert_allclose(y.get(), want, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("B,HW,C,K,ld", [(4, 1024, 32, 75, 76), (2, 225, 16, 27, 28), (3, 64, 96, 363, 364), (2, 100, 8, 30, 35),
                                         (130, 1024, 32, 75, 76)])
def test_conv_bias_relu_and_filter_gradient_on_padded_rows(rt, B, HW, C, K, ld):
    """cgtb_conv_bias_relu_ld and the filter-gradient product on a column matrix whose rows are `ld` >= K apart give
    what the unpadded matrix gives; the padding entries (NaN here) are never used."""
    rs = np.random.RandomState(52)
    M = B * HW
    col, w, bias = rs.randn(M, K).astype("f4"), (rs.randn(C, K) * 0.1).astype("f4"), rs.randn(C).astype("f4")
    colp = np.full((M, ld), np.nan, "f4")
    colp[:, :K] = col
    dcol, dw, db = Dev(colp), Dev(w), Dev(bias)
    y, mask = Dev(shape=(B, C, HW), dtype="f4"), Dev(shape=(B, C, HW), dtype="i1")
    L = runtime.lib()
    L.cgtb_conv_bias_relu_ld.restype = ctypes.c_int
    L.cgtb_conv_bias_relu_ld.argtypes = [ctypes.c_void_p, ctypes.c_long, ctypes.c_long, ctypes.c_long, ctypes.c_void_p, ctypes.c_int,
                                         ctypes.c_void_p, ctypes.c_long, ctypes.c_void_p, ctypes.c_void_p]
    call("cgtb_conv_bias_relu_ld", dcol.ptr, M, K, ld, dw.ptr, C, db.ptr, HW, y.ptr, mask.ptr)
    t = (col.astype("f8") @ w.astype("f8").T + bias).reshape(B, HW, C).transpose(0, 2, 1)
    np.testing.assert_allclose(y.get(), np.maximum(t, 0), rtol=1e-4, atol=1e-4)
    sure = np.abs(t) > 1e-3
    assert np.array_equal(mask.get()[sure], (t >= 0)[sure])
    # filter gradient: dy^T [C, M] . col[:, :K] -> [C, K] with ldb = ld, ldc = K
    dy = rs.randn(M, C).astype("f4")
    ddy, dwg = Dev(dy), Dev(shape=(C, K), dtype="f4")
    call("cgtb_sgemm", 1, 0, C, K, M, ddy.ptr, C, dcol.ptr, ld, dwg.ptr, K, 0)
    want = dy.astype("f8").T @ col.astype("f8")
    np.testing.assert_allclose(dwg.get(), want, rtol=1e-4, atol=1e-4 * np.sqrt(M))


@pytest.mark.parametrize("B,C,H,W", [(4, 32, 32, 32), (8, 32, 15, 15), (16, 64, 6, 6), (3, 48, 5, 3), (2, 16, 20, 13),
                                     (128, 32, 32, 32), (128, 32, 15, 15), (128, 64, 6, 6)])
def test_relu_grad_nhwc_matches_op_sequence(rt, B, C, H, W):
    """cgtb_relu_grad_nhwc against multiply -> transpose and Sum{0,2,3}: the transposed product bit for bit, the
    channel sums against float64 like every other sum."""
    rs = np.random.RandomState(61)
    mask = (rs.rand(B, C, H, W) > 0.4).astype("i1")
    g = rs.randn(B, C, H, W).astype("f4")
    dm, dg = Dev(mask), Dev(g)
    gt, bs = Dev(shape=(B, H, W, C), dtype="f4"), Dev(shape=(1, C, 1, 1), dtype="f4")
    L = runtime.lib()
    L.cgtb_relu_grad_nhwc.restype = ctypes.c_int
    L.cgtb_relu_grad_nhwc.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_long, ctypes.c_int, ctypes.c_long, ctypes.c_void_p,
                                      ctypes.c_void_p]
    call("cgtb_relu_grad_nhwc", dm.ptr, dg.ptr, B, C, H * W, gt.ptr, bs.ptr)
    n = B * C * H * W
    prod, prod_t = Dev(shape=(B, C, H, W), dtype="f4"), Dev(shape=(B, H, W, C), dtype="f4")
    call("cgtb_binary", 0, code("i1"), code("f4"), code("f4"), n, dm.ptr, dg.ptr, prod.ptr, 0, 0)
    call("cgtb_transpose", code("f4"), 4, longs((B, C, H, W)), ints((0, 2, 3, 1)), prod.ptr, prod_t.ptr)
    assert np.array_equal(gt.get(), prod_t.get())
    assert np.array_equal(gt.get(), (mask * g).transpose(0, 2, 3, 1))
    exact = (mask.astype("f8") * g.astype("f8")).sum(axis=(0, 2, 3))
    want = O.reduce("sum", (mask * g).astype("f4"), [0, 2, 3]).reshape(C)
    got = bs.get().reshape(C)
    tol = 1e-5 * max(1.0, np.sqrt(B * H * W))
    assert (np.abs(got - exact) <= 1e-4 * np.abs(exact) + tol).all()
    assert np.abs(got - exact).max() <= 2 * np.abs(want - exact).max() + tol


from cgt_b200.core import FusedElwise as _F   # the limits of include/cgt_b200.h (CGTB_FUSED_MAX_*)


class _FusedProgram(ctypes.Structure):
    _fields_ = [("n_in", ctypes.c_int), ("n_ops", ctypes.c_int), ("n_out", ctypes.c_int), ("in_kind", ctypes.c_int * _F.MAX_IN),
                ("op_arity", ctypes.c_int * _F.MAX_OPS), ("op_code", ctypes.c_int * _F.MAX_OPS), ("op_a", ctypes.c_int * _F.MAX_OPS),
                ("op_b", ctypes.c_int * _F.MAX_OPS), ("out_reg", ctypes.c_int * _F.MAX_OUT), ("out_dtype", ctypes.c_int * _F.MAX_OUT),
                ("launcher", ctypes.c_void_p),  # NULL: the library's own kernel runs the program
                ("view_width", ctypes.c_long)]


@pytest.mark.parametrize("shape", [(8, 32, 15, 15), (4, 6, 5, 7), (3, 5, 2, 2)])
def test_fused_elwise_matches_separate_kernels(rt, shape):
    """bias add (operand broadcast from [1,C,1,1]) -> x >= 0 -> x * mask -> sigmoid -> / scalar, in one
    kernel, against the same chain issued Op by Op through cgtb_repeat / cgtb_binary / cgtb_unary."""
    rs = np.random.RandomState(31)
    B, C, H, W = shape
    n = int(np.prod(shape))
    x, bias = rs.randn(*shape).astype("f4"), rs.randn(1, C, 1, 1).astype("f4")
    zero, div = np.array(0, "i8"), np.array(3.0, "f4")
    dx, db, dz, dd = Dev(x), Dev(bias), Dev(zero), Dev(div)
    # separate kernels
    rep, s1, m, s2, s3, s4 = (Dev(shape=shape, dtype=t) for t in ("f4", "f4", "i1", "f4", "f4", "f4"))
    call("cgtb_repeat", code("f4"), 4, longs(shape), ints([1, 0, 1, 1]), db.ptr, rep.ptr)
    call("cgtb_binary", 1, code("f4"), code("f4"), code("f4"), n, dx.ptr, rep.ptr, s1.ptr, 0, 0)
    call("cgtb_binary", 7, code("f4"), code("i8"), code("i1"), n, s1.ptr, dz.ptr, m.ptr, 0, 1)
    call("cgtb_binary", 0, code("f4"), code("i1"), code("f4"), n, s1.ptr, m.ptr, s2.ptr, 0, 0)
    call("cgtb_unary", 13, code("f4"), code("f4"), n, s2.ptr, s3.ptr)
    call("cgtb_binary", 3, code("f4"), code("f4"), code("f4"), n, s3.ptr, dd.ptr, s4.ptr, 0, 1)
    # one kernel: inputs x (f4), bias (broadcast), 0 (i8 scalar), 3.0 (f4 scalar): registers 0..3
    P = _FusedProgram()
    P.n_in, P.n_ops, P.n_out = 4, 5, 3
    for (k, kind) in enumerate([0, 4, 3, 2]):
        P.in_kind[k] = kind
    ops = [(2, 1, 0, 1), (2, 7, 4, 2), (2, 0, 4, 5), (1, 13, 6, 0), (2, 3, 7, 3)]  # registers 4..8
    for (j, (ar, opc, a, b)) in enumerate(ops):
        P.op_arity[j], P.op_code[j], P.op_a[j], P.op_b[j] = ar, opc, a, b
    for (q, (reg, dt)) in enumerate([(5, "i1"), (6, "f4"), (8, "f4")]):
        P.out_reg[q], P.out_dtype[q] = reg, code(dt)
    om, o2, o4 = Dev(shape=shape, dtype="i1"), Dev(shape=shape, dtype="f4"), Dev(shape=shape, dtype="f4")
    ins = (ctypes.c_void_p * _F.MAX_IN)(dx.ptr, db.ptr, dz.ptr, dd.ptr)
    outs = (ctypes.c_void_p * _F.MAX_OUT)(om.ptr, o2.ptr, o4.ptr)
    bk, binner = longs([1, C, 1, 1, 1, 1, 1, 1]), longs([1, H * W, 1, 1, 1, 1, 1, 1])
    call("cgtb_fused_elwise", ctypes.byref(P), n, ins, bk, binner, outs)
    assert np.array_equal(om.get(), m.get())
    assert np.array_equal(o2.get(), s2.get())
    assert np.array_equal(o4.get(), s4.get())
    # and against the CPU oracle
    t = x + bias
    want_mask = (t >= 0)
    assert np.array_equal(om.get().astype(bool), want_mask)
    np.testing.assert_allclose(o2.get(), t * want_mask, rtol=RTOL, atol=ATOL)


class _RowProgram(ctypes.Structure):
    _fields_ = [("n_in", ctypes.c_int), ("n_ops", ctypes.c_int), ("n_out", ctypes.c_int), ("in_kind", ctypes.c_int * _F.MAX_IN),
                ("op_arity", ctypes.c_int * _F.MAX_OPS), ("op_code", ctypes.c_int * _F.MAX_OPS), ("op_a", ctypes.c_int * _F.MAX_OPS),
                ("op_b", ctypes.c_int * _F.MAX_OPS), ("out_reg", ctypes.c_int * _F.MAX_OUT), ("out_col", ctypes.c_int * _F.MAX_OUT),
                ("launcher", ctypes.c_void_p)]  # NULL: the library's own kernel runs the program


@pytest.mark.parametrize("R,C", [(128, 10), (64, 65), (1, 1), (5, 32), (1000, 33), (7, 100), (300, 128)])
def test_fused_rows_softmax_chain(rt, R, C):
    """log(exp(x + bias) / rowsum(exp(x + bias))) with its pullback against a target matrix, the chain a softmax loss
    compiles to (cgt/nn.py:55-62), in one launch: against float64 numpy, and against the row sums of cgtb_reduce."""
    rs = np.random.RandomState(R * 131 + C)
    x, bias = rs.randn(R, C).astype("f4"), rs.randn(1, C).astype("f4")
    g, scale = rs.randn(R, C).astype("f4"), np.array(-1.0 / R, "f4")
    dx, db, dg, dsc = Dev(x), Dev(bias), Dev(g), Dev(scale)
    # registers: 0 x [R,C], 1 bias [1,C], 2 g [R,C], 3 scale (scalar)
    # 4 = x + bias, 5 = exp, 6 = rowsum(5), 7 = 5 / 6 (softmax), 8 = log(7), 9 = g * scale, 10 = 9 / 7 (d softmax),
    # 11 = 10 * 7, 12 = rowsum(11), 13 = 10 - 12, 14 = 13 * 7 (d logits)
    ops = [(2, 1, 0, 1), (1, 3, 4, 0), (3, 0, 5, 0), (2, 3, 5, 6), (1, 6, 7, 0), (2, 0, 2, 3), (2, 3, 9, 7),
           (2, 0, 10, 7), (3, 0, 11, 0), (2, 2, 10, 12), (2, 0, 13, 7)]
    P = _RowProgram()
    P.n_in, P.n_ops, P.n_out = 4, len(ops), 3
    for (k, kind) in enumerate([0, 6, 0, 2]):
        P.in_kind[k] = kind
    for (j, (ar, opc, a, b)) in enumerate(ops):
        P.op_arity[j], P.op_code[j], P.op_a[j], P.op_b[j] = ar, opc, a, b
    for (q, (reg, col)) in enumerate([(8, 0), (6, 1), (14, 0)]):
        P.out_reg[q], P.out_col[q] = reg, col
    o_log, o_sum, o_dl = Dev(shape=(R, C), dtype="f4"), Dev(shape=(R, 1), dtype="f4"), Dev(shape=(R, C), dtype="f4")
    ins = (ctypes.c_void_p * _F.MAX_IN)(dx.ptr, db.ptr, dg.ptr, dsc.ptr)
    outs = (ctypes.c_void_p * _F.MAX_OUT)(o_log.ptr, o_sum.ptr, o_dl.ptr)
    call("cgtb_fused_rows", ctypes.byref(P), R, C, ins, outs)
    e = np.exp(x.astype("f8") + bias.astype("f8"))
    ssum = e.sum(axis=1, keepdims=True)
    sm = e / ssum
    dsm = g.astype("f8") * float(scale) / sm
    dl = (dsm - (dsm * sm).sum(axis=1, keepdims=True)) * sm
    np.testing.assert_allclose(o_sum.get(), ssum, rtol=2e-6)
    np.testing.assert_allclose(o_log.get(), np.log(sm), rtol=1e-5, atol=2e-6)
    np.testing.assert_allclose(o_dl.get(), dl, rtol=1e-4, atol=1e-5 * np.abs(dl).max())
    # the separate reduction kernel over the same exponentials
    e4 = Dev(np.exp(x + bias).astype("f4"))
    red = Dev(shape=(R, 1), dtype="f4")
    call("cgtb_reduce", 0, code("f4"), 2, longs((R, C)), ints((0, 1)), e4.ptr, red.ptr)
    np.testing.assert_allclose(o_sum.get(), red.get(), rtol=3e-6)


@pytest.mark.parametrize("R,C", [(128, 10), (64, 65), (3, 128), (1000, 33)])
def test_row_selection_kernels(rt, R, C):
    """x[arange(R), idx] and its gradient as row arithmetic: cgtb_onehot_rows against the reference's
    IncFlatIndices(zeros, arange(R)*C + idx, ones) (cgt/core.py:1814-1860), cgtb_masked_row_sum against
    GetFlatIndices (cgt/core.py:1781-1812) bit for bit, with a -inf outside the selection that must not reach the
    result, and the same through one cgtb_fused_rows program (input kind 8, entry (4, 0, a, b))."""
    rs = np.random.RandomState(R + C)
    x = rs.randn(R, C).astype("f4")
    idx = rs.randint(0, C, size=R).astype("i8")
    x[0, (idx[0] + 1) % C] = -np.inf
    g = rs.randn(R).astype("f4")
    flat = np.arange(R, dtype="i8") * C + idx
    hot_np = O.incflat(np.zeros((R, C), "f4"), flat, np.ones(R, "f4"))
    assert np.array_equal(hot_np, (np.arange(C)[None, :] == idx[:, None]).astype("f4"))
    dx, didx, dg = Dev(x), Dev(idx), Dev(g.reshape(R, 1))
    hot, pick = Dev(np.full((R, C), np.nan, "f4")), Dev(np.full((R, 1), np.nan, "f4"))
    call("cgtb_onehot_rows", didx.ptr, R, C, hot.ptr)
    assert np.array_equal(hot.get(), hot_np)
    call("cgtb_masked_row_sum", dx.ptr, hot.ptr, R, C, pick.ptr)
    assert np.array_equal(pick.get().reshape(R), O.getflat(x, flat))
    # one program: 0 x, 1 idx (kind 8), 2 g [R,1]; 3 = pick(0 where 1), 4 = hot * g
    P = _RowProgram()
    P.n_in, P.n_ops, P.n_out = 3, 2, 2
    for (k, kind) in enumerate([0, 8, 5]):
        P.in_kind[k] = kind
    for (j, (ar, opc, a, b)) in enumerate([(4, 0, 0, 1), (2, 0, 1, 2)]):
        P.op_arity[j], P.op_code[j], P.op_a[j], P.op_b[j] = ar, opc, a, b
    for (q, (reg, col)) in enumerate([(3, 1), (4, 0)]):
        P.out_reg[q], P.out_col[q] = reg, col
    o_pick, o_grad = Dev(np.full((R, 1), np.nan, "f4")), Dev(np.full((R, C), np.nan, "f4"))
    ins = (ctypes.c_void_p * _F.MAX_IN)(dx.ptr, didx.ptr, dg.ptr)
    outs = (ctypes.c_void_p * _F.MAX_OUT)(o_pick.ptr, o_grad.ptr)
    call("cgtb_fused_rows", ctypes.byref(P), R, C, ins, outs)
    assert np.array_equal(o_pick.get().reshape(R), x.reshape(-1)[flat])
    assert np.array_equal(o_grad.get(), hot_np * g[:, None])


@pytest.mark.parametrize("tA,tB,M,N,K", [(0, 0, 64, 512, 128), (0, 0, 8, 512, 65), (1, 0, 37, 130, 50), (1, 1, 64, 96, 31)])
def test_sgemm_bias_add_has_the_bits_of_the_separate_kernels(rt, tA, tB, M, N, K):
    """cgtb_sgemm_bias_add = (addend + addend_bias) + (A.B + bias) in the product's output stage, against cgtb_sgemm
    followed by the three additions as separate kernels (the rows repeated by cgtb_repeat): identical bits. Products that
    the dispatcher does not give to the FMA-tile kernel are refused."""
    rs = np.random.RandomState(M + N + K)
    A = rs.randn(*((K, M) if tA else (M, K))).astype("f4")
    B = rs.randn(*((N, K) if tB else (K, N))).astype("f4")
    bias, abias, addend = rs.randn(1, N).astype("f4"), rs.randn(1, N).astype("f4"), rs.randn(M, N).astype("f4")
    dA, dB, dbias, dabias, dadd = Dev(A), Dev(B), Dev(bias), Dev(abias), Dev(addend)
    lda, ldb = A.shape[1], B.shape[1]
    prod, rep1, rep2, t1, t2, want = (Dev(shape=(M, N), dtype="f4") for _ in range(6))
    call("cgtb_sgemm", tA, tB, M, N, K, dA.ptr, lda, dB.ptr, ldb, prod.ptr, N, 0)
    call("cgtb_repeat", code("f4"), 2, longs((M, N)), ints([1, 0]), dbias.ptr, rep1.ptr)
    call("cgtb_repeat", code("f4"), 2, longs((M, N)), ints([1, 0]), dabias.ptr, rep2.ptr)
    call("cgtb_binary", 1, code("f4"), code("f4"), code("f4"), M * N, prod.ptr, rep1.ptr, t2.ptr, 0, 0)
    call("cgtb_binary", 1, code("f4"), code("f4"), code("f4"), M * N, dadd.ptr, rep2.ptr, t1.ptr, 0, 0)
    call("cgtb_binary", 1, code("f4"), code("f4"), code("f4"), M * N, t1.ptr, t2.ptr, want.ptr, 0, 0)
    got = Dev(np.full((M, N), np.nan, "f4"))
    k0 = runtime.kernel_launches()
    call("cgtb_sgemm_bias_add", tA, tB, M, N, K, dA.ptr, lda, dB.ptr, ldb, dbias.ptr, dadd.ptr, N, dabias.ptr, got.ptr, N)
    assert runtime.kernel_launches() - k0 == 1
    assert np.array_equal(got.get(), want.get())
    exact = (addend.astype("f8") + abias) + ((A.T if tA else A).astype("f8") @ (B.T if tB else B).astype("f8") + bias)
    np.testing.assert_allclose(got.get(), exact, rtol=1e-4, atol=1e-4 * np.sqrt(K))
    # without the optional operands it is the plain product
    call("cgtb_sgemm_bias_add", tA, tB, M, N, K, dA.ptr, lda, dB.ptr, ldb, None, None, 0, None, got.ptr, N)
    assert np.array_equal(got.get(), prod.get())
    # A.B^T and few outputs belong to the warp-per-output kernel: refused here
    L = runtime.lib()
    assert L.cgtb_sgemm_bias_add(0, 1, 64, 128, 512, dA.ptr, 512, dB.ptr, 512, None, None, 0, None, got.ptr, 128) != 0
    assert "FMA-tile" in runtime.last_error()


def test_fused_rows_refuses_long_rows(rt):
    P = _RowProgram()
    P.n_in, P.n_ops, P.n_out = 1, 1, 1
    P.op_arity[0], P.op_a[0] = 3, 0
    P.out_reg[0], P.out_col[0] = 1, 1
    d = Dev(shape=(4, 129), dtype="f4")
    o = Dev(shape=(4, 1), dtype="f4")
    rc = runtime.lib().cgtb_fused_rows(ctypes.byref(P), 4, 129, (ctypes.c_void_p * _F.MAX_IN)(d.ptr), (ctypes.c_void_p * _F.MAX_OUT)(o.ptr))
    assert rc != 0 and "128" in runtime.last_error()


@pytest.mark.parametrize("R,W,pitch,off", [(64, 128, 512, 384), (7, 5, 13, 3), (33, 12, 40, 8)])
def test_fused_elwise_reads_column_slices_in_place(rt, R, W, pitch, off):
    """tanh(S[:, off:off+W]) * g with S a wider matrix: the chain reads the columns of S where they lie (the GetSli of
    cgt/core.py:1767-1812 without its copy), bit-identical to slicing first."""
    rs = np.random.RandomState(R + W)
    S, g = rs.randn(R, pitch).astype("f4"), rs.randn(R, W).astype("f4")
    dS, dg = Dev(S), Dev(g)
    sl = Dev(np.ascontiguousarray(S[:, off:off + W]))
    t, want = Dev(shape=(R, W), dtype="f4"), Dev(shape=(R, W), dtype="f4")
    call("cgtb_unary", 12, code("f4"), code("f4"), R * W, sl.ptr, t.ptr)
    call("cgtb_binary", 0, code("f4"), code("f4"), code("f4"), R * W, t.ptr, dg.ptr, want.ptr, 0, 0)
    P = _FusedProgram()
    P.n_in, P.n_ops, P.n_out = 2, 2, 1
    P.in_kind[0], P.in_kind[1] = 7, 0
    P.op_arity[0], P.op_code[0], P.op_a[0] = 1, 12, 0
    P.op_arity[1], P.op_code[1], P.op_a[1], P.op_b[1] = 2, 0, 2, 1
    P.out_reg[0], P.out_dtype[0] = 3, code("f4")
    P.view_width = W
    out = Dev(shape=(R, W), dtype="f4")
    ins = (ctypes.c_void_p * _F.MAX_IN)(dS.ptr, dg.ptr)
    outs = (ctypes.c_void_p * _F.MAX_OUT)(out.ptr)
    bk, binner = longs([pitch] + [1] * (_F.MAX_IN - 1)), longs([off] + [1] * (_F.MAX_IN - 1))
    call("cgtb_fused_elwise", ctypes.byref(P), R * W, ins, bk, binner, outs)
    assert np.array_equal(out.get(), want.get())
    # a slice that sticks out of the matrix is refused
    bad = longs([pitch] + [1] * (_F.MAX_IN - 1)), longs([pitch - W + 1] + [1] * (_F.MAX_IN - 1))
    rc = runtime.lib().cgtb_fused_elwise(ctypes.byref(P), R * W, ins, bad[0], bad[1], outs)
    assert rc != 0 and "column range" in runtime.last_error()


def test_scatter_cols_places_pieces_into_zeros(rt):
    """The gradient of three column slices of a [R, 40] matrix: zeros, then each piece added into its columns
    (IncSli on a Fill, cgt/core.py:1786-1790, 1814-1861) and the three results added, against one launch."""
    rs = np.random.RandomState(9)
    R, C = 37, 40
    pieces = [(24, rs.randn(R, 9).astype("f4")), (0, rs.randn(R, 8).astype("f4")), (12, rs.randn(R, 12).astype("f4"))]
    want = np.zeros((R, C), "f4")
    for (o, y) in pieces:
        want = want + O.incsli(np.zeros((R, C), "f4"), 1, o, o + y.shape[1], 1, y)
    devs = [Dev(y) for (_o, y) in pieces]
    out = Dev(np.full((R, C), 7.0, "f4"))
    ptrs = (ctypes.c_void_p * _F.MAX_IN)(*[d.ptr for d in devs])
    call("cgtb_scatter_cols", R, C, 3, longs([o for (o, _y) in pieces]), longs([y.shape[1] for (_o, y) in pieces]), ptrs, out.ptr)
    assert np.array_equal(out.get(), want)
    rc = runtime.lib().cgtb_scatter_cols(R, C, 2, longs([0, 4]), longs([8, 8]), ptrs, out.ptr)
    assert rc != 0 and "overlap" in runtime.last_error()


def test_reduce_over_an_empty_axis_gives_the_identity(rt):
    """Sum / Max over an axis of extent 0: every kept element is the operation's initial value (the reference's
    loop never runs, cgt/core.py:1663-1685, 1708, 1737)."""
    x = Dev(shape=(1,), dtype="f4")
    for (kind, want) in ((0, 0.0), (1, -np.finfo("f4").max)):
        out = Dev(np.full((4, 1, 3), 9.0, "f4"))
        call("cgtb_reduce", kind, code("f4"), 3, longs((4, 0, 3)), ints((0, 1, 0)), x.ptr, out.ptr)
        assert np.array_equal(out.get(), np.full((4, 1, 3), want, "f4"))


def test_empty_inputs(rt):
    d = Dev(shape=(1,), dtype="f4")
    call("cgtb_unary", 3, code("f4"), code("f4"), 0, d.ptr, d.ptr)
    call("cgtb_binary", 1, code("f4"), code("f4"), code("f4"), 0, d.ptr, d.ptr, d.ptr, 0, 0)
    call("cgtb_fill", code("f4"), 0, ctypes.c_double(1.0), 0, d.ptr)
    call("cgtb_im2col", code("f4"), d.ptr, 0, 3, 8, 8, 3, 3, 1, 1, 1, 1, d.ptr)
    call("cgtb_sgemm", 0, 0, 0, 4, 4, d.ptr, 4, d.ptr, 4, d.ptr, 4, 0)
