"""Run single kernels of libcgt_b200.so through the C ABI on chosen shapes, for profiling.

    python -m cgt_b200.kernel_probe sgemm M N K tA tB [impl]     one product, timed with CUDA events
    python -m cgt_b200.kernel_probe stencils                      the CIFAR batch-128 stencil / movement kernels

Each kernel runs `--reps` times (default 2) after an L2 flush, so that a profiler attached to the process
(`ncu -k regex:<name> -c <n> ...`) sees cold-cache launches of exactly these kernels and nothing else.
"""
import argparse
import ctypes

import numpy as np

from . import runtime


def _dev(arr=None, shape=None, dtype="f4"):
    if arr is None:
        arr = np.zeros(shape, dtype)
    return runtime.device_array(np.ascontiguousarray(arr))


def _ptr(w):
    return ctypes.c_void_p(w.data)


def _timed(name, fn, reps, nbytes=None):
    e0, e1 = runtime.Event(), runtime.Event()
    ts = []
    for _ in range(reps):
        runtime.l2_flush()
        runtime.synchronize()
        e0.record()
        runtime.check(fn(), name)
        e1.record()
        ts.append(e0.elapsed_ms(e1) * 1e3)
    runtime.synchronize()
    best = min(ts[1:]) if len(ts) > 1 else ts[0]
    extra = "  %7.0f GB/s of %6.1f MB" % (nbytes / (best * 1e-6) / 1e9, nbytes / 1e6) if nbytes else ""
    print("%-34s %s us (launch included)%s" % (name, " ".join("%.1f" % t for t in ts), extra), flush=True)


def sgemm(M, N, K, tA, tB, impl, reps):
    L = runtime.lib()
    rs = np.random.RandomState(0)
    A = rs.randn(*((K, M) if tA else (M, K))).astype("f4")
    B = rs.randn(*((N, K) if tB else (K, N))).astype("f4")
    dA, dB, dC = _dev(A), _dev(B), _dev(shape=(M, N))
    _timed("sgemm %s impl %d" % ((M, N, K, tA, tB), impl),
           lambda: L.cgtb_sgemm(tA, tB, M, N, K, _ptr(dA), A.shape[1], _ptr(dB), B.shape[1], _ptr(dC), N, impl), reps,
           4 * (M * K + K * N + M * N))


def stencils(reps):
    L = runtime.lib()
    rs = np.random.RandomState(0)
    f4 = runtime._dtype_code(np.dtype("f4"))
    B = 128
    longs = lambda xs: (ctypes.c_long * len(xs))(*xs)
    ints = lambda xs: (ctypes.c_int * len(xs))(*xs)
    d = ctypes.c_double
    # conv2: 32 channels 15x15, 5x5 pad 2
    x2, col2 = _dev(rs.randn(B, 32, 15, 15).astype("f4")), _dev(shape=(B, 15, 15, 800))
    n2 = 4 * (B * 32 * 225 + B * 225 * 800)
    _timed("im2col conv2", lambda: L.cgtb_im2col(f4, _ptr(x2), B, 32, 15, 15, 5, 5, 2, 2, 1, 1, _ptr(col2)), reps, n2)
    _timed("col2im conv2", lambda: L.cgtb_col2im(f4, _ptr(col2), B, 32, 15, 15, 5, 5, 2, 2, 1, 1, _ptr(x2)), reps, n2)
    x1, col1 = _dev(rs.randn(B, 3, 32, 32).astype("f4")), _dev(shape=(B, 32, 32, 75))
    _timed("im2col conv1", lambda: L.cgtb_im2col(f4, _ptr(x1), B, 3, 32, 32, 5, 5, 2, 2, 1, 1, _ptr(col1)), reps,
           4 * (B * 3 * 1024 + B * 1024 * 75))
    col1p = _dev(shape=(B, 32, 32, 76))
    L.cgtb_im2col_ld.restype = ctypes.c_int
    L.cgtb_im2col_ld.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_long] + [ctypes.c_int] * 9 + [ctypes.c_long, ctypes.c_void_p]
    _timed("im2col conv1, rows of 76", lambda: L.cgtb_im2col_ld(f4, _ptr(x1), B, 3, 32, 32, 5, 5, 2, 2, 1, 1, 76, _ptr(col1p)), reps,
           4 * (B * 3 * 1024 + B * 1024 * 76))
    # data gradient of conv2 without a column matrix
    dy, wr, dx = _dev(rs.randn(B, 15, 15, 32).astype("f4")), _dev(rs.randn(32, 5, 5, 32).astype("f4")), _dev(shape=(B, 32, 15, 15))
    L.cgtb_conv_dgrad.restype = ctypes.c_int
    L.cgtb_conv_dgrad.argtypes = ([ctypes.c_void_p, ctypes.c_long] + [ctypes.c_int] * 3 + [ctypes.c_void_p] + [ctypes.c_int] * 7 +
                                  [ctypes.c_void_p])
    _timed("conv_dgrad conv2", lambda: L.cgtb_conv_dgrad(_ptr(dy), B, 15, 15, 32, _ptr(wr), 32, 15, 15, 5, 5, 2, 2, _ptr(dx)), reps,
           4 * (2 * B * 32 * 225 + 25600))
    # pool1: 32x32 -> 15x15, 3x3 stride 2
    xp = _dev(rs.randn(B, 32, 32, 32).astype("f4"))
    top, mask, gx = _dev(shape=(B, 32, 15, 15)), _dev(shape=(B, 32, 15, 15), dtype="i4"), _dev(shape=(B, 32, 32, 32))
    nin, nout = B * 32 * 1024, B * 32 * 225
    _timed("max_pool pool1", lambda: L.cgtb_max_pool(f4, _ptr(xp), B, 32, 32, 32, 3, 3, 0, 0, 2, 2, 15, 15, _ptr(top), _ptr(mask)),
           reps, 4 * nin + 8 * nout)
    _timed("max_pool_pullback pool1",
           lambda: L.cgtb_max_pool_pullback(f4, _ptr(mask), _ptr(top), B, 32, 15, 15, 32, 32, 3, 3, 0, 0, 2, 2, _ptr(gx)), reps,
           8 * nout + 4 * nin)
    # LRN on the pooled activations
    t, s, g = _dev(shape=(B, 32, 15, 15)), _dev(shape=(B, 32, 15, 15)), _dev(shape=(B, 32, 15, 15))
    _timed("lrn_forward", lambda: L.cgtb_lrn_forward(f4, _ptr(x2), B, 32, 15, 15, 5, d(1e-4), d(0.75), _ptr(t), _ptr(s)), reps,
           12 * nout)
    _timed("lrn_backward",
           lambda: L.cgtb_lrn_backward(f4, _ptr(x2), _ptr(t), _ptr(s), _ptr(x2), B, 32, 15, 15, 5, d(1e-4), d(0.75), _ptr(g)), reps,
           20 * nout)
    # activation-sized movement and reduction
    a, o = _dev(rs.randn(B, 32, 32, 32).astype("f4")), _dev(shape=(B, 32, 32, 32))
    _timed("transpose NHWC->NCHW act1", lambda: L.cgtb_transpose(f4, 4, longs([B, 32, 32, 32]), ints([0, 3, 1, 2]), _ptr(a), _ptr(o)),
           reps, 8 * nin)
    out = _dev(shape=(1, 32, 1, 1))
    _timed("sum{0,2,3} act1", lambda: L.cgtb_reduce(0, f4, 4, longs([B, 32, 32, 32]), ints([1, 0, 1, 1]), _ptr(a), _ptr(out)), reps,
           4 * nin)
    _timed("sum{0,2,3} act2", lambda: L.cgtb_reduce(0, f4, 4, longs([B, 32, 15, 15]), ints([1, 0, 1, 1]), _ptr(x2), _ptr(out)), reps,
           4 * nout)
    _timed("binary multiply act1", lambda: L.cgtb_binary(0, f4, f4, f4, nin, _ptr(a), _ptr(gx), _ptr(o), 0, 0), reps, 12 * nin)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["sgemm", "stencils"])
    ap.add_argument("dims", nargs="*", type=int)
    ap.add_argument("--reps", type=int, default=2)
    args = ap.parse_args()
    runtime.ensure_init()
    if args.what == "sgemm":
        assert len(args.dims) in (5, 6), "sgemm M N K tA tB [impl]"
        M, N, K, tA, tB = args.dims[:5]
        sgemm(M, N, K, tA, tB, args.dims[5] if len(args.dims) == 6 else 0, args.reps)
    else:
        stencils(args.reps)


if __name__ == "__main__":
    main()
