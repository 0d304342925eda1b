"""Generates tests/golden/*.npz from the reference's own native code (oracle/_ref: include/im2col.h,
include/pooling.h, include/lrn.cuh compiled as C++ from the reference tree). Run where the reference
tree is present:

    python tests/golden/make_golden.py

The fixtures are small seeded cases: inputs and the exact outputs of the reference code, used to pin
the CPU restatement (and, on the GPU box where the reference tree is absent, the CUDA kernels).
"""
import os
import os.path as osp
import sys

import numpy as np

HERE = osp.dirname(osp.abspath(__file__))
sys.path.insert(0, osp.normpath(osp.join(HERE, "..", "..")))

from oracle import oracle as O  # noqa: E402

assert O.have_ref(), "build oracle/_ref first (python oracle/build_oracle.py)"
rs = np.random.RandomState(20151)


def save(name, **arrays):
    np.savez_compressed(osp.join(HERE, name + ".npz"), **arrays)
    print(name, {k: v.shape for (k, v) in arrays.items()})


# im2col / col2im: the reference test geometries (cgt/tests/test_imgproc.py:59-61, test_conv.py:14-31)
# plus the conv geometries of the benchmark configurations
for (tag, shape, kernel, pad, stride) in [
    ("t4400", (2, 1, 28, 28), (4, 4), (0, 0), (1, 1)), ("t3312", (2, 1, 28, 28), (3, 3), (1, 1), (2, 2)),
    ("t3313", (2, 1, 28, 28), (3, 3), (1, 1), (3, 3)), ("conv", (2, 2, 5, 17), (4, 7), (3, 6), (1, 1)),
    ("cifar", (2, 3, 12, 12), (5, 5), (2, 2), (1, 1)), ("wide", (1, 3, 23, 23), (11, 11), (2, 2), (4, 4)),
]:
    x = rs.randn(*shape).astype("f4")
    col = O.im2col(x, kernel, pad, stride, impl="ref")
    g = rs.randn(*col.shape).astype("f4")
    im = O.col2im(g, shape, kernel, pad, stride, impl="ref")
    save("im2col_" + tag, x=x, geom=np.array(kernel + pad + stride), col=col, g=g, im=im)

# max pool: reference test geometry (test_imgproc.py:40-57) and the k3 s2 p0 pooling of the configs,
# once with ties (rounded values) so the first-maximum rule is pinned
for (tag, shape, kernel, pad, stride, ties) in [
    ("t44", (2, 3, 5, 7), (4, 4), (0, 0), (1, 1), False), ("k3s2", (2, 4, 15, 15), (3, 3), (0, 0), (2, 2), False),
    ("k3s2_ties", (2, 4, 9, 9), (3, 3), (0, 0), (2, 2), True), ("pad", (1, 2, 9, 11), (3, 3), (1, 1), (2, 2), True),
]:
    x = rs.randn(*shape).astype("f4")
    if ties:
        x = np.round(x).astype("f4")
    top, mask = O.max_pool(x, kernel, pad, stride, impl="ref")
    g = rs.randn(*top.shape).astype("f4")
    gx = O.max_pool_pullback(shape, mask, g, impl="ref")
    save("pool_" + tag, x=x, geom=np.array(kernel + pad + stride), top=top, mask=mask, g=g, gx=gx)

# LRN: reference test parameters (test_imgproc.py:84-87) and the configs' (5, 1e-4, 0.75)
for (tag, shape, size, alpha, beta) in [("t4", (2, 8, 5, 5), 4, 0.1, 0.5), ("n5", (2, 12, 4, 4), 5, 1e-4, 0.75)]:
    x = rs.randn(*shape).astype("f4")
    top, scale = O.lrn_forward(x, size, alpha, beta, impl="ref")
    g = rs.randn(*shape).astype("f4")
    gx = O.lrn_backward(x, top, scale, g, size, alpha, beta, impl="ref")
    save("lrn_" + tag, x=x, params=np.array([size, alpha, beta]), top=top, scale=scale, g=g, gx=gx)
