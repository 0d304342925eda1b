"""GPU parity at the sizes the benchmark times: the BASELINE configurations at their full shapes (CIFAR-shape
convnet and wide conv stack at batch 128, the two-layer LSTM at sequence length 50 and batch 64) against the
CPU oracle, and every tensor-core launch of the CIFAR batch-128 training step through the C ABI.

Kernel selection depends on the extents (split-K or not, fused output stage or staged, which feed), so parity at a
scaled-down batch does not cover the launches that are timed. Bars: losses within 1e-3 relative at every update
step, parameters within 1e-3 of their scale; per kernel rtol 1e-4 with an absolute bar scaled by sqrt(K) (the
fp32 rounding error of a K-term dot product grows like sqrt(K); 1e-5 is the bar for K = 1) and, next to it, an error
against float64 no larger than a small multiple of OpenBLAS's own fp32 error.
"""
import ctypes

import numpy as np
import pytest

import cgt_b200 as cgt
from cgt_b200 import configs, runtime
from oracle import cpu_backend
from oracle import oracle as O
from tests.gpu_util import Dev, call

pytestmark = pytest.mark.gpu

FULL = {
    "cifar": dict(batch=128),
    "wide": dict(batch=128),
    "lstm": dict(seq_len=50, batch=64),
}


@pytest.mark.parametrize("name", ["cifar", "wide", "lstm"])
def test_full_shape_training_steps_match_oracle(rt, name):
    """Three update steps eagerly, three more from captured CUDA graphs, against three steps of the oracle.

    Losses: 1e-3 relative at every step. Parameters: within 1e-3 of their scale plus the per-Op absolute bar of 1e-5;
    at these sizes a bias gradient is a sum of 10^5 mostly cancelling terms, and the reference's sequential float32
    order and the kernels' tree order round differently, so every parameter is also adjudicated against the same
    steps with float64 accumulation: the GPU must not be farther from that than a small multiple of the reference
    order's own distance."""
    kw = FULL[name]
    steps = 3
    ref = configs.BUILDERS[name](**kw)
    f_cpu = cpu_backend.function(ref.inputs, [ref.loss] + ref.extra_outputs, updates=ref.updates, impl="ref")
    f_adj = cpu_backend.function(ref.inputs, [ref.loss] + ref.extra_outputs, updates=ref.updates, impl="ref", wide_sums=True)
    batches = [ref.batch(seed) for seed in range(2)]
    cpu = [[np.asarray(o) for o in f_cpu(*batches[i % 2])] for i in range(steps)]
    for i in range(steps):
        f_adj(*batches[i % 2])
    want_params = [f_cpu.get_value(p) for p in ref.params]
    adj_params = [f_adj.get_value(p) for p in ref.params]
    for graphs in (False, True):
        with cgt.scoped_update_config(use_cuda_graphs=graphs):
            cfg = configs.BUILDERS[name](**kw)
            f_gpu = cfg.compile()
            for i in range(steps):
                got = [np.asarray(o) for o in f_gpu(*batches[i % 2])]
                for (a, b) in zip(got, cpu[i]):
                    assert np.isfinite(b).all(), "oracle diverged at step %d" % i
                    np.testing.assert_allclose(a, b, rtol=1e-3, atol=1e-6, err_msg="%s step %d graphs=%s" % (name, i, graphs))
            report = []
            for (p, want, adj) in zip(cfg.params, want_params, adj_params):
                gotp = p.op.get_value()
                scale = max(np.abs(want).max(), 1e-6)
                d_ref, d_adj, ref_adj = np.abs(gotp - want).max(), np.abs(gotp - adj).max(), np.abs(want - adj).max()
                ok = d_ref <= 1e-3 * scale + 1e-5 and d_adj <= 4 * ref_adj + 1e-3 * scale + 1e-5
                report.append((p.name, ok, float(d_ref), float(d_adj), float(ref_adj), float(scale)))
            assert all(r[1] for r in report), (name, graphs, report)
            if graphs:
                st = f_gpu.stats()
                assert st["segments_captured"] >= 1 and st["last_graph_launches"] >= 1, st


def _check_product(got, want, exact, K, what):
    scale = np.sqrt(K)
    assert np.abs(got - exact).max() <= 4 * np.abs(want - exact).max() + 1e-5 * scale, what
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-5 * scale, err_msg=what)


def _sig():
    L = runtime.lib()
    vp, ci, cl = ctypes.c_void_p, ctypes.c_int, ctypes.c_long
    L.cgtb_conv_bias_relu.restype = ci
    L.cgtb_conv_bias_relu.argtypes = [vp, cl, cl, vp, ci, vp, cl, vp, vp]
    L.cgtb_conv_bias_relu_ld.restype = ci
    L.cgtb_conv_bias_relu_ld.argtypes = [vp, cl, cl, cl, vp, ci, vp, cl, vp, vp]
    L.cgtb_conv_dgrad.restype = ci
    L.cgtb_conv_dgrad.argtypes = [vp, cl] + [ci] * 3 + [vp] + [ci] * 7 + [vp]
    return L


# (B, HW, C, K, ld): the three forward products of the CIFAR step with their output stage
@pytest.mark.parametrize("B,HW,C,K,ld", [(128, 1024, 32, 75, 76), (128, 225, 32, 800, 800), (128, 36, 64, 800, 800)])
def test_forward_products_of_the_cifar_step(rt, B, HW, C, K, ld):
    L = _sig()
    rs = np.random.RandomState(71)
    M = B * HW
    col = rs.randn(M, K).astype("f4")
    w, bias = (rs.randn(C, K) / np.sqrt(K)).astype("f4"), (0.1 * rs.randn(C)).astype("f4")
    colp = col
    if ld != K:
        colp = np.full((M, ld), np.nan, "f4")  # the padding entries must never be read
        colp[:, :K] = col
    dcol, dw, db = Dev(colp), Dev(w), Dev(bias)
    y, mask = Dev(np.full((B, C, HW), np.nan, "f4")), Dev(np.full((B, C, HW), 7, "i1"))
    n0 = runtime.kernel_launches()
    if ld != K:
        call("cgtb_conv_bias_relu_ld", dcol.ptr, M, K, ld, dw.ptr, C, db.ptr, HW, y.ptr, mask.ptr)
    else:
        call("cgtb_conv_bias_relu", dcol.ptr, M, K, dw.ptr, C, db.ptr, HW, y.ptr, mask.ptr)
    launches = runtime.kernel_launches() - n0
    want_t = (O.mul22(col, w, 0, 1) + bias).reshape(B, HW, C).transpose(0, 2, 1)
    exact_t = (col.astype("f8") @ w.astype("f8").T + bias.astype("f8")).reshape(B, HW, C).transpose(0, 2, 1)
    got, gmask = y.get(), mask.get()
    assert set(np.unique(gmask)) <= {0, 1}
    sure = np.abs(exact_t) > 1e-4 * np.sqrt(K)
    assert np.array_equal(gmask[sure], (exact_t >= 0)[sure].astype("i1"))
    # y = t * mask with the kernel's own mask: compare pre-activation values where the unit is on
    on = gmask == 1
    _check_product(got[on], want_t[on], exact_t[on], K, "forward product %dx%dx%d" % (M, C, K))
    assert (got[~on] == 0).all()
    # the product that fills the machine runs unsplit with the output stage in its epilogue (one kernel; the
    # padded variant adds the copy of the small filter matrix to the padded pitch)
    if M >= 128 * 148:
        assert launches <= 2, launches


# (C, K, M, ldb): the three filter gradients dy^T . col of the CIFAR step
@pytest.mark.parametrize("C,K,M,ldb", [(32, 75, 131072, 76), (32, 800, 28800, 800), (64, 800, 4608, 800)])
def test_filter_gradients_of_the_cifar_step(rt, C, K, M, ldb):
    rs = np.random.RandomState(72)
    dy = (rs.randn(M, C) * (rs.rand(M, C) > 0.5)).astype("f4")   # relu-masked gradient: half zeros
    col = rs.randn(M, K).astype("f4")
    colp = col
    if ldb != K:
        colp = np.full((M, ldb), np.nan, "f4")
        colp[:, :K] = col
    ddy, dcol, dwg = Dev(dy), Dev(colp), Dev(np.full((C, K), np.nan, "f4"))
    call("cgtb_sgemm", 1, 0, C, K, M, ddy.ptr, C, dcol.ptr, ldb, dwg.ptr, K, 0)
    want = O.mul22(dy, col, 1, 0)
    exact = dy.astype("f8").T @ col.astype("f8")
    _check_product(dwg.get(), want, exact, M, "filter gradient %dx%d K=%d" % (C, K, M))


# (B, C, H, W, Cin, k, pad): data gradients of CIFAR conv2 / conv3 and of the wide net's conv2
@pytest.mark.parametrize("B,C,H,W,Cin,k,pad", [(128, 32, 15, 15, 32, 5, 2), (128, 32, 6, 6, 64, 5, 2), (128, 96, 6, 6, 256, 5, 2)])
def test_data_gradients_at_batch_128(rt, B, C, H, W, Cin, k, pad):
    _sig()
    rs = np.random.RandomState(73)
    Ho, Wo = H + 2 * pad - k + 1, W + 2 * pad - k + 1
    dy = (rs.randn(B, Ho, Wo, Cin) * (rs.rand(B, Ho, Wo, Cin) > 0.5)).astype("f4")
    Wf = (rs.randn(Cin, C, k, k) / np.sqrt(Cin * k * k)).astype("f4")
    col = O.mul22(dy.reshape(B * Ho * Wo, Cin), Wf.reshape(Cin, C * k * k), 0, 0).reshape(B, Ho, Wo, C * k * k)
    want = O.col2im(col, (B, C, H, W), (k, k), (pad, pad), (1, 1))
    wr = np.ascontiguousarray(Wf.transpose(1, 2, 3, 0))
    ddy, dwr, ddx = Dev(dy), Dev(wr), Dev(np.full((B, C, H, W), np.nan, "f4"))
    call("cgtb_conv_dgrad", ddy.ptr, B, Ho, Wo, Cin, dwr.ptr, C, H, W, k, k, pad, pad, ddx.ptr)
    got = ddx.get()
    exact = np.zeros((B, C, H, W))
    dy8, W8 = dy.astype("f8"), Wf.astype("f8")
    for i in range(k):
        for j in range(k):
            ys, xs = np.arange(H) + pad - i, np.arange(W) + pad - j
            yv, xv = (ys >= 0) & (ys < Ho), (xs >= 0) & (xs < Wo)
            if not yv.any() or not xv.any():
                continue
            sub = dy8[:, ys[yv]][:, :, xs[xv]]
            exact[:, :, np.where(yv)[0][:, None], np.where(xv)[0][None, :]] += np.einsum("byxo,oc->bcyx", sub, W8[:, :, i, j])
    _check_product(got, want, exact, Cin * k * k, "data gradient")


def test_refused_launch_is_reported_once_and_leaves_the_library_usable(rt):
    """A launch configuration that the CUDA runtime refuses on the host (nothing reaches the GPU) fails that call
    only: the next, healthy call succeeds instead of tripping over a stale error."""
    L = runtime.lib()
    rc = L.cgtb_selftest_refused_launch()
    assert rc != 0 and "selftest_refused_launch launch failed" in runtime.last_error()
    x = Dev(np.arange(8, dtype="f4"))
    out = Dev(shape=(8,), dtype="f4")
    call("cgtb_unary", 10, runtime._dtype_code("f4"), runtime._dtype_code("f4"), 8, x.ptr, out.ptr)  # square
    assert np.array_equal(out.get(), np.arange(8, dtype="f4") ** 2)
