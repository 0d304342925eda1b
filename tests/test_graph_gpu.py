"""GPU parity at graph level: compiled training-step functions (forward + cgt.grad + updates) on the
B200 against the same graph evaluated by the CPU oracle, for every benchmark configuration.

Tolerances: fp32 losses within 1e-3 relative after 10 update steps (and every step on the way),
parameters within 1e-3 of the oracle's after those steps relative to their scale (plus 1e-5 absolute).
"""
import numpy as np
import pytest

import ctypes

import cgt_b200 as cgt
from cgt_b200 import configs, core, nn
from oracle import cpu_backend

pytestmark = pytest.mark.gpu

SMALL = {
    "mlp": dict(batch=128),
    "cifar": dict(batch=16),
    "wide": dict(batch=4, lr=0.0002),
    "lstm": dict(seq_len=6, batch=8),
    "vae": dict(batch=100),
}


def _run_both(name, kw, steps, graphs):
    with cgt.scoped_update_config(use_cuda_graphs=graphs):
        cfg = configs.BUILDERS[name](**kw)
        f_cpu = cpu_backend.function(cfg.inputs, [cfg.loss] + cfg.extra_outputs, updates=cfg.updates, impl="ref")
        f_gpu = cfg.compile()
        batches = [cfg.batch(seed) for seed in range(2)]
        gpu, cpu = [], []
        for i in range(steps):
            b = batches[i % 2]
            gpu.append([np.asarray(o) for o in f_gpu(*b)])
            cpu.append([np.asarray(o) for o in f_cpu(*b)])
        return cfg, f_cpu, f_gpu, gpu, cpu


@pytest.mark.parametrize("name", ["mlp", "cifar", "vae", "lstm", "wide"])
@pytest.mark.parametrize("graphs", [False, True])
def test_ten_step_loss_parity(rt, name, graphs):
    cfg, f_cpu, f_gpu, gpu, cpu = _run_both(name, SMALL[name], 10, graphs)
    for (step, (g, c)) in enumerate(zip(gpu, cpu)):
        for (a, b) in zip(g, c):
            assert np.isfinite(b).all(), "oracle diverged at step %d" % step
            np.testing.assert_allclose(a, b, rtol=1e-3, atol=1e-6, err_msg="step %d" % step)
    for p in cfg.params:
        got, want = p.op.get_value(), f_cpu.get_value(p)
        scale = max(np.abs(want).max(), 1e-6)
        # 1e-3 of the parameter's scale, plus the per-Op absolute bar for parameters that are still tiny (a bias that
        # started at zero is 1e-4 after ten small steps: its relative error is the float32 noise of everything upstream)
        assert np.abs(got - want).max() <= 1e-3 * scale + 1e-5, p.name
    if graphs:
        st = f_gpu.stats()
        assert st["segments_captured"] >= 1 and st["last_graph_launches"] >= 1, st


def test_graph_replay_matches_eager(rt):
    """Captured CUDA graphs replay the same kernels on the same buffers: bit-identical results."""
    outs = {}
    for graphs in (False, True):
        with cgt.scoped_update_config(use_cuda_graphs=graphs):
            cfg = configs.build_cifar(batch=8)
            f = cfg.compile()
            b = cfg.batch(3)
            outs[graphs] = [f(*b)[0] for _ in range(6)] + [p.op.get_value() for p in cfg.params]
    for (a, b) in zip(outs[False], outs[True]):
        assert np.array_equal(a, b)


def test_updates_and_set_value(rt):
    """Update semantics (reference test_optimizers.py:8-21, test_array_wrapper.py): the final op of an
    update writes into the shared variable's storage; sgd on scale*x^2 from 1.0 gives (1-0.2*scale)^10."""
    for scale in (0.1, 0.2, 0.3):
        A = cgt.shared(np.array([1.0], "f4"))
        cost = (scale * A ** 2).sum()
        step = cgt.function([], [], updates=nn.sgd(cost, [A], 0.1))
        for _ in range(10):
            step()
        np.testing.assert_allclose(A.op.get_value(), (1 - 0.2 * scale) ** 10, rtol=1e-5)
    x = cgt.shared(np.arange(6, dtype="f4").reshape(2, 3), fixed_shape_mask="all")
    f = cgt.function([], x * 2.0)
    assert np.array_equal(f(), np.arange(6, dtype="f4").reshape(2, 3) * 2)
    f(); f()  # reach the captured-graph steady state, then change the value behind it
    x.op.set_value(np.ones((2, 3), "f4"))
    assert np.array_equal(f(), np.full((2, 3), 2, "f4"))


def test_shape_change_recaptures(rt):
    """No fixed shape: the same compiled function serves different batch sizes (Alloc re-allocates on a
    shape change and captured graphs are dropped)."""
    x = cgt.matrix("x")
    w = cgt.shared(np.random.RandomState(0).randn(5, 3).astype("f4"))
    y = cgt.tanh(x.dot(w)).sum(axis=1)
    f = cgt.function([x], y)
    rs = np.random.RandomState(1)
    for n in (4, 4, 4, 4, 9, 9, 9, 2, 4):
        xv = rs.randn(n, 5).astype("f4")
        np.testing.assert_allclose(f(xv), np.tanh(xv @ w.op.get_value()).sum(axis=1), rtol=1e-4, atol=1e-5)


def test_equal_size_shapes_do_not_share_a_captured_graph(rt):
    """Two input shapes with the same number of elements: the pool hands the same blocks back, so buffer addresses
    and sizes repeat while the extents differ. A captured graph holds launch parameters derived from the extents and
    must not be replayed for the other shape."""
    x = cgt.matrix("x")
    y = cgt.tanh(x).sum(axis=1)
    f = cgt.function([x], y)
    rs = np.random.RandomState(5)
    for shape in [(4, 6)] * 4 + [(6, 4)] + [(4, 6)] + [(6, 4)] * 4 + [(4, 6)] * 2 + [(2, 12), (12, 2), (2, 12)]:
        xv = rs.randn(*shape).astype("f4")
        got = f(xv)
        assert got.shape == (shape[0],)
        np.testing.assert_allclose(got, np.tanh(xv).sum(axis=1), rtol=1e-4, atol=1e-5)


def test_no_cpu_fallback(rt):
    """Tensor work placed on the host is refused, not emulated."""
    with cgt.scoped_update_config(default_device=cgt.Device("cpu", 0)):
        x = cgt.matrix("x", fixed_shape=(100, 100))
        y = cgt.exp(x)
    f = cgt.function([x], y)
    with pytest.raises(Exception, match="no CPU implementation"):
        f(np.zeros((100, 100), "f4"))


@pytest.mark.parametrize("name,generated", [("mlp", True), ("cifar", True), ("vae", True), ("lstm", True), ("cifar", False),
                                            ("lstm", False)])
def test_elementwise_fusion_changes_no_bit(rt, name, generated):
    """The compiler's fused elementwise chains carry out every operation as the separate kernels do:
    with fusion on and off the losses and the updated parameters are identical, and fusion did happen.
    generated=True: kernels generated per chain; False: the library's register-machine kernel."""
    results = {}
    for fuse in (False, True):
        # padded column rows and the convolutions without a column matrix need the fused output stage, which needs the
        # fused chains, and they change the order of the sums: off on both sides here
        # (the row chains sum in another order as well: off)
        with cgt.scoped_update_config(fuse_elementwise=fuse, jit_fused_elementwise=generated, pad_conv_columns=False,
                                      fuse_conv_implicit=False, fuse_conv_direct=False, fuse_rows=False, use_cuda_graphs=False):
            cfg = configs.BUILDERS[name](**SMALL[name])
            f = cfg.compile()
            n_fused = sum(1 for instr in f.eg.instrs if "FusedElwise" in repr(instr))
            batches = [cfg.batch(seed) for seed in range(2)]
            losses = [np.asarray(f(*batches[i % 2])[0]).copy() for i in range(4)]
            params = [np.asarray(p.op.get_value()).copy() for p in cfg.params]
            results[fuse] = (n_fused, len(f.eg.instrs), losses, params)
    assert results[False][0] == 0 and results[True][0] > 0
    assert results[True][1] < results[False][1]
    for (a, b) in zip(results[False][2], results[True][2]):
        assert np.array_equal(a, b)
    for (a, b) in zip(results[False][3], results[True][3]):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("name", ["mlp", "cifar", "lstm"])
def test_row_fusion_matches_separate_kernels(rt, name):
    """Softmax, its logarithm and its pullback as one FusedRows launch per [batch, classes] matrix: the row sums are
    taken in another order than the reduction kernel's, so losses and parameters agree to rounding, not bit for bit."""
    results = {}
    for fuse in (False, True):
        with cgt.scoped_update_config(fuse_rows=fuse, use_cuda_graphs=False):
            cfg = configs.BUILDERS[name](**SMALL[name])
            f = cfg.compile()
            n_rows = sum(1 for instr in f.eg.instrs if "FusedRows" in repr(instr))
            batches = [cfg.batch(seed) for seed in range(2)]
            losses = [np.asarray(f(*batches[i % 2])[0]).copy() for i in range(4)]
            params = [np.asarray(p.op.get_value()).copy() for p in cfg.params]
            results[fuse] = (n_rows, len(f.eg.instrs), losses, params)
    assert results[False][0] == 0 and results[True][0] > 0
    assert results[True][1] < results[False][1]
    for (a, b) in zip(results[False][2], results[True][2]):
        np.testing.assert_allclose(a, b, rtol=2e-5)
    for (a, b) in zip(results[False][3], results[True][3]):
        np.testing.assert_allclose(a, b, rtol=1e-4, atol=1e-6 * max(1.0, float(np.abs(a).max())))


@pytest.mark.parametrize("name", ["mlp", "cifar"])
@pytest.mark.parametrize("generated", [True, False])
def test_flat_index_rows_substitution(rt, name, generated):
    """logprobs[arange(batch), y] and its gradient inside the softmax row chain (the labels are read by the FusedRows
    kernel; no index arithmetic, zero fill, increment or gather is launched): the selected elements are the same
    numbers, so the losses agree to the last bits of the row-sum order and the parameters to float32 tolerance;
    fewer kernels per step. generated: the kernel generated for the chain / the library's register machine."""
    res = {}
    for on in (False, True):
        with cgt.scoped_update_config(fuse_flat_index_rows=on, jit_fused_elementwise=generated, use_cuda_graphs=False):
            cfg = configs.BUILDERS[name](**SMALL[name])
            f = cfg.compile()
            reprs = [repr(i) for i in f.eg.instrs]
            batches = [cfg.batch(seed) for seed in range(2)]
            losses = [float(f(*batches[i % 2])[0]) for i in range(6)]
            res[on] = (reprs, losses, [np.asarray(p.op.get_value()).copy() for p in cfg.params], f.stats()["last_kernel_launches"])
    assert any("FlatIndices" in r for r in res[False][0]) and not any("FlatIndices" in r for r in res[True][0])
    assert res[True][3] <= res[False][3] - 3
    np.testing.assert_allclose(res[True][1], res[False][1], rtol=1e-5)
    for (a, b) in zip(res[False][2], res[True][2]):
        np.testing.assert_allclose(a, b, rtol=1e-3, atol=1e-5 * max(1.0, float(np.abs(a).max())))


@pytest.mark.parametrize("name", ["cifar", "wide"])
def test_filter_splits_hoisted_change_no_bit(rt, name):
    """The [w_hi | w_lo] copies of all filter banks made by one SplitFilterBanks launch at the head of the step instead of
    one small kernel inside every convolution call: the same copies, so losses and parameters are identical; fewer
    kernels per step."""
    res = {}
    for on in (False, True):
        with cgt.scoped_update_config(hoist_filter_splits=on, use_cuda_graphs=False):
            cfg = configs.BUILDERS[name](**SMALL[name])
            f = cfg.compile()
            reprs = [repr(i) for i in f.eg.instrs]
            batches = [cfg.batch(seed) for seed in range(2)]
            losses = [np.asarray(f(*batches[i % 2])[0]).copy() for i in range(5)]
            res[on] = (reprs, losses, [np.asarray(p.op.get_value()).copy() for p in cfg.params], f.stats()["last_kernel_launches"])
    n_split = sum("op:SplitFilterBanks" in r for r in res[True][0])
    assert n_split == 1 and not any("SplitFilterBanks" in r for r in res[False][0])
    assert res[True][3] < res[False][3]
    for (a, b) in zip(res[False][1], res[True][1]):
        assert np.array_equal(a, b)
    for (a, b) in zip(res[False][2], res[True][2]):
        assert np.array_equal(a, b)


def test_product_sums_in_the_output_stage_change_no_bit(rt):
    """(x.W + b) + (h.U + c) with the three additions in the output stage of the product h.U (fuse_product_sums): the
    additions keep their association, so the LSTM's losses and parameters are identical; one launch less per layer and
    time step."""
    results = {}
    for on in (False, True):
        with cgt.scoped_update_config(fuse_product_sums=on, use_cuda_graphs=False):
            cfg = configs.BUILDERS["lstm"](seq_len=6, batch=64)
            f = cfg.compile()
            reprs = [repr(i) for i in f.eg.instrs]
            batches = [cfg.batch(seed) for seed in range(2)]
            losses = [np.asarray(f(*batches[i % 2])[0]).copy() for i in range(4)]
            params = [np.asarray(p.op.get_value()).copy() for p in cfg.params]
            results[on] = (reprs, f.stats()["last_kernel_launches"], losses, params)
    assert sum("op:Mul22BiasAdd" in r for r in results[True][0]) == 2 * 6 and not any("Mul22BiasAdd" in r for r in results[False][0])
    assert results[True][1] <= results[False][1] - 2 * 6
    for (a, b) in zip(results[False][2], results[True][2]):
        assert np.array_equal(a, b)
    for (a, b) in zip(results[False][3], results[True][3]):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("generated", [True, False])
def test_gate_columns_split_changes_no_bit(rt, generated):
    """The LSTM's gate arithmetic written per gate on [batch, hidden] blocks (split_gate_columns) instead of on slabs of
    the [batch, 4 * hidden] pre-activation: elementwise work on the same elements, so losses and parameters are
    identical; one chain then holds a whole cell, and far fewer kernels are launched per step."""
    results = {}
    for on in (False, True):
        with cgt.scoped_update_config(split_gate_columns=on, jit_fused_elementwise=generated, use_cuda_graphs=False):
            cfg = configs.BUILDERS["lstm"](**SMALL["lstm"])
            f = cfg.compile()
            batches = [cfg.batch(seed) for seed in range(2)]
            losses = [np.asarray(f(*batches[i % 2])[0]).copy() for i in range(4)]
            params = [np.asarray(p.op.get_value()).copy() for p in cfg.params]
            results[on] = (f.stats()["last_kernel_launches"], losses, params)
    assert results[True][0] < 0.9 * results[False][0]
    for (a, b) in zip(results[False][1], results[True][1]):
        assert np.array_equal(a, b)
    for (a, b) in zip(results[False][2], results[True][2]):
        assert np.array_equal(a, b)


def test_conv_direct_substitution(rt):
    """The compiler computes the 3-channel first layer of the CIFAR-shape convnet directly from the image (no column
    matrix): losses and parameters stay within the float32 tolerance of the column-matrix graph."""
    res = {}
    for fuse in (False, True):
        with cgt.scoped_update_config(fuse_conv_direct=fuse, use_cuda_graphs=False):
            cfg = configs.build_cifar(batch=16)
            f = cfg.compile()
            reprs = [repr(i) for i in f.eg.instrs]
            losses = [float(f(*cfg.batch(s))[0]) for s in range(4)]
            res[fuse] = (reprs, losses, [np.asarray(p.op.get_value()).copy() for p in cfg.params])
    assert any("ConvDirectFwd" in r for r in res[True][0]) and any("ConvDirectWgradRelu" in r for r in res[True][0])
    # the first layer's channels-last gradient is never formed: one ReluGradNHWC per later layer is left
    assert sum("op:ReluGradNHWC" in r for r in res[True][0]) == sum("op:ReluGradNHWC" in r for r in res[False][0]) - 1
    assert not any("Im2Col" in r for r in res[True][0]) and any("Im2Col" in r for r in res[False][0])
    np.testing.assert_allclose(res[True][1], res[False][1], rtol=1e-4)
    for (a, b) in zip(res[False][2], res[True][2]):
        np.testing.assert_allclose(a, b, rtol=1e-3, atol=1e-5 * max(1.0, float(np.abs(a).max())))


@pytest.mark.parametrize("generated", [True, False])
def test_slice_rewrites_change_no_bit(rt, generated):
    """The LSTM's gate slices: column slices read in place by the fused chains (no GetSli launch) and the gradient of the
    slices placed by one ScatterCols launch (no zero fills, slice increments and additions). Placing a piece next to
    zeros and adding it to zeros give the same values, and a view reads the same words: losses and parameters are
    identical with the rewrites on and off. generated: kernels generated per chain / the library's register machine."""
    results = {}
    for on in (False, True):
        with cgt.scoped_update_config(fuse_slice_sums=on, fuse_slice_views=on, jit_fused_elementwise=generated, use_cuda_graphs=False):
            cfg = configs.BUILDERS["lstm"](**SMALL["lstm"])
            f = cfg.compile()
            reprs = [repr(instr) for instr in f.eg.instrs]
            batches = [cfg.batch(seed) for seed in range(2)]
            losses = [np.asarray(f(*batches[i % 2])[0]).copy() for i in range(4)]
            params = [np.asarray(p.op.get_value()).copy() for p in cfg.params]
            results[on] = (reprs, losses, params)
    assert not any("ScatterCols" in r for r in results[False][0]) and any("ScatterCols" in r for r in results[True][0])
    n_getsli = [sum(1 for r in results[on][0] if "GetSli" in r and "/gpu" in r) for on in (False, True)]
    assert n_getsli[1] < n_getsli[0]
    assert len(results[True][0]) < len(results[False][0])
    for (a, b) in zip(results[False][1], results[True][1]):
        assert np.array_equal(a, b)
    for (a, b) in zip(results[False][2], results[True][2]):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("name", ["mlp", "cifar", "lstm"])
def test_merged_parameter_updates_change_no_bit(rt, name):
    """The step's parameter updates as one multi-tensor launch: the same operations on the same values as one launch
    per parameter, so losses and parameters are identical."""
    results = {}
    for merge in (False, True):
        with cgt.scoped_update_config(merge_parameter_updates=merge, use_cuda_graphs=False):
            cfg = configs.BUILDERS[name](**SMALL[name])
            f = cfg.compile()
            n_multi = sum(1 for instr in f.eg.instrs if "MultiFusedElwise" in repr(instr))
            batches = [cfg.batch(seed) for seed in range(2)]
            losses = [np.asarray(f(*batches[i % 2])[0]).copy() for i in range(4)]
            params = [np.asarray(p.op.get_value()).copy() for p in cfg.params]
            results[merge] = (n_multi, len(f.eg.instrs), losses, params)
    assert results[False][0] == 0 and results[True][0] >= 1
    assert results[True][1] < results[False][1]
    for (a, b) in zip(results[False][2], results[True][2]):
        assert np.array_equal(a, b)
    for (a, b) in zip(results[False][3], results[True][3]):
        assert np.array_equal(a, b)


def test_conv_dgrad_substitution(rt):
    """The compiler replaces Mul22 + Col2Im of the stride-1 convolutions' data gradients by ConvDgrad; the
    losses and parameters stay within the float32 tolerance of the Op-by-Op graph."""
    res = {}
    for fuse in (False, True):
        with cgt.scoped_update_config(fuse_conv_dgrad=fuse, use_cuda_graphs=False):
            cfg = configs.BUILDERS["cifar"](**SMALL["cifar"])
            f = cfg.compile()
            names = [repr(instr) for instr in f.eg.instrs]
            batches = [cfg.batch(seed) for seed in range(2)]
            losses = [float(f(*batches[i % 2])[0]) for i in range(6)]
            params = [np.asarray(p.op.get_value()).copy() for p in cfg.params]
            res[fuse] = (sum("ConvDgrad" in n for n in names), sum("Col2Im" in n for n in names), losses, params)
    assert res[False][0] == 0 and res[True][0] == 2 and res[True][1] == 0
    np.testing.assert_allclose(res[True][2], res[False][2], rtol=1e-4)
    for (a, b) in zip(res[True][3], res[False][3]):
        np.testing.assert_allclose(a, b, rtol=1e-3, atol=1e-5)


def test_conv_output_substitution_changes_no_bit(rt):
    """ConvBiasRelu (GEMM + NCHW + bias + relu in one call) gives the bits of the Op sequence it replaces."""
    res = {}
    for fuse in (False, True):
        # padded column rows apply only next to ConvBiasRelu and change which product kernel runs: off here; the
        # convolutions without a column matrix sum in another order: off here too
        with cgt.scoped_update_config(fuse_conv_output=fuse, pad_conv_columns=False, fuse_conv_implicit=False, fuse_conv_direct=False, use_cuda_graphs=False):
            cfg = configs.BUILDERS["cifar"](**SMALL["cifar"])
            f = cfg.compile()
            names = [repr(instr) for instr in f.eg.instrs]
            batches = [cfg.batch(seed) for seed in range(2)]
            losses = [np.asarray(f(*batches[i % 2])[0]).copy() for i in range(4)]
            params = [np.asarray(p.op.get_value()).copy() for p in cfg.params]
            res[fuse] = (sum("ConvBiasRelu" in n for n in names), losses, params)
    assert res[False][0] == 0 and res[True][0] == 3
    for (a, b) in zip(res[False][1], res[True][1]):
        assert np.array_equal(a, b)
    for (a, b) in zip(res[False][2], res[True][2]):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("name,n_padded", [("cifar", 1), ("wide", 1)])
def test_padded_column_rows(rt, name, n_padded):
    """The first convolution's column matrix (rows of 75 / 363 entries) gets rows of 76 / 364 entries, its products
    become ConvBiasRelu on the padded matrix and ConvWgrad; losses and parameters stay within float32 tolerance."""
    res = {}
    for pad in (False, True):
        with cgt.scoped_update_config(pad_conv_columns=pad, fuse_conv_direct=False, use_cuda_graphs=False):
            cfg = configs.BUILDERS[name](**SMALL[name])
            f = cfg.compile()
            names = [repr(instr) for instr in f.eg.instrs]
            batches = [cfg.batch(seed) for seed in range(2)]
            losses = [float(f(*batches[i % 2])[0]) for i in range(6)]
            params = [np.asarray(p.op.get_value()).copy() for p in cfg.params]
            res[pad] = (sum("/pitch" in n for n in names), sum("ConvWgrad{" in n for n in names), losses, params)
    assert res[False][:2] == (0, 0) and res[True][:2] == (n_padded, n_padded)
    np.testing.assert_allclose(res[True][2], res[False][2], rtol=1e-4)
    for (a, b) in zip(res[True][3], res[False][3]):
        np.testing.assert_allclose(a, b, rtol=1e-3, atol=1e-5)


@pytest.mark.parametrize("graphs", [False, True])
def test_prefetched_inputs_give_the_same_steps(rt, graphs):
    """f.prefetch(next batch) before f(batch) uploads on the copy stream; losses and parameters are those of the
    plain calls bit for bit, also when a prefetched batch is never consumed or a batch is called without prefetch."""
    from cgt_b200 import runtime
    res = {}
    for pre in (False, True):
        with cgt.scoped_update_config(use_cuda_graphs=graphs):
            cfg = configs.BUILDERS["cifar"](**SMALL["cifar"])
            f = cfg.compile()
            batches = []
            for seed in range(3):
                pinned = []
                for a in cfg.batch(seed):
                    p = runtime.pinned_empty(a.shape, a.dtype)
                    p[...] = a
                    pinned.append(p)
                batches.append(pinned)
            order = [0, 1, 2, 0, 0, 2, 1, 1]
            losses = []
            if pre:
                f.prefetch(*batches[order[0]])
            for (i, b) in enumerate(order):
                if pre and i + 1 < len(order) and i != 3:   # step 4 runs without a prefetched batch
                    f.prefetch(*batches[order[i + 1]])
                if pre and i == 5:
                    f.prefetch(*batches[0])                  # replaces the upload queued for step 6: never consumed
                losses.append(np.asarray(f(*batches[b])[0]).copy())
            res[pre] = (losses, [np.asarray(p.op.get_value()).copy() for p in cfg.params])
    for (a, b) in zip(res[False][0], res[True][0]):
        assert np.array_equal(a, b)
    for (a, b) in zip(res[False][1], res[True][1]):
        assert np.array_equal(a, b)


def test_conv_grad_input_substitution(rt):
    """ReluGradNHWC replaces multiply + Transpose{0,2,3,1} + Sum{0,2,3}; only the bias gradients' summation order
    changes, so losses and parameters agree to float32 tolerance."""
    res = {}
    for fuse in (False, True):
        with cgt.scoped_update_config(fuse_conv_grad_input=fuse, fuse_conv_direct=False, use_cuda_graphs=False):
            cfg = configs.BUILDERS["cifar"](**SMALL["cifar"])
            f = cfg.compile()
            names = [repr(instr) for instr in f.eg.instrs]
            batches = [cfg.batch(seed) for seed in range(2)]
            losses = [float(f(*batches[i % 2])[0]) for i in range(6)]
            params = [np.asarray(p.op.get_value()).copy() for p in cfg.params]
            res[fuse] = (sum("ReluGradNHWC" in n for n in names), losses, params)
    assert res[False][0] == 0 and res[True][0] == 3
    np.testing.assert_allclose(res[True][1], res[False][1], rtol=1e-4)
    for (a, b) in zip(res[True][2], res[False][2]):
        np.testing.assert_allclose(a, b, rtol=1e-3, atol=1e-5)


@pytest.mark.parametrize("name", ["cifar", "vae"])
@pytest.mark.parametrize("graphs", [False, True])
def test_checkpoint_resume_is_bit_exact(rt, tmp_path, name, graphs):
    """save -> 5 steps, reload -> the same 5 steps: losses and every shared variable (parameters, Adam slots and step
    counter for the VAE) identical bit for bit, eagerly and from captured CUDA graphs. The reload writes into the
    variables' existing device buffers, so the captured graphs stay valid."""
    from cgt_b200 import checkpoint
    with cgt.scoped_update_config(use_cuda_graphs=graphs):
        cfg = configs.BUILDERS[name](**SMALL[name])
        f = cfg.compile()
        variables = cfg.state_variables()
        batches = [cfg.batch(seed) for seed in range(3)]
        for i in range(4):   # leave the initial state (and reach graph replay) before the checkpoint
            f(*batches[i % 3])
        path = str(tmp_path / "ckpt.npz")
        checkpoint.save_state(path, variables, extra={"step": 4})
        first = [np.asarray(f(*batches[i % 3])[0]).copy() for i in range(4, 9)]
        state1 = [v.op.get_value() for v in variables]
        assert checkpoint.load_state(path, variables) == {"step": 4}
        second = [np.asarray(f(*batches[i % 3])[0]).copy() for i in range(4, 9)]
        state2 = [v.op.get_value() for v in variables]
    for (a, b) in zip(first, second):
        assert np.array_equal(a, b)
    for (a, b) in zip(state1, state2):
        assert np.array_equal(a, b)
    assert not np.array_equal(first[0], first[4])  # the steps did change the model


class ScaleShiftCuda(core.Op):
    """A user-defined Op that brings its own CUDA source (reference contract: NativeCompileInfo with extra_srcs =
    [SrcFile("cuda", ...)], $function / $closure templating, cgt/core.py:734-769; the pattern of
    cgt/tests/test_par_interp.py:11-27 and test_multi_output.py:32-58 with devtype "gpu")."""
    available_impls = ("native_gpu",)

    def __init__(self, scale, shift):
        self.scale, self.shift = float(scale), float(shift)

    def typ_apply(self, input_types):
        return input_types[0]

    def shp_apply(self, inputs):
        return cgt.shape(inputs[0])

    def get_native_compile_info(self, input_types, devtype):
        assert devtype == "gpu"
        code = r"""
            extern "C" void ${function}_launch(const float* x, float* y, long n, float a, float b, void* stream);
            CGT_EXPORT_C void $function($closure* cl, cgtArray** reads, cgtArray* write) {
                ${function}_launch((const float*)reads[0]->data(), (float*)write->data(), (long)reads[0]->size(),
                                   cl->scale, cl->shift, cgt_current_stream());
            }"""
        cuda = r"""
            #include <cuda_runtime.h>
            __global__ void ${function}_kernel(const float* x, float* y, long n, float a, float b) {
                for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
                    y[i] = __fmaf_rn(a, x[i], b);
            }
            extern "C" void ${function}_launch(const float* x, float* y, long n, float a, float b, void* stream) {
                if (n <= 0) return;
                int blocks = (int)((n + 255) / 256);
                if (blocks > 1184) blocks = 1184;
                ${function}_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(x, y, n, a, b);
            }"""
        return core.NativeCompileInfo(code, closure_triples=[("scale", ctypes.c_float, self.scale), ("shift", ctypes.c_float, self.shift)],
                                      extra_srcs=[core.SrcFile("cuda", cuda)])


@pytest.mark.parametrize("graphs", [False, True])
def test_user_op_with_cuda_source_runs_on_the_gpu(rt, graphs):
    """The Op's CUDA source is compiled by nci2callable (nvcc, sm_100a) into the hash-keyed cache, the node is placed on
    the GPU, its kernel is launched on the runtime stream and therefore lands inside the captured span."""
    with cgt.scoped_update_config(use_cuda_graphs=graphs):
        x = cgt.matrix("x", fixed_shape=(37, 129))
        h = core.Result(ScaleShiftCuda(2.5, -1.0), [cgt.tanh(x)])
        y = (h * h).sum(axis=1)
        f = cgt.function([x], [y, h])
        assert any("ScaleShiftCuda" in repr(i) and i.write_loc.devtype == "gpu" for i in f.eg.instrs if hasattr(i, "op"))
        rs = np.random.RandomState(2)
        for _ in range(5):
            xv = rs.randn(37, 129).astype("f4")
            (gy, gh) = f(xv)
            want_h = np.float32(2.5) * np.tanh(xv) + np.float32(-1.0)
            np.testing.assert_allclose(gh, want_h, rtol=1e-5, atol=1e-6)
            np.testing.assert_allclose(gy, (want_h.astype("f8") ** 2).sum(axis=1), rtol=1e-4)
        if graphs:
            st = f.stats()
            assert st["segments_captured"] >= 1 and st["last_graph_launches"] >= 1, st


@pytest.mark.parametrize("name", ["cifar", "wide"])
def test_conv_implicit_substitution(rt, name):
    """ConvFwdBiasRelu / ConvWgradImplicit replace Im2Col + ConvBiasRelu + Mul22{T,N} for the stride-1 convolutions with
    32-channel-aligned inputs (CIFAR conv2 and conv3, the wide net's conv2): those column matrices disappear; losses and
    parameters stay within float32 tolerance of the graph that keeps them."""
    res = {}
    for fuse in (False, True):
        with cgt.scoped_update_config(fuse_conv_implicit=fuse, fuse_conv_direct=False, use_cuda_graphs=False):
            cfg = configs.BUILDERS[name](**SMALL[name])
            f = cfg.compile()
            names = [repr(instr) for instr in f.eg.instrs]
            batches = [cfg.batch(seed) for seed in range(2)]
            losses = [float(f(*batches[i % 2])[0]) for i in range(6)]
            params = [np.asarray(p.op.get_value()).copy() for p in cfg.params]
            res[fuse] = (sum("ConvFwdBiasRelu" in n for n in names), sum("ConvWgradImplicit" in n for n in names),
                         sum("op:Im2Col" in n for n in names), losses, params)
    n_conv = {"cifar": 2, "wide": 1}[name]
    assert res[False][:2] == (0, 0) and res[True][:2] == (n_conv, n_conv)
    assert res[False][2] == n_conv + 1 and res[True][2] == 1   # only the 3-channel first layer keeps its column matrix
    np.testing.assert_allclose(res[True][3], res[False][3], rtol=1e-4)
    for (a, b) in zip(res[True][4], res[False][4]):
        np.testing.assert_allclose(a, b, rtol=1e-3, atol=1e-5)
