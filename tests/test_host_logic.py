"""CPU tests of the host side (no GPU): the C-ABI library and its symbols, the graph front-end
(simplifier, autodiff), the compilation pipeline up to the execution graph, run-time compilation of
Ops that carry C++ source, and the configuration dictionary. Numerics are evaluated with the CPU
oracle; nothing here touches a device.
"""
import ctypes
import os
import os.path as osp
import re

import numpy as np
import pytest

import cgt_b200 as cgt
from cgt_b200 import compilation, configs, core, nn, runtime
from oracle import cpu_backend

ROOT = osp.dirname(osp.dirname(osp.abspath(__file__)))


# ------------------------------------------------------------------------------------------------
# C ABI
# ------------------------------------------------------------------------------------------------
def _declared_symbols():
    text = open(osp.join(ROOT, "include", "cgt_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cgtb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = runtime.lib()
    names = _declared_symbols()
    assert len(names) > 60
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    # every symbol the Python side binds is declared in the header
    undeclared = [n for n in runtime.C_ABI_SYMBOLS if n not in names]
    assert not undeclared, undeclared


def test_builtin_op_callables_are_exported():
    lib = runtime.lib()
    for name in ("elwise_unary", "elwise_binary", "mul22", "batched_mul22", "im2col", "col2im", "max_pool", "max_pool_pullback",
                 "lrn_forward", "lrn_backward", "reduce", "repeat", "transpose", "getsli", "incsli", "getflat", "incflat",
                 "concatenate", "fill", "constant", "transport", "reshape", "size", "arange", "tuple_index", "in_memory_data",
                 "allreduce"):
        assert hasattr(lib, "cgtb_op_" + name), name


def test_compute_entry_points_fail_loudly_without_a_gpu():
    lib = runtime.lib()
    if lib.cgtb_initialized():
        pytest.skip("a GPU is bound in this process")
    buf = (ctypes.c_float * 4)()
    rc = lib.cgtb_unary(3, 11, 11, 4, buf, buf)
    assert rc != 0 and "no CPU fallback" in runtime.last_error()
    assert lib.cgtb_array_new(1, (ctypes.c_long * 1)(4), 11, runtime.GPU) is None
    with pytest.raises(runtime.BackendError):
        runtime.device_array(np.zeros(3, "f4"))


def test_host_objects_round_trip():
    a = np.arange(6, dtype="f4").reshape(2, 3)
    h, keep = runtime.py2cgt_array(a, runtime.CPU, view=True)
    lib = runtime.lib()
    assert lib.cgtb_array_ndim(h) == 2 and lib.cgtb_array_dtype(h) == 11 and lib.cgtb_array_devtype(h) == 0
    assert np.array_equal(runtime.cgt2py_object(h), a)
    t = lib.cgtb_tuple_new(2)
    lib.cgtb_tuple_set(t, 0, h)
    lib.cgtb_tuple_set(t, 1, h)
    assert lib.cgtb_tuple_len(t) == 2
    out = runtime.cgt2py_object(t)
    assert isinstance(out, tuple) and np.array_equal(out[1], a)
    lib.cgtb_release(t)
    lib.cgtb_release(h)


# ------------------------------------------------------------------------------------------------
# front-end
# ------------------------------------------------------------------------------------------------
def test_simplifier_folds_shapes_and_constants():
    x = cgt.matrix("x", fixed_shape=(4, 3))
    y = (x * 1.0 + 0.0).sum(axis=0)
    assert cgt.infer_shape(y) == (3,)
    (s,) = cgt.simplify([cgt.size(x, 0) * cgt.size(x, 1)])
    assert isinstance(s.op, core.Constant) and int(s.op.value) == 12
    # x*1 and +0 vanish; common subexpressions merge
    a = cgt.exp(x) + cgt.exp(x)
    (sa,) = cgt.simplify([a])
    assert sa.parents[0] is sa.parents[1]
    (sy,) = cgt.simplify([x * 1.0])
    assert sy is x or sy.is_argument()


def test_broadcast_requires_explicit_pattern():
    x = cgt.matrix("x", fixed_shape=(4, 3))
    b = cgt.matrix("b", fixed_shape=(1, 3))
    z = cgt.broadcast("+", x, b, "xx,1x")
    f = cpu_backend.function([x, b], z)
    xv, bv = np.arange(12, dtype="f4").reshape(4, 3), np.float32([[1, 2, 3]])
    assert np.array_equal(f(xv, bv), xv + bv)
    with pytest.raises(AssertionError):
        cgt.vector("v") + x  # rank mismatch: no implicit broadcasting


def test_pullback_sums_in_order_and_matches_finite_differences():
    with cgt.scoped_update_config(precision="double"):
        x = cgt.matrix("x", fixed_shape=(3, 4))
        w = cgt.matrix("w", fixed_shape=(4, 2))
        y = cgt.tanh(x.dot(w))
        cost = (y * y).sum() + cgt.sigmoid(y).sum() + (cgt.exp(x) / 3.0).sum()
        gx, gw = cgt.grad(cost, [x, w])
        f = cpu_backend.function([x, w], [cost, gx, gw])
        rs = np.random.RandomState(0)
        xv, wv = rs.randn(3, 4), rs.randn(4, 2)
        c0, gxv, gwv = f(xv, wv)
        eps = 1e-6
        for (arr, g) in ((xv, gxv), (wv, gwv)):
            for idx in [(0, 0), (1, 1), (2, 1)]:
                old = arr[idx]
                arr[idx] = old + eps
                cp = f(xv, wv)[0]
                arr[idx] = old - eps
                cm = f(xv, wv)[0]
                arr[idx] = old
                assert abs((cp - cm) / (2 * eps) - g[idx]) < 1e-6


def test_convnet_gradients_match_independent_autograd():
    """Independent cross-check of the autodiff and of the conv / pool / LRN Ops: PyTorch float64 autograd
    on the same network (sizes chosen so that the pooled extent agrees with PyTorch's formula)."""
    torch = pytest.importorskip("torch")
    import torch.nn.functional as F
    with cgt.scoped_update_config(precision="double"):
        rs = np.random.RandomState(3)
        B = 3
        X = cgt.tensor4("X", fixed_shape=(B, 2, 12, 12))
        y = cgt.vector("y", dtype="i8", fixed_shape=(B,))
        Wv, bv = rs.randn(6, 2, 5, 5) * 0.3, rs.randn(1, 6, 1, 1) * 0.1
        Vv, cv = rs.randn(6 * 5 * 5, 4) * 0.2, rs.randn(1, 4) * 0.1
        W, b = cgt.shared(Wv, fixed_shape_mask="all"), cgt.shared(bv, fixed_shape_mask="all")
        V, c = cgt.shared(Vv, fixed_shape_mask="all"), cgt.shared(cv, fixed_shape_mask="all")
        h = nn.rectify(cgt.broadcast("+", nn.conv2d(X, W, (5, 5), (2, 2)), b, "xxxx,1x11"))
        h = nn.max_pool_2d(h, (3, 3), stride=(2, 2))          # 12 -> ceil(9/2) = 5, as PyTorch's floor(9/2)+1
        h = nn.cross_channel_lrn(h, 5, 1e-2, 0.75)
        flat = h.reshape([B, 6 * 5 * 5])
        logits = cgt.broadcast("+", flat.dot(V), c, "xx,1x")
        loss = -cgt.log(nn.softmax(logits))[cgt.arange(B), y].mean()
        grads = cgt.grad(loss, [W, b, V, c])
        f = cpu_backend.function([X, y], [loss] + grads)
        Xv, yv = rs.randn(B, 2, 12, 12), rs.randint(0, 4, size=B)
        got = f(Xv, yv)

        tW, tb, tV, tc = [torch.tensor(v, requires_grad=True) for v in (Wv, bv, Vv, cv)]
        th = F.relu(F.conv2d(torch.tensor(Xv), tW, padding=2) + tb)
        th = F.max_pool2d(th, 3, 2)
        th = F.local_response_norm(th, 5, alpha=1e-2, beta=0.75, k=1.0)
        tl = F.cross_entropy(th.reshape(B, -1) @ tV + tc, torch.tensor(yv))
        tl.backward()
        np.testing.assert_allclose(got[0], tl.item(), rtol=1e-10)
        for (g, t) in zip(got[1:], (tW, tb, tV, tc)):
            np.testing.assert_allclose(g, t.grad.numpy(), rtol=1e-8, atol=1e-10)


def test_update_semantics_on_the_oracle():
    """sgd on scale*x^2 from 1.0 (reference test_optimizers.py golden values)."""
    for (scale, want) in zip([0.1, 0.2, 0.3], [0.81707280688755, 0.6648326359915, 0.5386151140949]):
        A = cgt.shared(np.array([1.0], "f4"))
        cost = (scale * A ** 2).sum()
        step = cpu_backend.function([], [], updates=nn.sgd(cost, [A], 0.1))
        for _ in range(10):
            step()
        np.testing.assert_allclose(step.get_value(A), want, rtol=1e-5)


# ------------------------------------------------------------------------------------------------
# compilation pipeline (everything before the native interpreter is created)
# ------------------------------------------------------------------------------------------------
def _plan(cfg):
    outs, srcs, targs, analysis = compilation.simplify_for_execution([cfg.loss], cfg.updates)
    all_out = outs + targs
    nodelist = core.topsorted(all_out)
    node2dev = compilation.determine_devices(nodelist, dict(zip(targs, srcs)))
    compilation.add_transports(nodelist, node2dev, analysis["node2shape"])
    updates = list(zip(srcs, targs))
    extra = compilation._update_control_deps(all_out, updates)
    order = compilation.topsorted_shapes_first(all_out, analysis["node2shape"], extra)
    const = compilation.compute_const_nodes(order)
    owner = compilation.determine_memowner(order, updates, node2dev, outs, analysis["node2shape"], const)
    written = set(o for (n, o) in owner.items() if o is not n)
    eg, node2memloc = compilation.create_execution_graph(cfg.inputs, order, analysis["node2shape"], owner, node2dev,
                                                         set(n for n in const if n not in written))
    return dict(outs=outs, srcs=srcs, targs=targs, order=order, node2dev=node2dev, owner=owner, eg=eg, memloc=node2memloc)


def test_placement_transports_and_memory_owners():
    cfg = configs.build_cifar(batch=4)
    pl = _plan(cfg)
    for node in pl["order"]:
        dev = pl["node2dev"][node]
        if isinstance(node.op, core.Transport):
            continue  # the device copy of a scalar operand is the one scalar that lives on the GPU
        if node.is_scalar() or node.is_argument():
            assert dev.devtype == "cpu", node
        elif node.is_data():
            assert dev.devtype == "gpu"
    # arguments reach the device through a Transport; every Transport crosses devices
    transports = [n for n in pl["order"] if isinstance(n.op, core.Transport)]
    assert any(t.parents[0].is_argument() for t in transports)
    for t in transports:
        assert pl["node2dev"][t].devtype != pl["node2dev"][t.parents[0]].devtype
    # an update's final op writes into the shared variable's own location
    for (src, targ) in zip(pl["srcs"], pl["targs"]):
        assert pl["owner"][targ] is src
        assert pl["memloc"][targ] is pl["memloc"][src]
    # with fixed shapes every Alloc reads constant shape components, all fired once
    by_loc = {}
    for instr in pl["eg"].instrs:
        by_loc[instr.write_loc.index] = instr
    for instr in pl["eg"].instrs:
        if isinstance(instr, compilation.Alloc):
            for loc in instr.read_locs:
                src = by_loc[loc.index]
                assert isinstance(src.op, core.Constant) and src.once
    kinds = set(type(i).__name__ for i in pl["eg"].instrs)
    assert kinds == {"LoadArgument", "Alloc", "BuildTup", "ReturnByRef", "ReturnByVal"}


def test_odd_column_rows_are_padded_for_both_products():
    """compilation.pad_conv_columns: the column matrix of a 3-channel 5x5 convolution (rows of 75) gets rows of 76,
    its forward product stays ConvBiasRelu on the padded matrix, its filter gradient becomes ConvWgrad{75} with the
    unpadded result shape; the 32-channel layers (rows of 800) are left alone."""
    from cgt_b200.nn_ops import im2col as im2col_ops
    cfg = configs.build_cifar(batch=4)
    outs, _usrc, utargs, analysis = compilation.simplify_for_execution([cfg.loss] + list(cfg.extra_outputs), cfg.updates)
    n2s = analysis["node2shape"]
    o, u = compilation.fuse_conv_dgrad(outs, utargs, n2s)
    o, u = compilation.fuse_conv_grad_input(o, u, n2s)
    o, u = compilation.fuse_elementwise(o, u, n2s)
    o, u = compilation.fuse_conv_output(o, u, n2s)
    before = [n for n in core.topsorted(o + u) if not n.is_input() and isinstance(n.op, core.Mul22) and n.op.tA and not n.op.tB]
    o, u = compilation.pad_conv_columns(o, u, n2s)
    nodes = [n for n in core.topsorted(o + u) if not n.is_input()]
    ims = [n for n in nodes if isinstance(n.op, im2col_ops.Im2Col)]
    assert sorted(n.op.pitch for n in ims) == [0, 0, 76]
    padded = [n for n in ims if n.op.pitch][0]
    assert compilation._static_shape(n2s[padded]) == (4, 32, 32, 76)
    wg = [n for n in nodes if isinstance(n.op, im2col_ops.ConvWgrad)]
    assert len(wg) == 1 and wg[0].op.k == 75 and compilation._static_shape(n2s[wg[0]]) == (32, 75)
    after = [n for n in nodes if isinstance(n.op, core.Mul22) and n.op.tA and not n.op.tB]
    assert len(after) == len(before) - 1
    # both consumers read the one padded matrix
    r = wg[0].parents[1]
    assert isinstance(r.op, core.Reshape) and r.parents[0] is padded and compilation._static_shape(n2s[r]) == (4096, 76)
    fwd = [n for n in nodes if isinstance(n.op, im2col_ops.ConvBiasRelu) and n.parents[0] is r]
    assert len(fwd) == 1
    # a second application finds nothing left to do
    o2, u2 = compilation.pad_conv_columns(o, u, n2s)
    assert [n for n in core.topsorted(o2 + u2) if not n.is_input() and isinstance(n.op, im2col_ops.ConvWgrad)] == wg


def test_convnet_graph_rewrites():
    """The rewrites aimed at the CIFAR-shape convnet, on its batch-16 graph (no GPU needed: only the rewritten graph is
    inspected). No column matrix is left: the 3-channel first layer is computed directly (ConvDirectFwd, and
    ConvDirectWgradRelu, which absorbs that layer's relu and bias gradients), conv2 / conv3 are implicit convolutions
    whose filter banks are split by one SplitFilterBanks node with four jobs; the softmax loss with the label selection
    and its pullback is one FusedRows node; every switch turns its rewrite off."""
    from cgt_b200.nn_ops import im2col as im2col_ops
    cfg = configs.build_cifar(batch=16)

    def rewritten(**flags):
        with cgt.scoped_update_config(**flags):
            sim = compilation.simplify_for_execution([cfg.loss] + list(cfg.extra_outputs), cfg.updates)
            o, u = compilation.apply_graph_rewrites(sim[0], sim[2], sim[3]["node2shape"])
        return [n for n in core.topsorted(o + u) if not n.is_input()]     # topsorted raises on a cycle

    nodes = rewritten()
    count = lambda ns, cls: sum(1 for n in ns if isinstance(n.op, cls))
    assert count(nodes, im2col_ops.Im2Col) == 0 and count(nodes, im2col_ops.Col2Im) == 0
    assert count(nodes, im2col_ops.ConvDirectFwd) == 1 and count(nodes, im2col_ops.ConvDirectWgradRelu) == 1
    assert count(nodes, im2col_ops.ConvFwdBiasRelu) == 2 and count(nodes, im2col_ops.ConvDgrad) == 2
    assert count(nodes, im2col_ops.ConvWgradImplicit) == 2 and count(nodes, im2col_ops.ReluGradNHWC) == 2
    splits = [n for n in nodes if isinstance(n.op, im2col_ops.SplitFilterBanks)]
    assert len(splits) == 1 and len(splits[0].op.jobs) == 4 and len(splits[0].parents) == 2
    assert sorted(job[4] for job in splits[0].op.jobs) == [1, 1, 2, 2]       # two forward products, two data gradients
    assert all(n.op.pre and len(n.parents) == (8 if isinstance(n.op, im2col_ops.ConvFwdBiasRelu) else 7)
               for n in nodes if isinstance(n.op, (im2col_ops.ConvFwdBiasRelu, im2col_ops.ConvDgrad)))
    rows = [n for n in nodes if isinstance(n.op, core.FusedRows)]
    assert len(rows) == 1 and 8 in rows[0].op.in_kinds
    assert count(nodes, core.GetFlatIndices) == 0 and count(nodes, core.IncFlatIndices) == 0
    # the switches
    off = rewritten(fuse_conv_direct=False)
    assert count(off, im2col_ops.Im2Col) == 1 and count(off, im2col_ops.ConvDirectFwd) == 0 and count(off, im2col_ops.ReluGradNHWC) == 3
    off = rewritten(hoist_filter_splits=False)
    assert count(off, im2col_ops.SplitFilterBanks) == 0 and not any(n.op.pre for n in off if isinstance(n.op, im2col_ops.ConvDgrad))
    off = rewritten(fuse_flat_index_rows=False)
    assert count(off, core.GetFlatIndices) == 1 and count(off, core.IncFlatIndices) == 1


def test_flat_index_rows_rewrite():
    """logprobs[arange(batch), y] and its gradient on the MLP configuration (no GPU needed: only the rewritten graph is
    inspected, and the new Ops' host implementations are evaluated with numpy): GetFlatIndices / IncFlatIndices / the
    zero fill / the index addition disappear, and one FusedRows node reads the labels themselves (input kind 8) and
    holds the selection as entry (4, 0, a, b)."""
    cfg = configs.build_mlp(batch=16)
    outs, _usrc, utargs, analysis = compilation.simplify_for_execution([cfg.loss] + list(cfg.extra_outputs), cfg.updates)
    n2s = analysis["node2shape"]
    before = [n for n in core.topsorted(outs + utargs) if not n.is_input()]
    assert any(isinstance(n.op, core.GetFlatIndices) for n in before) and any(isinstance(n.op, core.IncFlatIndices) for n in before)
    o, u = compilation.apply_graph_rewrites(outs, utargs, n2s)
    nodes = [n for n in core.topsorted(o + u) if not n.is_input()]
    assert not any(isinstance(n.op, (core.GetFlatIndices, core.IncFlatIndices, core.OneHotRows, core.MaskedRowSum)) for n in nodes)
    rows = [n for n in nodes if isinstance(n.op, core.FusedRows)]
    assert len(rows) == 1 and 8 in rows[0].op.in_kinds and any(p[0] == 4 for p in rows[0].op.program)
    assert rows[0].parents[rows[0].op.in_kinds.index(8)].dtype == "i8"
    # with the switch off the flat-index Ops stay
    with cgt.scoped_update_config(fuse_flat_index_rows=False):
        outs2, _s, utargs2, analysis2 = compilation.simplify_for_execution([cfg.loss] + list(cfg.extra_outputs), cfg.updates)
        o2, u2 = compilation.apply_graph_rewrites(outs2, utargs2, analysis2["node2shape"])
    assert any(isinstance(n.op, core.GetFlatIndices) for n in core.topsorted(o2 + u2) if not n.is_input())
    # host implementations of the two Ops
    rs = np.random.RandomState(0)
    x, idx = rs.randn(5, 7).astype("f4"), np.array([6, 0, 3, 3, 1], "i8")
    x[2, 0] = -np.inf
    hot = np.empty((5, 7), "f4")
    core.OneHotRows(7).get_py_func(None)([idx], hot)
    assert np.array_equal(hot, (np.arange(7)[None, :] == idx[:, None]).astype("f4"))
    pick = np.empty((5, 1), "f4")
    core.MaskedRowSum().get_py_func(None)([x, hot], pick)
    assert np.array_equal(pick[:, 0], x[np.arange(5), idx])


def test_recurrent_graph_rewrites():
    """The rewrites aimed at unrolled recurrent networks, on the LSTM configuration with six time steps (no GPU needed:
    only the rewritten graph is inspected). x[t] becomes a view, the gate slices are read in place by the fused chains (no
    GetSli is left), the gradients of the slices are placed by ScatterCols (no IncSli / Fill is left), the softmax
    chains are FusedRows, and the per-time-step weight and bias gradient terms are one product / one reduction over
    row-concatenated operands per parameter."""
    T = 6
    cfg = configs.build_lstm(seq_len=T, batch=8)
    outs, _usrc, utargs, analysis = compilation.simplify_for_execution([cfg.loss] + list(cfg.extra_outputs), cfg.updates)
    n2s = analysis["node2shape"]
    before = [n for n in core.topsorted(outs + utargs) if not n.is_input()]
    o, u = compilation.apply_graph_rewrites(outs, utargs, n2s)
    nodes = [n for n in core.topsorted(o + u) if not n.is_input()]     # topsorted raises on a cycle
    count = lambda pred: sum(1 for n in nodes if pred(n))
    assert count(lambda n: isinstance(n.op, core.GetSli)) == 0
    assert count(lambda n: isinstance(n.op, core.IncSli)) == 0
    # x[t] and targ[t], and the per-time-step views of the five batched shared-weight products
    assert count(lambda n: isinstance(n.op, core.LeadingSlice)) == 2 * T + 5 * T
    # the hidden-to-hidden products stay (each needs the step before it); input-to-hidden of both layers and the output
    # projection are one product each, so are the two data-gradient products that do not feed a recurrence
    assert count(lambda n: isinstance(n.op, core.Mul22) and not n.op.tA and not n.op.tB) == 3
    # each hidden-to-hidden product carries the sum of the two pre-activations in its output stage
    assert count(lambda n: isinstance(n.op, core.Mul22BiasAdd)) == 2 * T
    assert count(lambda n: isinstance(n.op, core.Mul22) and not n.op.tA and n.op.tB) == 2 * (T - 1) + 2   # h at t = 0 is a constant
    # one placement of the four gates' gradients per layer and time step (two, per slab shape, without split_gate_columns)
    assert count(lambda n: isinstance(n.op, core.ScatterCols)) == 2 * T
    assert all(len(n.parents) == 4 for n in nodes if isinstance(n.op, core.ScatterCols))
    with cgt.scoped_update_config(split_gate_columns=False):
        sim = compilation.simplify_for_execution([cfg.loss] + list(cfg.extra_outputs), cfg.updates)
        o1, u1 = compilation.apply_graph_rewrites(sim[0], sim[2], sim[3]["node2shape"])
        nodes1 = [n for n in core.topsorted(o1 + u1) if not n.is_input()]
        assert sum(1 for n in nodes1 if isinstance(n.op, core.ScatterCols)) == 2 * 2 * T
        # per gate, every node of a cell has one shape: one chain holds the cell's forward arithmetic, and fewer launches remain
        launches = lambda ns: sum(1 for n in ns if isinstance(n.op, (core.FusedElwise, core.ScatterCols, core.ElwiseBinary, core.ElwiseUnary))
                                  and n.ndim > 0)
        assert launches(nodes) < 0.7 * launches(nodes1)
    assert count(lambda n: isinstance(n.op, core.FusedRows)) == T
    # the loss is accumulated term by term, one full reduction per time step: batch_scalar_sums leaves one reduction over
    # the row-concatenated terms (T >= 4 terms of one shape)
    full = lambda ns, rows: sum(1 for n in ns if isinstance(n.op, core.Sum) and sorted(n.op.axes) == [0, 1]
                                and compilation._static_shape(n2s.get(n.parents[0], [])) == (rows, 65))
    assert sum(1 for n in before if isinstance(n.op, core.Sum) and sorted(n.op.axes) == [0, 1]
               and compilation._static_shape(n2s[n.parents[0]]) == (8, 65)) == T
    assert full(nodes, 8) == 0 and full(nodes, 8 * T) == 1
    wgrads = [n for n in nodes if isinstance(n.op, core.Mul22) and n.op.tA and not n.op.tB]
    assert len(wgrads) == 5 and all(isinstance(p.op, core.Concatenate) and len(p.parents) == T for n in wgrads for p in n.parents)
    assert sum(1 for n in before if isinstance(n.op, core.Mul22) and n.op.tA and not n.op.tB) == 5 * T
    views = [n for n in nodes if isinstance(n.op, core.FusedElwise) and n.op.views]
    assert views and all(n.op.static_shape is not None and 7 in n.op.in_kinds for n in views)
    assert len(nodes) < 0.6 * len(before)
    # every rewrite has its switch: with all of them off the graph is the simplified one
    off = dict(fuse_slice_views=False, fuse_slice_sums=False, split_gate_columns=False, batch_summed_products=False, fuse_rows=False, fuse_elementwise=False,
               fuse_conv_dgrad=False, fuse_conv_grad_input=False)
    with cgt.scoped_update_config(**off):
        o2, u2 = compilation.apply_graph_rewrites(*compilation.simplify_for_execution([cfg.loss] + list(cfg.extra_outputs), cfg.updates)[0:3:2], n2s)
        assert not any(isinstance(n.op, (core.ScatterCols, core.LeadingSlice, core.FusedRows, core.FusedElwise))
                       for n in core.topsorted(o2 + u2) if not n.is_input())


@pytest.mark.parametrize("name,kw", [("cifar", dict(batch=4)), ("mlp", dict(batch=8)), ("lstm", dict(seq_len=3, batch=2))])
def test_edge_copies_are_scheduled_at_the_edges(name, kw):
    """compilation._transport_schedule: the uploads of the function arguments come before every device Op, and a
    copy-back whose descendants are all host-side (the loss) comes after every update, so the device work between
    them is one span. A copy-back that an update depends on (the LSTM's gradient norm) stays where it is."""
    cfg = configs.BUILDERS[name](**kw)
    outs, srcs, targs, analysis = compilation.simplify_for_execution([cfg.loss] + list(cfg.extra_outputs), cfg.updates)
    all_out = outs + targs
    nodelist = core.topsorted(all_out)
    node2dev = compilation.determine_devices(nodelist, dict(zip(targs, srcs)))
    compilation.add_transports(nodelist, node2dev, analysis["node2shape"])
    first, last = compilation._transport_schedule(all_out, targs, node2dev)
    assert first and all(t.parents[0].is_argument() for t in first)
    assert last and all(node2dev[t].devtype == "cpu" for t in last)
    extra = compilation._update_control_deps(all_out, list(zip(srcs, targs)))
    for node in last:
        extra[node] = extra.get(node, []) + [t for t in targs if t is not node]
    order = compilation.topsorted_shapes_first(first + all_out, analysis["node2shape"], extra)
    assert len(order) == len(set(order)) and set(nodelist) <= set(order)
    pos = {n: i for (i, n) in enumerate(order)}
    for node in order:                                   # still a topological order
        assert all(pos[p] < pos[node] for p in node.parents)
    device_ops = [n for n in order if not n.is_input() and n in node2dev and node2dev[n].devtype == "gpu" and not isinstance(n.op, core.Transport)
                  and n.op.return_type == "byref"]
    assert max(pos[t] for t in first) < min(pos[n] for n in device_ops)
    assert min(pos[t] for t in last) > max(pos[t] for t in targs)
    if name == "lstm":   # the clipping factor is computed on the host from a copied-back norm and feeds the updates
        mid = [n for n in order if not n.is_input() and isinstance(n.op, core.Transport) and n in node2dev and node2dev[n].devtype == "cpu"
               and n not in last]
        assert mid and all(pos[n] < max(pos[t] for t in targs) for n in mid)


def test_update_is_ordered_after_other_readers_of_the_variable():
    """Updates listed last-layer-first: the dgrad product that still needs the old last-layer weight
    must be scheduled before the in-place update of that weight."""
    x = cgt.matrix("x", fixed_shape=(5, 4))
    w1 = nn.parameter(np.random.RandomState(0).randn(4, 3).astype("f4"), name="w1")
    w2 = nn.parameter(np.random.RandomState(1).randn(3, 2).astype("f4"), name="w2")
    loss = cgt.tanh(cgt.tanh(x.dot(w1)).dot(w2)).sum()
    g1, g2 = cgt.grad(loss, [w1, w2])
    updates = [(w2, w2 - 0.1 * g2), (w1, w1 - 0.1 * g1)]  # reversed on purpose
    cfg = configs.Config("t", [x], loss, [w1, w2], updates, None, 5)
    pl = _plan(cfg)
    order = pl["order"]
    pos = {n: i for (i, n) in enumerate(order)}
    w2_node = pl["srcs"][0]
    w2_update = pl["targs"][0]
    readers = [n for n in order if w2_node in n.parents and n is not w2_update]
    assert readers and all(pos[r] < pos[w2_update] for r in readers)
    # and the oracle (which applies updates after evaluating everything) agrees with plain numpy
    f = cpu_backend.function([x], loss, updates=updates)
    xv = np.random.RandomState(2).randn(5, 4).astype("f4")
    f(xv)
    h = np.tanh(xv @ w1.op.get_value())
    o = np.tanh(h @ w2.op.get_value())
    go = 1 - o * o
    gh = (go @ w2.op.get_value().T) * (1 - h * h)
    np.testing.assert_allclose(f.get_value(w1), w1.op.get_value() - 0.1 * (xv.T @ gh), rtol=1e-5, atol=1e-6)


def test_all_configs_build_and_run_on_the_oracle():
    small = {"mlp": dict(batch=8), "cifar": dict(batch=2), "wide": dict(batch=2), "lstm": dict(seq_len=3, batch=4),
             "vae": dict(batch=5)}
    for (name, kw) in small.items():
        cfg = configs.BUILDERS[name](**kw)
        f = cpu_backend.function(cfg.inputs, [cfg.loss] + cfg.extra_outputs, updates=cfg.updates)
        b = cfg.batch(0)
        l0 = float(f(*b)[0])
        l1 = float(f(*b)[0])
        assert np.isfinite(l0) and np.isfinite(l1) and l0 != l1, name


# ------------------------------------------------------------------------------------------------
# Ops that carry C++ source (reference: NativeCompileInfo with $function / $closure templating)
# ------------------------------------------------------------------------------------------------
class ScaleBy(core.Op):
    """User-defined Op in the style of the reference's tests (cgt/tests/test_multi_output.py:32-58)."""
    available_impls = ("native_cpu",)

    def __init__(self, factor):
        self.factor = factor

    def typ_apply(self, input_types):
        return input_types[0]

    def shp_apply(self, inputs):
        return cgt.shape(inputs[0])

    def get_native_compile_info(self, input_types, devtype):
        code = r"""
            CGT_EXPORT_C void $function($closure* cl, cgtArray** reads, cgtArray* write) {
                for (long i = 0; i < reads[0]->size(); ++i) write->at<float>(i) = cl->factor * reads[0]->at<float>(i);
            }"""
        return core.NativeCompileInfo(code, closure_triples=[("factor", ctypes.c_float, self.factor)])


def test_op_with_cpp_source_is_compiled_and_callable():
    op = ScaleBy(2.5)
    callable_ = compilation.get_native_callable(op, [core.TensorType("f4", 1)], "cpu")
    x = np.arange(5, dtype="f4")
    out = np.zeros(5, "f4")
    callable_.call([x], out)
    assert np.array_equal(out, 2.5 * x)
    # the library is cached under its hash
    again = compilation.get_native_callable(ScaleBy(2.5), [core.TensorType("f4", 1)], "cpu")
    assert ctypes.cast(again.fptr, ctypes.c_void_p).value == ctypes.cast(callable_.fptr, ctypes.c_void_p).value


# ------------------------------------------------------------------------------------------------
# configuration
# ------------------------------------------------------------------------------------------------
def test_config_flags_and_scopes(monkeypatch):
    assert cgt.get_config()["backend"] == "native"
    with cgt.scoped_update_config(precision="double", verbose=True):
        assert cgt.floatX == "f8" and cgt.get_config()["verbose"] is True
        assert cgt.matrix().dtype == "f8"
    assert cgt.floatX == "f4" and cgt.get_config()["verbose"] is False
    with pytest.raises(ValueError):
        cgt.update_config(no_such_option=1)
    monkeypatch.setenv("CGT_FLAGS", "use_cuda_graphs=False,num_threads=3")
    try:
        cfg = core.get_config(True)
        assert cfg["use_cuda_graphs"] is False and cfg["num_threads"] == 3
    finally:
        monkeypatch.delenv("CGT_FLAGS")
        core.get_config(True)


def test_checkpoint_file_round_trip(tmp_path):
    """save_state / load_state (the file format over InMemoryData.get_value / set_value, cgt/core.py:569-582) and the
    flat-vector helper (examples/param_collection.py:37-56), on host-resident values: no GPU needed."""
    from cgt_b200 import checkpoint, configs
    cfg = configs.build_vae(batch=4)
    variables = cfg.state_variables()
    # parameters, two Adam slots per parameter and the step counter
    assert len(variables) == 3 * len(cfg.params) + 1
    assert variables[:len(cfg.params)] == list(cfg.params)
    rs = np.random.RandomState(0)
    saved = []
    for v in variables:
        val = rs.randn(*v.op.get_shape()).astype(v.dtype)
        v.op.set_value(val)
        saved.append(val)
    path = str(tmp_path / "state.npz")
    checkpoint.save_state(path, variables, extra={"step": 7, "seed": 3})
    for v in variables:
        v.op.set_value(np.zeros(v.op.get_shape(), v.dtype))
    extra = checkpoint.load_state(path, variables)
    assert extra == {"step": 7, "seed": 3}
    for (v, want) in zip(variables, saved):
        assert np.array_equal(v.op.get_value(), want)
    # a checkpoint of another model is refused before anything is written
    other = configs.build_mlp(batch=4)
    before = [p.op.get_value() for p in other.params]
    with pytest.raises(ValueError):
        checkpoint.load_state(path, other.state_variables())
    for (p, b) in zip(other.params, before):
        assert np.array_equal(p.op.get_value(), b)
    pc = checkpoint.ParamCollection(other.params)
    theta = pc.get_value_flat()
    assert theta.shape == (pc.get_total_size(),) and pc.num_vars() == len(other.params)
    pc.set_value_flat(theta * 2)
    for (p, b) in zip(other.params, before):
        assert np.array_equal(p.op.get_value(), b * 2)
