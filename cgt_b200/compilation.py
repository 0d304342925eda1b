"""Compiler from expression graphs to execution graphs, and the native-callable cache.

Counterpart of the reference's ``cgt/compilation.py``: ``function`` (:8), the pipeline
``run_compilation_pipeline`` (:312-367: simplify -> device placement -> transports -> shapes-first
topological order -> memory owners -> execution graph -> interpreter) and ``nci2callable`` (:529-551,
hash-keyed shared-library cache for Ops that carry C++/CUDA source).

What is specific to this backend:
  * placement follows the reference rule (scalars, arguments and shape arithmetic on the host,
    everything with a native_gpu implementation on the GPU) but honours ``Op.host_inputs`` /
    ``Op.meta_inputs`` so that launch-time operands are not shipped to the device and shape queries do
    not ship tensors to the host;
  * an update's right-hand side is ordered after every other reader of the variable it overwrites;
  * instructions whose inputs are all compile-time constants are marked to fire once;
  * the interpreter is the stream-issuing native one in ``libcgt_b200.so``; there is no Python or
    CPU interpreter in this package.
"""
import ctypes
import os
import os.path as osp
import pickle
import string
import subprocess
import sys
from collections import defaultdict
from io import StringIO

import numpy as np

from . import core, utils

cgt = core  # filled by attribute access through core.cgt at call time


def _cgt():
    return core.cgt


def function(inputs, outputs, dbg=None, updates=None, givens=None):
    """Compile `outputs` (a Node or list of Nodes) as a function of the Argument nodes `inputs`.
    `updates` is a list of (shared variable, new value) pairs applied in place on every call."""
    assert isinstance(inputs, list), "Inputs must be a list"
    assert all(el.is_argument() for el in inputs), "Invalid input: should be a list of Argument nodes"
    if isinstance(outputs, list):
        assert all(isinstance(el, core.Node) for el in outputs), "Invalid output: should all be symbolic variables"
        return _function_listout(inputs, outputs, dbg, updates, givens)
    elif isinstance(outputs, core.Node):
        f_listout = _function_listout(inputs, [outputs], dbg, updates, givens)
        return _SingleOut(f_listout)
    raise ValueError("Expected `outputs` to be a Node or a list of Nodes. Got an object of type %s" % type(outputs))


class _SingleOut(object):
    def __init__(self, f):
        self.f = f

    def __call__(self, *args):
        return self.f(*args)[0]

    def __getattr__(self, name):
        return getattr(self.f, name)


def _check_updates(updates):
    if isinstance(updates, dict):
        updates = list(updates.items())
    if updates is None:
        updates = []
    assert isinstance(updates, list) and all(
        isinstance(a, tuple) and len(a) == 2 and isinstance(a[0], core.Node) and isinstance(a[1], core.Node)
        for a in updates), "updates should be a list of pairs (before, after)"
    assert all(before.is_data() for (before, _) in updates), "lhs of updates must be Data instances"
    return updates


def _function_listout(inputs, outputs, dbg=None, updates=None, givens=None):
    updates = _check_updates(updates)
    if dbg:
        raise core.Todo("debug functionality is broken")
    outputs = [_cgt().make_tuple(*x) if isinstance(x, tuple) else x for x in outputs]
    return run_compilation_pipeline(inputs, outputs, updates, givens or [])


# ================================================================
# Phase 1: simplification (shared with the test oracle's evaluator)
# ================================================================

def simplify_for_execution(outputs, updates, givens=()):
    """Returns (outputs_simple, update_sources, update_targets_simple, analysis)."""
    config = core.get_config()
    outputs_updatetargs = list(outputs) + [after for (_before, after) in updates]
    if givens:
        outputs_updatetargs = core.clone(outputs_updatetargs, dict(givens))
    if config["enable_simplification"]:
        simple, _analysis, _ = core.simplify_and_analyze(outputs_updatetargs)
    else:
        simple = outputs_updatetargs
    # fresh copy of the graph: later passes rewrite parent lists in place
    simple = core.clone(simple)
    analysis = core.init_analysis()
    repl = {}
    main_nodes = core.topsorted(simple)
    for node in main_nodes:
        core.do_analysis(node, analysis)
        repl[node] = node
    if config["enable_simplification"]:
        # Shape expressions are simplified against the same analysis, so that with fixed input shapes
        # every extent folds to a constant instead of being recomputed by host instructions on each run.
        def simp(s):
            core.update_simplify_map(s, analysis, repl)
            return repl[s]
        node2shape = analysis["node2shape"]
        for node in main_nodes:
            shp = node2shape[node]
            if isinstance(shp, tuple):
                node2shape[node] = tuple([simp(s) for s in arrshp] for arrshp in shp)
            else:
                node2shape[node] = [simp(s) for s in shp]
    n = len(outputs)
    return simple[:n], [before for (before, _) in updates], simple[n:], analysis


# ================================================================
# Phase 1b: elementwise fusion
# ================================================================

_FUSABLE_WITH_INT_SCALAR = ("*", "+", "-", "/", "<", ">", "<=", ">=", "==", "!=")


def _small_int_constant(node):
    if not isinstance(node.op, core.Constant):
        return False
    v = np.asarray(node.op.value)
    return v.size == 1 and abs(int(v.reshape(-1)[0])) < (1 << 24)


def _fusable(node):
    """An elementwise node whose arithmetic the fused kernel reproduces bit for bit: float32 (or 0/1
    truth value) operands and results, built-in operations."""
    if node.is_input() or node.ndim == 0:
        return False
    op = node.op
    if isinstance(op, core.ElwiseUnary):
        return node.dtype == "f4" and node.parents[0].dtype == "f4" and op.opname in core.UNARY_OPCODE
    if isinstance(op, core.ElwiseBinary):
        if node.dtype not in ("f4", "i1") or op.opname not in core.BINARY_OPCODE:
            return False
        kinds = []
        for par in node.parents:
            if par.dtype in ("f4", "i1"):
                kinds.append(par.dtype)
            elif par.ndim == 0 and par.dtype == "i8" and _small_int_constant(par) and op.opname in _FUSABLE_WITH_INT_SCALAR:
                kinds.append("i8")
            else:
                return False
        if "f4" not in kinds:
            return False
        if op.opname == "**" and kinds != ["f4", "f4"]:
            return False
        return True
    return False


def _foldable_repeat(node):
    """Repeat of a float32 tensor along a prefix and a suffix of its axes (a bias [1,C,1,1] -> [B,C,H,W],
    a row [1,N] -> [B,N], a column [B,1] -> [B,N]): the fused kernel reads the small operand directly."""
    if node.is_input() or not isinstance(node.op, core.Repeat) or node.dtype != "f4":
        return False
    nd = node.ndim
    axes = sorted(node.op.axes)
    kept = [d for d in range(nd) if d not in axes]
    return all(b - a == 1 for (a, b) in zip(kept[:-1], kept[1:]))


def view_leading_slices(outputs, updatetargs, node2shape):
    """GetSli along axis 0 with step 1 and constant bounds -> LeadingSlice: the rows of a C-contiguous array are contiguous,
    so the slice is a view at an offset instead of a copy kernel. Only where the source cannot change under the view:
    it is an argument's device copy or any other node that no instruction writes into (no update target, no IncSli /
    IncFlatIndices base)."""
    all_out = list(outputs) + list(updatetargs)
    nodes = core.topsorted(all_out)
    written = set()
    for node in nodes:
        if not node.is_input() and node.op.writes_to_input >= 0:
            written.add(node.parents[node.op.writes_to_input])
    replace = {}
    for node in nodes:
        if node.is_input() or not isinstance(node.op, core.GetSli) or node.op.axis != 0 or node in all_out:
            continue
        (x, start, stop, step) = node.parents
        if not all(isinstance(q.op, core.Constant) for q in (start, stop, step) if not q.is_input()) or any(q.is_input() for q in (start, stop, step)):
            continue
        xshp = _static_shape(node2shape[x])
        (a, b, st) = (int(start.op.value), int(stop.op.value), int(step.op.value))
        if st != 1 or xshp is None or not (0 <= a <= b <= xshp[0]) or x in written or x in updatetargs:
            continue
        if not x.is_input() and isinstance(x.op, core.InMemoryData):
            continue   # a shared variable can be updated in place while the view is alive
        new = core.Result(core.LeadingSlice(), [x, start, stop])
        node2shape[new] = node2shape[node]
        new.props.update(node.props)
        replace[node] = new
    if not replace:
        return list(outputs), list(updatetargs)
    return _rewire(outputs, updatetargs, replace)


def batch_summed_products(outputs, updatetargs, node2shape):
    """Sums over many terms of one form, as an unrolled recurrent network's parameter gradients arrive (one term per time
    step, added one after the other): sum_t Mul22{T,N}(a_t, b_t) with equal shapes is ONE product of the operands
    concatenated along the contracted axis, Mul22{T,N}(concat_t a_t, concat_t b_t); sum_t Sum{0}(g_t) is
    Sum{0}(concat_t g_t). Fifty products and forty-nine additions of [in, out] matrices become two row concatenations
    (one launch each, shared between the sums that use the same operands) and one product with a fifty times longer
    contraction. The order of the float32 additions changes: float32 tolerance against the term-by-term graph."""
    MIN_TERMS, MAX_PIECES = 4, 64
    all_out = list(outputs) + list(updatetargs)
    nodes = core.topsorted(all_out)
    children = defaultdict(list)
    for node in nodes:
        for par in node.parents:
            children[par].append(node)
    out_set = set(all_out)

    def is_add(node):
        return (not node.is_input() and isinstance(node.op, core.ElwiseBinary) and node.op.opname == "+" and node.ndim == 2
                and node.dtype == "f4" and all(par.ndim == 2 for par in node.parents))

    def leaves_of(node, acc):
        for par in node.parents:
            if is_add(par) and len(children[par]) == 1 and par not in out_set:
                leaves_of(par, acc)
            else:
                acc.append(par)

    def form(leaf):
        if leaf.is_input() or len(children[leaf]) != 1 or leaf in out_set or leaf.dtype != "f4":
            return None
        if isinstance(leaf.op, core.Mul22) and leaf.op.tA and not leaf.op.tB:
            sa, sb = _static_shape(node2shape[leaf.parents[0]]), _static_shape(node2shape[leaf.parents[1]])
            if sa is not None and sb is not None and all(p.dtype == "f4" for p in leaf.parents):
                return ("mul22", sa, sb)
        if isinstance(leaf.op, core.Sum) and tuple(leaf.op.axes) == (0,):
            sx = _static_shape(node2shape[leaf.parents[0]])
            if sx is not None and len(sx) == 2 and leaf.parents[0].dtype == "f4":
                return ("sum0", sx)
        return None

    concat_cache = {}

    def concat_rows(parts):
        key = tuple(id(q) for q in parts)
        if key not in concat_cache:
            shp = _static_shape(node2shape[parts[0]])
            new = core.Result(core.Concatenate(0), list(parts))
            node2shape[new] = [core.cgt.constant(np.array(shp[0] * len(parts), "i8")), core.cgt.constant(np.array(shp[1], "i8"))]
            concat_cache[key] = new
        return concat_cache[key]

    replace = {}
    covered = set()
    for node in reversed(nodes):   # the root of an addition tree comes before its inner nodes
        if node in covered or not is_add(node):
            continue
        leaves = []
        leaves_of(node, leaves)
        stack = [node]
        while stack:
            q = stack.pop()
            covered.add(q)
            stack.extend(par for par in q.parents if is_add(par) and len(children[par]) == 1 and par not in out_set)
        groups = defaultdict(list)
        for leaf in leaves:
            f = form(leaf)
            if f is not None:
                groups[f].append(leaf)
        terms, batched = [], set()
        for (f, members) in groups.items():
            if len(members) < MIN_TERMS:
                continue
            for lo in range(0, len(members), MAX_PIECES):
                chunk = members[lo:lo + MAX_PIECES]
                if len(chunk) < 2:
                    continue
                if f[0] == "mul22":
                    new = core.Result(core.Mul22(True, False), [concat_rows([m.parents[0] for m in chunk]), concat_rows([m.parents[1] for m in chunk])])
                else:
                    new = core.Result(core.Sum((0,)), [concat_rows([m.parents[0] for m in chunk])])
                node2shape[new] = node2shape[chunk[0]]
                terms.append(new)
                batched.update(chunk)
        if not batched:
            continue
        terms += [leaf for leaf in leaves if leaf not in batched]
        total = terms[0]
        for t in terms[1:]:
            total = core.Result(core.ElwiseBinary("+", (False, False)), [total, t])
            node2shape[total] = node2shape[node]
        total.props.update(node.props)
        replace[node] = total
    if not replace:
        return list(outputs), list(updatetargs)
    return _rewire(outputs, updatetargs, replace)


def batch_scalar_sums(outputs, updatetargs, node2shape):
    """A scalar accumulated term by term, loss = ((0 - X_0.sum()) - X_1.sum()) - ... with one [R, C] matrix per time step:
    every term is a full reduction on the GPU, a copy of one float to the host and a host subtraction. Terms of one
    sign and one matrix shape (at least four) become ONE reduction over the row-concatenated matrices,
    +/- Sum{0,1}(concat_t X_t): one concatenation, one reduction, one copy. The order of the float32 additions changes:
    float32 tolerance against the term-by-term graph (the value is the reported loss; no gradient flows through it,
    this runs after differentiation)."""
    MIN_TERMS, MAX_PIECES = 4, 64
    all_out = list(outputs) + list(updatetargs)
    nodes = core.topsorted(all_out)
    children = defaultdict(list)
    for node in nodes:
        for par in node.parents:
            children[par].append(node)
    out_set = set(all_out)

    def is_acc(node):
        return (not node.is_input() and isinstance(node.op, core.ElwiseBinary) and node.op.opname in ("+", "-") and node.ndim == 0
                and node.dtype == "f4"
                and all(par.ndim == 0 and (par.dtype == "f4" or isinstance(getattr(par, "op", None), core.Constant)) for par in node.parents))

    def terms_of(node, sign, acc):
        for (pos, par) in enumerate(node.parents):
            sg = -sign if (node.op.opname == "-" and pos == 1) else sign
            while (not par.is_input() and isinstance(par.op, core.ElwiseUnary) and par.op.opname == "neg" and par.ndim == 0
                   and len(children[par]) == 1 and par not in out_set):
                (sg, par) = (-sg, par.parents[0])     # 0 - x arrives as neg(x)
            if is_acc(par) and len(children[par]) == 1 and par not in out_set:
                terms_of(par, sg, acc)
            else:
                acc.append((sg, par))

    def full_sum(term):
        """X when term = X.sum() of a static float32 matrix read by nothing else"""
        q = term
        while not q.is_input() and isinstance(q.op, core.Reshape) and len(children[q]) == 1 and q not in out_set:
            q = q.parents[0]
        if q.is_input() or not isinstance(q.op, core.Sum) or len(children[q]) != 1 or q in out_set:
            return None
        x = q.parents[0]
        shp = _static_shape(node2shape[x]) if x in node2shape else None
        if shp is None or len(shp) != 2 or x.dtype != "f4" or sorted(q.op.axes) != [0, 1]:
            return None
        return x

    const = lambda v: core.cgt.constant(np.array(v, "i8"))
    replace, covered = {}, set()
    for node in reversed(nodes):
        if node in covered or not is_acc(node):
            continue
        terms = []
        terms_of(node, 1, terms)
        stack = [node]
        while stack:
            q = stack.pop()
            covered.add(q)
            stack.extend(par for par in q.parents if is_acc(par) and len(children[par]) == 1 and par not in out_set)
        groups = defaultdict(list)
        for (k, (sg, t)) in enumerate(terms):
            x = full_sum(t)
            if x is not None:
                groups[(sg, _static_shape(node2shape[x]))].append((k, x))
        batched, new_terms = set(), []
        for ((sg, shp), members) in groups.items():
            if len(members) < MIN_TERMS:
                continue
            for lo in range(0, len(members), MAX_PIECES):
                chunk = members[lo:lo + MAX_PIECES]
                if len(chunk) < 2:
                    continue
                cat = core.Result(core.Concatenate(0), [x for (_k, x) in chunk])
                node2shape[cat] = [const(shp[0] * len(chunk)), const(shp[1])]
                tot = core.Result(core.Sum((0, 1)), [cat])
                node2shape[tot] = [const(1), const(1)]
                sc = core.Result(core.Reshape(), [tot])
                node2shape[sc] = []
                new_terms.append((sg, sc))
                batched.update(k for (k, _x) in chunk)
        if not batched:
            continue
        rest = [(sg, t) for (k, (sg, t)) in enumerate(terms) if k not in batched] + new_terms
        rest.sort(key=lambda st: -st[0])      # a positive term first, if there is one
        (sg0, total) = rest[0]
        if sg0 < 0:
            total = core.Result(core.ElwiseUnary("neg"), [total])
            node2shape[total] = []
        for (sg, t) in rest[1:]:
            total = core.Result(core.ElwiseBinary("+" if sg > 0 else "-", (True, True)), [total, t])
            node2shape[total] = []
        total.props.update(node.props)
        replace[node] = total
    if not replace:
        return list(outputs), list(updatetargs)
    return _rewire(outputs, updatetargs, replace)


def batch_shared_weight_products(outputs, updatetargs, node2shape):
    """Products that share their right operand and do not need each other: Mul22{N,N}(a_t, W) or Mul22{N,T}(a_t, W) for
    many t with a_t of one shape, none of which depends on another's result (the input-to-hidden products of an unrolled
    recurrent layer over all time steps, the output projection, the matching data-gradient products) become ONE product
    of the row-concatenated a_t with W; every original result is a LeadingSlice view of it. When the a_t are the
    consecutive leading slices of one array, that array itself (reshaped) is the concatenation. Same sums in the same
    order per output element as far as the kernels' tiling allows: float32 tolerance."""
    MIN_TERMS, MAX_PIECES = 4, 64
    all_out = list(outputs) + list(updatetargs)
    nodes = core.topsorted(all_out)
    out_set = set(all_out)
    topo = dict((n, i) for (i, n) in enumerate(nodes))
    groups = defaultdict(list)
    for node in nodes:
        if node.is_input() or not isinstance(node.op, core.Mul22) or node.op.tA or node in out_set or node.dtype != "f4":
            continue
        (a, w) = node.parents
        sa, sw = _static_shape(node2shape[a]), _static_shape(node2shape[w])
        if sa is None or sw is None or a.dtype != "f4" or w.dtype != "f4":
            continue
        groups[(id(w), node.op.tB, sa, sw)].append(node)

    def depends_on_any(start, targets, floor):
        """does `start` depend on a node of `targets`? (nodes before topological index `floor` cannot)"""
        seen, stack = set(), [start]
        while stack:
            q = stack.pop()
            if q in seen or topo[q] < floor:
                continue
            seen.add(q)
            if q in targets:
                return True
            stack.extend(q.parents)
        return False

    def as_whole_array(parts):
        """the array of which `parts` are, in order, the consecutive leading slices (through reshapes to [rows, cols]);
        None otherwise"""
        src, pos = None, 0
        for q in parts:
            while not q.is_input() and isinstance(q.op, core.Reshape):
                q = q.parents[0]
            if q.is_input() or not isinstance(q.op, core.LeadingSlice):
                return None
            (x, start, stop) = q.parents
            if src is None:
                src = x
            if x is not src or not isinstance(start.op, core.Constant) or not isinstance(stop.op, core.Constant):
                return None
            if int(start.op.value) != pos:
                return None
            pos = int(stop.op.value)
        shp = _static_shape(node2shape[src]) if src is not None else None
        return src if shp is not None and pos == shp[0] else None

    # row concatenations that the graph already holds (made for the summed products of the same operands)
    existing = {}
    for node in nodes:
        if not node.is_input() and isinstance(node.op, core.Concatenate) and node.op.axis == 0:
            existing[tuple(id(q) for q in node.parents)] = node
    replace = {}
    for (key, members) in groups.items():
        if len(members) < MIN_TERMS:
            continue
        memberset = set(members)
        floor = min(topo[m] for m in members)
        if any(depends_on_any(m.parents[0], memberset, floor) for m in members):
            continue
        (rows, cols) = key[2]
        for lo in range(0, len(members), MAX_PIECES):
            chunk = members[lo:lo + MAX_PIECES]
            if len(chunk) < 2:
                continue
            parts = [m.parents[0] for m in chunk]
            total = core.cgt.constant(np.array(rows * len(chunk), "i8"))
            ncol = core.cgt.constant(np.array(cols, "i8"))
            whole = as_whole_array(parts)
            if whole is not None:
                acat = core.Result(core.Reshape(), [whole, total, ncol])
            else:
                acat = existing.get(tuple(id(q) for q in parts)) or core.Result(core.Concatenate(0), parts)
            node2shape[acat] = [total, ncol]
            z = core.Result(core.Mul22(False, chunk[0].op.tB), [acat, chunk[0].parents[1]])
            zcols = _static_shape(node2shape[chunk[0]])[1]
            node2shape[z] = [total, core.cgt.constant(np.array(zcols, "i8"))]
            for (t, m) in enumerate(chunk):
                view = core.Result(core.LeadingSlice(), [z, core.cgt.constant(np.array(t * rows, "i8")),
                                                         core.cgt.constant(np.array((t + 1) * rows, "i8"))])
                node2shape[view] = node2shape[m]
                view.props.update(m.props)
                replace[m] = view
    if not replace:
        return list(outputs), list(updatetargs)
    return _rewire(outputs, updatetargs, replace)


def fuse_slice_sums(outputs, updatetargs, node2shape):
    """Sums of IncSli(zeros, start, stop, 1, y) over disjoint column ranges of one float32 matrix -> ScatterCols.

    That is the form in which the gradient of several column slices of one matrix reaches the compiler (every
    GetSli.pullback makes its own zero matrix and increments its slice; the contributions are then added): k zero
    fills, k slice increments and k - 1 additions on [R, C] matrices for what is a placement of k pieces. A single
    padded slice (no addition) is rewritten as well: it saves the fill. Returns the new (outputs, updatetargs)."""
    all_out = list(outputs) + list(updatetargs)
    nodes = core.topsorted(all_out)
    children = defaultdict(list)
    for node in nodes:
        for par in node.parents:
            children[par].append(node)
    out_set = set(all_out)

    def const_int(node):
        if node.is_input() or not isinstance(node.op, core.Constant):
            return None
        v = np.asarray(node.op.value)
        return int(v.reshape(-1)[0]) if v.size == 1 else None

    def pad_piece(node):
        """(offset, width, y, C) when node = IncSli{1}(Fill{0}, start, stop, 1, y) on a static float32 matrix"""
        if node.is_input() or not isinstance(node.op, core.IncSli) or node.op.axis != 1 or node.ndim != 2 or node.dtype != "f4":
            return None
        (z, start, stop, step, y) = node.parents
        if z.is_input() or not isinstance(z.op, core.Fill) or float(z.op.value) != 0.0 or len(children[z]) != 1 or z in out_set:
            return None
        shp, yshp = _static_shape(node2shape[node]), _static_shape(node2shape[y])
        (a, b, st) = (const_int(start), const_int(stop), const_int(step))
        if shp is None or yshp is None or a is None or b is None or st != 1 or y.dtype != "f4" or len(yshp) != 2:
            return None
        if not (0 <= a <= b <= shp[1]) or yshp != (shp[0], b - a):
            return None
        return (a, b - a, y, shp[1])

    def collect(node, pieces):
        """leaves of the addition tree below `node`; False when something else than padded slices is added"""
        piece = pad_piece(node)
        if piece is not None:
            pieces.append(piece)
            return True
        if node.is_input() or not isinstance(node.op, core.ElwiseBinary) or node.op.opname != "+" or node.ndim != 2:
            return False
        for par in node.parents:
            if par.ndim != 2 or len(children[par]) != 1 or par in out_set:
                return False
            if not collect(par, pieces):
                return False
        return True

    replace = {}
    covered = set()
    for node in reversed(nodes):   # consumers first: the root of an addition tree is met before its parts
        if node in covered or node.is_input():
            continue
        pieces = []
        if not collect(node, pieces) or not pieces or len(pieces) > 8:
            continue
        C = pieces[0][3]
        spans = sorted((o, o + w) for (o, w, _y, _c) in pieces)
        if any(c != C for (_o, _w, _y, c) in pieces) or any(a1 < b0 for ((_a0, b0), (a1, _b1)) in zip(spans[:-1], spans[1:])):
            continue
        new = core.Result(core.ScatterCols([o for (o, _w, _y, _c) in pieces], [w for (_o, w, _y, _c) in pieces], C),
                          [y for (_o, _w, y, _c) in pieces])
        node2shape[new] = node2shape[node]
        new.props.update(node.props)
        replace[node] = new
        stack = [node]
        while stack:   # the tree's inner nodes are gone with it
            q = stack.pop()
            covered.add(q)
            if not q.is_input() and isinstance(q.op, core.ElwiseBinary):
                stack.extend(q.parents)
    if not replace:
        return list(outputs), list(updatetargs)
    return _rewire(outputs, updatetargs, replace)


def fuse_product_sums(outputs, updatetargs, node2shape):
    """z = (X + Repeat(b)) + (Mul22(h, U) + Repeat(c)), the pre-activation of a layer fed by two inputs (an unrolled
    recurrent cell forms it once per layer and time step) -> Mul22BiasAdd(h, U, c, X, b): the three additions run in
    the output stage of the product, in the same association, so no bit changes; one launch instead of two. Only for
    products that Mul22 gives to its FMA-tile kernel (the output stage lives there), whose result and whose sum with its
    bias have no other reader."""
    all_out = list(outputs) + list(updatetargs)
    nodes = core.topsorted(all_out)
    children = defaultdict(list)
    for node in nodes:
        for par in node.parents:
            children[par].append(node)
    out_set = set(all_out)

    def is_add(n):
        return (not n.is_input() and isinstance(n.op, core.ElwiseBinary) and n.op.opname == "+" and n.op.scalar_mask == (False, False)
                and n.dtype == "f4" and n.ndim == 2)

    def row_repeat(n, N):
        """the [1, N] row when n = Repeat{0}(row)"""
        if n.is_input() or not isinstance(n.op, core.Repeat) or list(n.op.axes) != [0] or n.dtype != "f4":
            return None
        row = n.parents[0]
        shp = _static_shape(node2shape[row]) if row in node2shape else None
        return row if shp == (1, N) else None

    def affine(n, N, want_product):
        """(x, row) when n = x + Repeat{0}(row) is read once; with want_product x must be a Mul22 read once"""
        if not is_add(n) or n in out_set or len(children[n]) != 1:
            return None
        for (x, r) in ((n.parents[0], n.parents[1]), (n.parents[1], n.parents[0])):
            row = row_repeat(r, N)
            if row is None or x.dtype != "f4":
                continue
            if want_product and (x.is_input() or not isinstance(x.op, core.Mul22) or len(children[x]) != 1 or x in out_set):
                continue
            return (x, row)
        return None

    replace = {}
    for z in nodes:
        if not is_add(z) or z in out_set:
            continue
        shp = _static_shape(node2shape[z]) if z in node2shape else None
        if shp is None:
            continue
        (M, N) = shp
        for (p, q) in ((z.parents[0], z.parents[1]), (z.parents[1], z.parents[0])):
            prod = affine(p, N, True)
            side = affine(q, N, False)
            if prod is None or side is None or p is q:
                continue
            (m, c_row) = prod
            (x, b_row) = side
            if _static_shape(node2shape[x]) != (M, N):
                continue
            (tA, tB) = (m.op.tA, m.op.tB)
            ashp = _static_shape(node2shape[m.parents[0]])
            if ashp is None or any(par.dtype != "f4" for par in m.parents):
                continue
            K = ashp[0] if tA else ashp[1]
            if M * N <= 2048 or (not tA and tB) or M * N * K > (1 << 25):
                continue     # not a product of the FMA-tile kernel
            new = core.Result(core.Mul22BiasAdd(tA, tB), [m.parents[0], m.parents[1], c_row, x, b_row])
            node2shape[new] = node2shape[z]
            new.props.update(z.props)
            replace[z] = new
            break
    if not replace:
        return list(outputs), list(updatetargs)
    return _rewire(outputs, updatetargs, replace)


def split_gate_columns(outputs, updatetargs, node2shape):
    """Elementwise arithmetic on column blocks of one matrix, written per block.

    A recurrent cell computes its gates on slabs of a [R, 4H] matrix: sigmoid on columns [0, 3H), slices of the result
    per gate; the gradient arrives as ScatterCols of the gates' gradients, multiplied as a slab by the slab's
    derivative and placed again into [R, 4H]. The arithmetic is elementwise, so it can be done per gate on [R, H]
    blocks, which lets one fused chain hold a whole cell (all its nodes then have one shape) instead of one chain per
    slab shape. Three local rewrites, repeated until nothing changes; the values do not change by a bit:
      * f(ScatterCols(p_1..p_k), y) for an elementwise binary f whose first or second operand is a ScatterCols that
        covers all columns and has no other reader -> ScatterCols(f(p_1, y[:, cols_1]), ..., f(p_k, y[:, cols_k]));
      * a ScatterCols piece that is itself such a ScatterCols -> its pieces at shifted offsets (one placement);
      * x[:, a:b] of an elementwise unary node, or of a binary node with a scalar operand, all of whose readers are
        column slices -> the same operation on (operand)[:, a:b]; slices of slices are composed;
      * a Reshape to the shape its operand already has -> the operand.
    A slice of anything else stays a GetSli, which the fused chains read in place."""
    const = lambda v: core.cgt.constant(np.array(v, "i8"))

    def const_int(node):
        if not isinstance(getattr(node, "op", None), core.Constant):
            return None
        v = np.asarray(node.op.value)
        return int(v.reshape(-1)[0]) if v.size == 1 else None

    def shape2(node):
        shp = _static_shape(node2shape[node]) if node in node2shape else None
        return shp if shp is not None and len(shp) == 2 else None

    def ident(q):
        """q without reshapes that change nothing"""
        while not q.is_input() and isinstance(q.op, core.Reshape) and shape2(q) is not None and shape2(q) == shape2(q.parents[0]):
            q = q.parents[0]
        return q

    def col_slice(n):
        """(x, a, b) when n = x[:, a:b] with constant bounds on a static float32 matrix"""
        if n.is_input() or not isinstance(n.op, core.GetSli) or n.op.axis != 1 or n.dtype != "f4":
            return None
        (x, start, stop, step) = n.parents
        (a, b, st) = (const_int(start), const_int(stop), const_int(step))
        xs = shape2(x)
        if xs is None or a is None or b is None or st != 1 or not (0 <= a < b <= xs[1]) or shape2(n) != (xs[0], b - a):
            return None
        return (x, a, b)

    def full_cover(sc):
        spans = sorted((o, o + w) for (o, w) in zip(sc.op.offsets, sc.op.widths))
        return spans[0][0] == 0 and spans[-1][1] == sc.op.C and all(b0 == a1 for ((_a0, b0), (a1, _b1)) in zip(spans[:-1], spans[1:]))

    def pushable(e):
        """an elementwise node through which a column slice may be moved to its operand"""
        if e.is_input() or e.dtype != "f4" or shape2(e) is None or not _fusable(e):
            return False
        if isinstance(e.op, core.ElwiseUnary):
            return True
        return isinstance(e.op, core.ElwiseBinary) and sum(e.op.scalar_mask) == 1

    cache = {}

    def sliced(node, a, b):
        """a node with the value of node[:, a:b]"""
        node = ident(node)
        shp = shape2(node)
        if a == 0 and b == shp[1]:
            return node
        key = (node, a, b)
        if key in cache:
            return cache[key]
        cs = col_slice(node)
        if cs is not None:
            new = sliced(cs[0], cs[1] + a, cs[1] + b)
        elif pushable(node):
            pars = [par if par.ndim == 0 else sliced(par, a, b) for par in node.parents]
            new = core.Result(node.op, pars)
            node2shape[new] = [const(shp[0]), const(b - a)]
        elif not node.is_input() and isinstance(node.op, core.ScatterCols) and (a, b - a) in list(zip(node.op.offsets, node.op.widths)):
            new = ident(node.parents[list(zip(node.op.offsets, node.op.widths)).index((a, b - a))])
        else:
            new = core.Result(core.GetSli(1), [node, const(a), const(b), const(1)])
            node2shape[new] = [const(shp[0]), const(b - a)]
        cache[key] = new
        return new

    for _round in range(8):
        all_out = list(outputs) + list(updatetargs)
        nodes = core.topsorted(all_out)
        children = defaultdict(list)
        for node in nodes:
            for par in node.parents:
                children[par].append(node)
        out_set = set(all_out)

        def sole_reader(q, reader):
            """q (below identity reshapes of `reader`'s operand) is read by nothing else"""
            while True:
                if q in out_set or len(children[q]) != 1:
                    return False
                c = children[q][0]
                if c is reader:
                    return True
                if not (isinstance(c.op, core.Reshape) and shape2(c) is not None and shape2(c) == shape2(q)):
                    return False
                q = c

        replace = {}
        for node in nodes:
            if node.is_input() or node in out_set or node.dtype != "f4" or shape2(node) is None:
                continue
            op = node.op
            # a reshape that changes nothing stands between two elementwise nodes that one chain could hold
            if isinstance(op, core.Reshape):
                if ident(node) is not node:
                    replace[node] = ident(node)
                continue
            # elementwise binary on a placed matrix -> placed results of the per-piece operation
            if isinstance(op, core.ElwiseBinary) and op.scalar_mask == (False, False) and _fusable(node) and node.parents[0] is not node.parents[1]:
                done = False
                for pos in (0, 1):
                    sc = ident(node.parents[pos])
                    other = node.parents[1 - pos]
                    if sc.is_input() or not isinstance(sc.op, core.ScatterCols) or sc.dtype != "f4" or shape2(other) != shape2(node) \
                            or other.dtype != "f4" or not full_cover(sc) or not sole_reader(sc, node) or sc in replace:
                        continue
                    pieces = []
                    for (piece, o, w) in zip(sc.parents, sc.op.offsets, sc.op.widths):
                        ops = [ident(piece), sliced(other, o, o + w)]
                        if pos == 1:
                            ops.reverse()
                        q = core.Result(op, ops)
                        node2shape[q] = [const(shape2(node)[0]), const(w)]
                        pieces.append(q)
                    new = core.Result(core.ScatterCols(sc.op.offsets, sc.op.widths, sc.op.C), pieces)
                    node2shape[new] = node2shape[node]
                    new.props.update(node.props)
                    replace[node] = new
                    done = True
                    break
                if done:
                    continue
            # a placed piece that is itself a placement
            if isinstance(op, core.ScatterCols):
                offsets, widths, pieces, changed = [], [], [], False
                for (piece, o, w) in zip(node.parents, op.offsets, op.widths):
                    inner = ident(piece)
                    if not inner.is_input() and isinstance(inner.op, core.ScatterCols) and inner.op.C == w and inner not in replace \
                            and sole_reader(inner, node) and len(offsets) + len(inner.parents) <= 8:
                        for (q, io, iw) in zip(inner.parents, inner.op.offsets, inner.op.widths):
                            offsets.append(o + io)
                            widths.append(iw)
                            pieces.append(q)
                        changed = True
                    else:
                        offsets.append(o)
                        widths.append(w)
                        pieces.append(piece)
                if changed and len(pieces) <= 8:
                    new = core.Result(core.ScatterCols(offsets, widths, op.C), pieces)
                    node2shape[new] = node2shape[node]
                    new.props.update(node.props)
                    replace[node] = new
                continue
            # a column slice of an elementwise node that only column slices read
            cs = col_slice(node)
            if cs is not None:
                src = ident(cs[0])
                if (pushable(src) or col_slice(src) is not None) and src not in out_set:
                    readers_ok = True
                    stack = [src]
                    seen_r = set()
                    q0 = cs[0]
                    # every reader of src (through identity reshapes) is a column slice
                    front = [src]
                    while front and readers_ok:
                        q = front.pop()
                        for c in children[q]:
                            if isinstance(c.op, core.Reshape) and shape2(c) is not None and shape2(c) == shape2(q) and c not in out_set:
                                front.append(c)
                            elif col_slice(c) is None:
                                readers_ok = False
                    if readers_ok:
                        new = sliced(cs[0], cs[1], cs[2])
                        if new is not node:
                            replace[node] = new
        if not replace:
            break
        outputs, updatetargs = _rewire(outputs, updatetargs, replace)
    return list(outputs), list(updatetargs)


def _row_member(node, node2shape):
    """(R, C) when `node` can live in a FusedRows group over [R, C] rows: an elementwise float32 node of static shape
    [R, C] or [R, 1] (C is None then: it fits any row length), a Sum over axis 1 of an [R, C] node, or the Repeat of
    an [R, 1] node along axis 1. None otherwise."""
    if node.is_input() or node.ndim != 2 or node.dtype != "f4":
        return None
    shp = _static_shape(node2shape[node])
    if shp is None:
        return None
    (R, Cn) = shp
    op = node.op
    max_c = core.FusedRows.MAX_C
    if isinstance(op, core.Sum):
        par = node.parents[0]
        pshp = _static_shape(node2shape[par])
        if tuple(op.axes) != (1,) or par.dtype != "f4" or pshp is None or not (1 < pshp[1] <= max_c):
            return None
        return (R, pshp[1])
    if isinstance(op, core.MaskedRowSum):
        pshp = _static_shape(node2shape[node.parents[0]])
        if pshp is None or not (1 < pshp[1] <= max_c) or any(par.dtype != "f4" for par in node.parents):
            return None
        return (R, pshp[1])
    if isinstance(op, core.Repeat):
        par = node.parents[0]
        pshp = _static_shape(node2shape[par])
        if list(op.axes) != [1] or par.dtype != "f4" or pshp is None or pshp != (R, 1) or not (1 < Cn <= max_c):
            return None
        return (R, Cn)
    if _fusable(node) and all(par.dtype == "f4" or par.ndim == 0 for par in node.parents):
        if Cn == 1:
            return (R, None)
        if Cn <= max_c:
            return (R, Cn)
    return None


def fuse_flat_index_rows(outputs, updatetargs, node2shape):
    """x[arange(R), idx] on a float32 [R, C] matrix and its gradient, as row arithmetic. The front end spells the
    selection as GetFlatIndices(x, arange(R)*C + idx) (after constant folding: a constant vector 0, C, 2C, ... plus idx)
    and differentiates it into IncFlatIndices(zeros[R, C], the same indices, g). With H = OneHotRows{C}(idx):
        GetFlatIndices(x, K + idx)                -> Reshape(MaskedRowSum(x, H), [R])   (the row's selected element)
        IncFlatIndices(Fill{0}[R, C], K + idx, g) -> H * Repeat{1}(Reshape(g, [R, 1]), C)
    Every row holds exactly one selected element, so both forms give the reference's values (MaskedRowSum selects, it
    does not multiply: an infinite log-probability elsewhere in the row stays out; a row whose gradient g is not finite
    becomes NaN as a whole, where the reference leaves zeros beside the one element). For C <= 128 the row pass then takes them into the FusedRows chain around them, and the index
    arithmetic, the zero fill, the increment and the gather are no longer launched. Runs before fuse_elementwise."""
    all_out = list(outputs) + list(updatetargs)
    nodes = core.topsorted(all_out)
    out_set = set(all_out)
    const = lambda v: core.cgt.constant(np.array(v, "i8"))

    def row_index(ind, R, C):
        """idx when `ind` is (constant vector arange(R)*C) + idx with idx an int64 [R] node"""
        if ind.is_input() or not isinstance(ind.op, core.ElwiseBinary) or ind.op.opname != "+" or ind.dtype != "i8" or ind.ndim != 1:
            return None
        for (k, other) in ((ind.parents[0], ind.parents[1]), (ind.parents[1], ind.parents[0])):
            if isinstance(getattr(k, "op", None), core.Constant) and other.ndim == 1 and other.dtype == "i8":
                v = np.asarray(k.op.value)
                if v.shape == (R,) and np.array_equal(v, np.arange(R, dtype="i8") * C):
                    return other
        return None

    hot_of, replace = {}, {}

    def hot(idx, R, C):
        key = (idx, C)
        if key not in hot_of:
            h = core.Result(core.OneHotRows(C), [idx])
            node2shape[h] = [const(R), const(C)]
            hot_of[key] = h
        return hot_of[key]

    for node in nodes:
        if node.is_input() or node in out_set or node.dtype != "f4":
            continue
        if isinstance(node.op, core.GetFlatIndices):
            (x, ind) = node.parents
            shp = _static_shape(node2shape[x]) if x in node2shape else None
            if shp is None or len(shp) != 2 or x.dtype != "f4" or not (1 < shp[1] <= core.FusedRows.MAX_C):
                continue
            (R, C) = shp
            idx = row_index(ind, R, C)
            if idx is None:
                continue
            rowsum = core.Result(core.MaskedRowSum(), [x, hot(idx, R, C)])
            node2shape[rowsum] = [const(R), const(1)]
            new = core.Result(core.Reshape(), [rowsum, const(R)])
            node2shape[new] = [const(R)]
            replace[node] = new
        elif isinstance(node.op, core.IncFlatIndices):
            (z, ind, g) = node.parents
            shp = _static_shape(node2shape[node]) if node in node2shape else None
            if shp is None or len(shp) != 2 or not (1 < shp[1] <= core.FusedRows.MAX_C) or g.dtype != "f4" or g.ndim != 1:
                continue
            if z.is_input() or not isinstance(z.op, core.Fill) or float(z.op.value) != 0.0:
                continue
            (R, C) = shp
            idx = row_index(ind, R, C)
            if idx is None:
                continue
            gcol = core.Result(core.Reshape(), [g, const(R), const(1)])
            node2shape[gcol] = [const(R), const(1)]
            grep = core.Result(core.Repeat([1]), [gcol, const(C)])
            node2shape[grep] = [const(R), const(C)]
            new = core.Result(core.ElwiseBinary("*", (False, False)), [hot(idx, R, C), grep])
            node2shape[new] = [const(R), const(C)]
            replace[node] = new
    if not replace:
        return list(outputs), list(updatetargs)
    return _rewire(outputs, updatetargs, replace)


def fuse_elementwise(outputs, updatetargs, node2shape, rows=False):
    """Replace connected groups of elementwise nodes of one shape by FusedElwise nodes; with rows=True, connected
    groups of elementwise nodes, sums along axis 1 and repeats along axis 1 over [R, C] rows that contain at least one
    such sum by FusedRows nodes (groups without a sum are left for the plain pass).

    A node joins the group of one of its fusable parents when that cannot create a cycle (no other
    parent depends on the group). Groups stay within the kernel's limits; a group that would need
    several outputs while one of them is an update target (which must be written into the variable's
    own memory) is left alone. Returns the new (outputs, updatetargs)."""
    all_out = list(outputs) + list(updatetargs)
    nodes = core.topsorted(all_out)
    children = defaultdict(list)
    for node in nodes:
        for par in node.parents:
            children[par].append(node)
    # Group dependencies are kept as Python-int bitmasks (bit g = group g): anc[x] is the set of groups
    # that x depends on, directly or through other groups, at the time x is visited; gclosure[g] the
    # set of groups that group g depends on, kept transitively closed as groups grow. Joining g makes g
    # depend on every group among the node's other ancestors: that is allowed only if none of them
    # depends on g, or the fused nodes would need each other.
    group_of = {}
    members = defaultdict(list)
    anc = {}
    gclosure = []
    topo_index = dict((node, i) for (i, node) in enumerate(nodes))
    row_class = {}    # rows mode: node -> (R, C or None)
    group_rc = {}     # rows mode: group -> [R, C or None]

    def joinable(node, par, g):
        if par.ndim == 0:
            return False
        if not rows:
            return _same_shape(node2shape[node], node2shape[par])
        (R, C) = row_class[node]
        (Rg, Cg) = group_rc[g]
        return R == Rg and (C is None or Cg is None or C == Cg)

    def mergeable(g, g2):
        if not rows:
            return True
        (R, C), (R2, C2) = group_rc[g], group_rc[g2]
        return R == R2 and (C is None or C2 is None or C == C2)

    def closed(mask):
        """mask plus everything its groups depend on"""
        out, m = mask, mask
        while m:
            low = m & -m
            out |= gclosure[low.bit_length() - 1]
            m ^= low
        return out

    for node in nodes:
        parent_masks = []
        for par in node.parents:
            pm = anc[par]
            if par in group_of:
                pm |= 1 << group_of[par]
            parent_masks.append(pm)
        if rows:
            row_class[node] = _row_member(node, node2shape)
        if (row_class[node] is not None) if rows else _fusable(node):
            cands = []
            for par in node.parents:
                g = group_of.get(par)
                if g is None or g in cands or not joinable(node, par, g):
                    continue
                cands.append(g)
            chosen = None

            def n_ops(g):   # a Repeat costs the row kernel nothing: the value already sits in every lane
                return sum(1 for m in members[g] if not isinstance(m.op, core.Repeat)) if rows else len(members[g])
            for g in cands:
                if n_ops(g) >= core.FusedElwise.MAX_OPS:
                    continue
                # other parents' groups that neither depend on g nor g on them (x.W + b and h.U + c: two
                # independent chains that meet in this node) are merged into g
                merged = [g]
                for g2 in cands:
                    if g2 == g or any((gclosure[m] >> g2) & 1 or (gclosure[g2] >> m) & 1 for m in merged):
                        continue
                    if not all(mergeable(m, g2) for m in merged):
                        continue
                    if sum(n_ops(m) for m in merged) + n_ops(g2) >= core.FusedElwise.MAX_OPS:
                        continue
                    merged.append(g2)
                outside = 0
                for (q, pm) in zip(node.parents, parent_masks):
                    if group_of.get(q) not in merged:
                        outside |= pm
                outside = closed(outside)
                if any((outside >> m) & 1 for m in merged):
                    continue
                chosen = g
                deps = outside
                bits = 0
                for m in merged:
                    deps |= gclosure[m]
                    bits |= 1 << m
                for g2 in merged[1:]:
                    for mnode in members[g2]:
                        group_of[mnode] = g
                    members[g] = sorted(members[g] + members[g2], key=topo_index.__getitem__)
                    members[g2] = []
                    if rows and group_rc[g][1] is None:
                        group_rc[g][1] = group_rc[g2][1]
                if deps & ~gclosure[g] or len(merged) > 1:
                    for k in range(len(gclosure)):   # groups that depend on a merged group inherit the new dependencies
                        if gclosure[k] & bits:
                            gclosure[k] |= deps | (1 << g)
                    gclosure[g] = deps
                    for g2 in merged[1:]:
                        gclosure[g2] = deps | (1 << g)   # a stale reference to an emptied group sees the merged one
                break
            if chosen is None:
                chosen = len(gclosure)
                total = 0
                for pm in parent_masks:
                    total |= pm
                gclosure.append(closed(total))
            group_of[node] = chosen
            members[chosen].append(node)
            if rows:
                rc = group_rc.setdefault(chosen, list(row_class[node]))
                if rc[1] is None:
                    rc[1] = row_class[node][1]
        total = 0
        for pm in parent_masks:
            total |= pm
        anc[node] = closed(total) & ~((1 << group_of[node]) if node in group_of else 0)
    out_set = set(all_out)
    target_set = set(updatetargs)
    replace = {}
    config_views = core.get_config().get("fuse_slice_views", True)

    def emit(mem):
        """One FusedElwise node for `mem` (topologically ordered); a group beyond the kernel's limits is cut in two
        (a prefix and the rest of a topological order cannot need each other both ways) and each part tried again."""
        memset = set(mem)
        inputs, in_kinds, reg_of, views = [], [], {}, {}
        group_shape = _static_shape(node2shape[mem[0]])

        def column_view(par):
            """(matrix, first column, row length) when `par` is a column slice (through reshapes that change nothing)
            of a static float32 matrix and the group's index space is that slice's [R, W]"""
            if not config_views or group_shape is None or len(group_shape) != 2 or par.dtype != "f4":
                return None
            q = par
            while not q.is_input() and isinstance(q.op, core.Reshape) and _static_shape(node2shape[q]) == group_shape \
                    and _static_shape(node2shape[q.parents[0]]) == group_shape:
                q = q.parents[0]
            if q.is_input() or not isinstance(q.op, core.GetSli) or q.op.axis != 1 or _static_shape(node2shape[q]) != group_shape:
                return None
            (x, start, _stop, step) = q.parents
            xshp = _static_shape(node2shape[x])
            if x.dtype != "f4" or xshp is None or len(xshp) != 2 or xshp[0] != group_shape[0]:
                return None
            if not (isinstance(start.op, core.Constant) and isinstance(step.op, core.Constant)) or int(step.op.value) != 1:
                return None
            first = int(start.op.value)
            if first < 0 or first + group_shape[1] > xshp[1]:
                return None
            return (x, first, xshp[1])

        def input_reg(par):
            if par in reg_of:
                return reg_of[par]
            view = column_view(par) if par.ndim == 2 else None
            if par.ndim == 0:
                kind = 2 if par.dtype == "f4" else 3
                src = par
            elif view is not None:
                kind, src = 7, view[0]
                views[len(inputs)] = (view[1], view[2])
            elif _foldable_repeat(par):
                # the small operand is read directly; the Repeat node itself stays for whoever else uses it
                kind, src = 4, par.parents[0]
            else:
                kind = 0 if par.dtype == "f4" else 1
                src = par
            reg_of[par] = len(inputs)
            inputs.append(src)
            in_kinds.append(kind)
            return reg_of[par]

        for node in mem:   # inputs in order of first use
            for par in node.parents:
                if par not in memset:
                    input_reg(par)
        n_in = len(inputs)
        folded = sum(1 for k in in_kinds if k == 4)
        if len(mem) + folded < 2:
            return
        outs = [node for node in mem if node in out_set or any(c not in memset for c in children[node])]
        if n_in > core.FusedElwise.MAX_IN or len(outs) > core.FusedElwise.MAX_OUT or len(mem) > core.FusedElwise.MAX_OPS:
            if len(mem) >= 2:
                emit(mem[:len(mem) // 2])
                emit(mem[len(mem) // 2:])
            return
        if not outs:
            return
        if len(outs) > 1 and any(o in target_set for o in outs):
            # an update target must be the only result of its kernel (it is written into the variable's own memory):
            # one piece per target, holding the members that this target is the first to need (optimizers with several
            # state variables per parameter: one chain per state variable); halves when that separates nothing
            owner = {}
            for t in [node for node in mem if node in target_set]:   # in topological order
                stack = [t]
                while stack:
                    q = stack.pop()
                    if q in owner:
                        continue
                    owner[q] = t
                    stack.extend(par for par in q.parents if par in memset and par not in owner)
            pieces = defaultdict(list)
            for node in mem:
                pieces[owner.get(node)].append(node)
            if len(pieces) > 1:
                for piece in pieces.values():   # each piece: the members that its target needs first, in order
                    emit(piece)
            elif len(mem) >= 2:
                emit(mem[:len(mem) // 2])
                emit(mem[len(mem) // 2:])
            return
        program, result_reg = [], {}
        for (j, node) in enumerate(mem):
            regs = [result_reg[par] if par in memset else reg_of[par] for par in node.parents]
            if isinstance(node.op, core.ElwiseUnary):
                program.append((1, core.UNARY_OPCODE[node.op.opname], regs[0], 0))
            else:
                program.append((2, core.BINARY_OPCODE[node.op.opname], regs[0], regs[1]))
            result_reg[node] = n_in + j
        shape_input = None
        for (k, (src, kind)) in enumerate(zip(inputs, in_kinds)):
            if kind in (0, 1) and _same_shape(node2shape[src], node2shape[mem[0]]):
                shape_input = k
                break
        if shape_input is None and group_shape is None:
            return
        descr = ",".join(str(node.op) for node in mem)
        fop = core.FusedElwise(program, in_kinds, [result_reg[o] for o in outs], [o.dtype for o in outs], mem[0].ndim,
                               shape_input, descr, views=views, static_shape=group_shape if (views or shape_input is None) else None)
        fnode = core.Result(fop, inputs)
        shp = node2shape[mem[0]]
        if len(outs) == 1:
            node2shape[fnode] = shp
            replace[outs[0]] = fnode
            fnode.props.update(outs[0].props)
        else:
            node2shape[fnode] = tuple(list(shp) for _ in outs)
            fnode.props.update(outs[0].props)
            for (q, o) in enumerate(outs):
                ti = core.Result(core.TupleIndex(q), [fnode])
                node2shape[ti] = shp
                replace[o] = ti

    def emit_rows(mem):
        """One FusedRows node for `mem`, if it holds a sum; halves of a group beyond the kernel's limits are tried again."""
        if not any(isinstance(node.op, (core.Sum, core.MaskedRowSum)) for node in mem):
            return
        F = core.FusedElwise
        memset = set(mem)
        C = None
        for node in mem:
            C = C or row_class[node][1]
        if C is None:
            return
        inputs, in_kinds, reg_of = [], [], {}

        def data_parents(node):
            return node.parents[:1] if isinstance(node.op, (core.Sum, core.Repeat)) else node.parents

        def input_reg(par):
            if par in reg_of:
                return reg_of[par]
            src = par
            if par.ndim == 0:
                kind = 2 if par.dtype == "f4" else 3
            else:
                shp = _static_shape(node2shape[par])
                if par.dtype != "f4" or shp is None or len(shp) != 2:
                    return None
                if not par.is_input() and isinstance(par.op, core.OneHotRows) and shp[1] == C and par.parents[0].dtype == "i8":
                    kind, src = 8, par.parents[0]      # the selection matrix of a column number per row: read the numbers
                elif isinstance(par.op, core.Repeat) and not par.is_input() and list(par.op.axes) == [0] and shp[1] == C \
                        and par.parents[0].dtype == "f4":
                    kind, src = 6, par.parents[0]      # a [1, C] row repeated down the rows: read the row itself
                elif shp[1] == C:
                    kind = 0
                elif shp[1] == 1:
                    kind = 5
                else:
                    return None
            reg_of[par] = len(inputs)
            inputs.append(src)
            in_kinds.append(kind)
            return reg_of[par]

        for node in mem:
            for par in data_parents(node):
                if par not in memset and input_reg(par) is None:
                    return
        n_in = len(inputs)
        n_ops = sum(1 for node in mem if not isinstance(node.op, core.Repeat))
        outs = [node for node in mem if node in out_set or any(c not in memset for c in children[node])]
        if n_in > F.MAX_IN or len(outs) > F.MAX_OUT or n_ops > F.MAX_OPS:
            if len(mem) >= 2:
                emit_rows(mem[:len(mem) // 2])
                emit_rows(mem[len(mem) // 2:])
            return
        if not outs or any(o in target_set for o in outs) or n_ops < 2:
            return
        program, result_reg = [], {}
        for node in mem:
            regs = [result_reg[par] if par in memset else reg_of[par] for par in data_parents(node)]
            if isinstance(node.op, core.Repeat):
                result_reg[node] = regs[0]     # one value per row already sits in every lane
                continue
            if isinstance(node.op, core.Sum):
                program.append((3, 0, regs[0], 0))
            elif isinstance(node.op, core.MaskedRowSum):
                program.append((4, 0, regs[0], regs[1]))
            elif isinstance(node.op, core.ElwiseUnary):
                program.append((1, core.UNARY_OPCODE[node.op.opname], regs[0], 0))
            else:
                program.append((2, core.BINARY_OPCODE[node.op.opname], regs[0], regs[1]))
            result_reg[node] = n_in + len(program) - 1
        shape_input = None
        for (k, kind) in enumerate(in_kinds):
            if kind in (0, 5, 8):
                shape_input = k
                break
        if shape_input is None:
            return
        descr = ",".join(str(node.op) for node in mem if not isinstance(node.op, core.Repeat))
        out_cols = [_static_shape(node2shape[o])[1] == 1 for o in outs]
        fop = core.FusedRows(program, in_kinds, [result_reg[o] for o in outs], out_cols, C, shape_input, descr)
        fnode = core.Result(fop, inputs)
        fnode.props.update(outs[0].props)
        if len(outs) == 1:
            node2shape[fnode] = node2shape[outs[0]]
            replace[outs[0]] = fnode
        else:
            node2shape[fnode] = tuple(list(node2shape[o]) for o in outs)
            for (q, o) in enumerate(outs):
                ti = core.Result(core.TupleIndex(q), [fnode])
                node2shape[ti] = node2shape[o]
                replace[o] = ti

    for mem in list(members.values()):
        if mem:
            (emit_rows if rows else emit)(mem)
    if not replace:
        return list(outputs), list(updatetargs)
    return _rewire(outputs, updatetargs, replace)


def _rewire(outputs, updatetargs, replace):
    """Point every surviving consumer at the replacement nodes (the replacements' own inputs included)."""
    seen = set()
    stack = [replace.get(o, o) for o in list(outputs) + list(updatetargs)]
    while stack:
        node = stack.pop()
        if node in seen or node.is_input():
            continue
        seen.add(node)
        for (pos, par) in enumerate(node.parents):
            if par in replace:
                node.parents[pos] = replace[par]
            stack.append(node.parents[pos])
    return [replace.get(o, o) for o in outputs], [replace.get(o, o) for o in updatetargs]


def fuse_conv_dgrad(outputs, updatetargs, node2shape):
    """Col2Im(Reshape(Mul22{N,N}(Reshape(dy NHWC), Reshape(W)))) -> ConvDgrad(dy, W) (the filter bank as stored;
    the kernel's filter-splitting pass rearranges it) for stride-1 convolutions whose extents the kernel supports (input channels of the
    product a multiple of 32, at most 128 image channels in multiples of 16, rows of at most 128 pixels).
    The intermediate nodes must have no other consumer."""
    from .nn_ops import im2col as im2col_ops
    all_out = list(outputs) + list(updatetargs)
    nodes = core.topsorted(all_out)
    nchildren = defaultdict(int)
    for node in nodes:
        for par in node.parents:
            nchildren[par] += 1
    out_set = set(all_out)
    replace = {}
    for node in nodes:
        if node.is_input() or not isinstance(node.op, im2col_ops.Col2Im) or node.dtype != "f4":
            continue
        info = node.op.info
        if info.stride_h != 1 or info.stride_w != 1:
            continue
        r1 = node.parents[0]
        if r1.is_input() or not isinstance(r1.op, core.Reshape) or nchildren[r1] != 1 or r1 in out_set:
            continue
        m = r1.parents[0]
        if m.is_input() or not isinstance(m.op, core.Mul22) or m.op.tA or m.op.tB or nchildren[m] != 1 or m in out_set:
            continue
        (a, w2) = m.parents
        if a.is_input() or w2.is_input() or not isinstance(a.op, core.Reshape) or not isinstance(w2.op, core.Reshape):
            continue
        t4, w4 = a.parents[0], w2.parents[0]
        if t4.ndim != 4 or w4.ndim != 4 or t4.dtype != "f4" or w4.dtype != "f4":
            continue
        shapes = [_static_shape(node2shape[x]) if x in node2shape else None for x in (node, t4, w4, a, r1)]
        if any(sh is None for sh in shapes):
            continue
        (dx_s, t4_s, w4_s, a_s, r1_s) = shapes
        (B, C, H, W) = dx_s
        (Bt, Ho, Wo, Cin) = t4_s
        if Bt != B or w4_s != (Cin, C, info.kernel_h, info.kernel_w) or a_s != (B * Ho * Wo, Cin):
            continue
        if r1_s != (B, Ho, Wo, C * info.kernel_h * info.kernel_w):
            continue
        if Ho != H + 2 * info.pad_h - info.kernel_h + 1 or Wo != W + 2 * info.pad_w - info.kernel_w + 1:
            continue
        if Cin % 32 != 0 or C % 16 != 0 or C > 128 or W > 128:
            continue
        dx = core.Result(im2col_ops.ConvDgrad(info, w_bank=True), [t4, w4] + list(node.parents[1:]))
        node2shape[dx] = node2shape[node]
        dx.props.update(node.props)
        replace[node] = dx
    if not replace:
        return list(outputs), list(updatetargs)
    return _rewire(outputs, updatetargs, replace)


def fuse_conv_output(outputs, updatetargs, node2shape):
    """FusedElwise{add bias, >= 0, multiply}(Transpose{0,3,1,2}(Reshape(Mul22{N,T}(col, W)))) -> ConvBiasRelu(col, W, bias).
    Runs after fuse_elementwise; the GEMM, reshape and transpose nodes must have no other consumer."""
    from .nn_ops import im2col as im2col_ops
    all_out = list(outputs) + list(updatetargs)
    nodes = core.topsorted(all_out)
    nchildren = defaultdict(int)
    for node in nodes:
        for par in node.parents:
            nchildren[par] += 1
    out_set = set(all_out)
    want_program = [(2, core.BINARY_OPCODE["+"], 0, 1), (2, core.BINARY_OPCODE[">="], 3, 2), (2, core.BINARY_OPCODE["*"], 3, 4)]
    replace = {}
    for node in nodes:
        if node.is_input() or not isinstance(node.op, core.FusedElwise):
            continue
        op = node.op
        if (op.program != want_program or op.in_kinds != [0, 4, 3] or op.out_regs != [4, 5] or op.out_dtypes != ["i1", "f4"]
                or op.ndim != 4):
            continue
        (t, bias, zero) = node.parents
        if not _small_int_constant(zero) or int(np.asarray(zero.op.value).reshape(-1)[0]) != 0:
            continue
        if t.is_input() or not isinstance(t.op, core.Transpose) or list(t.op.axes) != [0, 3, 1, 2] or nchildren[t] != 1 or t in out_set:
            continue
        r = t.parents[0]
        if r.is_input() or not isinstance(r.op, core.Reshape) or nchildren[r] != 1 or r in out_set:
            continue
        m = r.parents[0]
        if m.is_input() or not isinstance(m.op, core.Mul22) or m.op.tA or not m.op.tB or nchildren[m] != 1 or m in out_set:
            continue
        if m.dtype != "f4" or bias.dtype != "f4" or bias.ndim != 4:
            continue
        shp = node2shape[node][0]
        static = _static_shape(shp)
        if static is None or static[1] > 384:   # the kernel stages 128 pixels x C channels in shared memory
            continue
        new = core.Result(im2col_ops.ConvBiasRelu(), [m.parents[0], m.parents[1], bias] + list(shp))
        node2shape[new] = node2shape[node]
        new.props.update(node.props)
        replace[node] = new
    if not replace:
        return list(outputs), list(updatetargs)
    return _rewire(outputs, updatetargs, replace)


def fuse_conv_grad_input(outputs, updatetargs, node2shape):
    """X = mask * g (relu pullback, NCHW) consumed only by Transpose{0,2,3,1}(X) and Sum{0,2,3}(X) -> one
    ReluGradNHWC(mask, g) node whose two outputs replace the transpose and the sum."""
    from .nn_ops import im2col as im2col_ops
    all_out = list(outputs) + list(updatetargs)
    nodes = core.topsorted(all_out)
    children = defaultdict(list)
    for node in nodes:
        for par in node.parents:
            children[par].append(node)
    out_set = set(all_out)
    replace = {}
    for x in nodes:
        if x.is_input() or not isinstance(x.op, core.ElwiseBinary) or x.op.opname != "*" or x.ndim != 4 or x.dtype != "f4" or x in out_set:
            continue
        (a, b) = x.parents
        if a.ndim != 4 or b.ndim != 4:
            continue
        if a.dtype == "i1" and b.dtype == "f4":
            (mask, g) = (a, b)
        elif b.dtype == "i1" and a.dtype == "f4":
            (mask, g) = (b, a)
        else:
            continue
        cs = children[x]
        if len(cs) != 2:
            continue
        t = [c for c in cs if isinstance(c.op, core.Transpose) and list(c.op.axes) == [0, 2, 3, 1]]
        sm = [c for c in cs if isinstance(c.op, core.Sum) and tuple(c.op.axes) == (0, 2, 3)]
        if len(t) != 1 or len(sm) != 1:
            continue
        static = _static_shape(node2shape[x]) if x in node2shape else None
        if static is None or static[1] > 384 or static[0] > 65535:
            continue
        new = core.Result(im2col_ops.ReluGradNHWC(), [mask, g])
        node2shape[new] = (node2shape[t[0]], node2shape[sm[0]])
        new.props.update(x.props)
        for (q, old) in enumerate((t[0], sm[0])):
            ti = core.Result(core.TupleIndex(q), [new])
            node2shape[ti] = node2shape[old]
            replace[old] = ti
    if not replace:
        return list(outputs), list(updatetargs)
    return _rewire(outputs, updatetargs, replace)


def fuse_conv_implicit(outputs, updatetargs, node2shape):
    """ConvBiasRelu(Reshape(Im2Col(x)), Reshape(W), bias, ...) -> ConvFwdBiasRelu(x NHWC, W, bias, ...)
    and, for the same column matrix, Mul22{T,N}(Reshape(dy NHWC), Reshape(Im2Col(x))) -> ConvWgradImplicit(x NHWC, dy NHWC),
    for stride-1 convolutions whose extents the kernels support (input channels a multiple of 32, output channels a
    multiple of 16, rows of at most 32 pixels). Applies only when every consumer of the column matrix is one of the
    two, so that Im2Col disappears; the one NCHW -> NHWC transpose of x serves both. Runs after fuse_conv_output."""
    from .nn_ops import im2col as im2col_ops
    all_out = list(outputs) + list(updatetargs)
    nodes = core.topsorted(all_out)
    children = defaultdict(list)
    for node in nodes:
        for par in node.parents:
            children[par].append(node)
    out_set = set(all_out)
    replace = {}
    for im in nodes:
        if im.is_input() or not isinstance(im.op, im2col_ops.Im2Col) or im.op.pitch or im.dtype != "f4" or im in out_set:
            continue
        info = im.op.info
        if info.stride_h != 1 or info.stride_w != 1 or len(children[im]) != 1:
            continue
        r = children[im][0]
        if not isinstance(r.op, core.Reshape) or r in out_set or r.ndim != 2 or r.parents[0] is not im:
            continue
        x = im.parents[0]
        x_s = _static_shape(node2shape[x]) if x in node2shape else None
        im_s = _static_shape(node2shape[im]) if im in node2shape else None
        if x_s is None or im_s is None or len(x_s) != 4:
            continue
        (B, Cin, H, W) = x_s
        (_b, Ho, Wo, Z) = im_s
        if Cin % 32 != 0 or Wo > 32 or Z != Cin * info.kernel_h * info.kernel_w:
            continue
        fwd, wgrads, ok = [], [], bool(children[r])
        for c in children[r]:
            if isinstance(c.op, im2col_ops.ConvBiasRelu) and c.parents[0] is r and r not in c.parents[1:]:
                w2 = c.parents[1]
                shp = _static_shape(node2shape[c][0]) if c in node2shape else None
                if (not w2.is_input() and isinstance(w2.op, core.Reshape) and w2.parents[0].ndim == 4 and shp is not None
                        and _static_shape(node2shape[w2.parents[0]]) == (shp[1], Cin, info.kernel_h, info.kernel_w)
                        and shp == (B, shp[1], Ho, Wo) and _conv_channels_ok(shp[1])):
                    fwd.append(c)
                    continue
            if (isinstance(c.op, core.Mul22) and c.op.tA and not c.op.tB and c.parents[1] is r and c.parents[0] is not r
                    and c.dtype == "f4"):
                a = c.parents[0]
                if not a.is_input() and isinstance(a.op, core.Reshape) and a.parents[0].ndim == 4 and a.parents[0].dtype == "f4":
                    dy_s = _static_shape(node2shape[a.parents[0]]) if a.parents[0] in node2shape else None
                    if dy_s is not None and dy_s[:3] == (B, Ho, Wo) and _conv_channels_ok(dy_s[3]):
                        wgrads.append(c)
                        continue
            ok = False
        if not ok or not fwd:
            continue
        xs = node2shape[x]
        xt = core.Result(core.Transpose((0, 2, 3, 1)), [x])
        node2shape[xt] = [xs[0], xs[2], xs[3], xs[1]]
        xt.props.update(im.props)
        for c in fwd:
            w4 = c.parents[1].parents[0]
            new = core.Result(im2col_ops.ConvFwdBiasRelu(info, w_bank=True), [xt, w4] + list(c.parents[2:]))
            node2shape[new] = node2shape[c]
            new.props.update(c.props)
            replace[c] = new
        for c in wgrads:
            new = core.Result(im2col_ops.ConvWgradImplicit(info), [xt, c.parents[0].parents[0]])
            node2shape[new] = node2shape[c]
            new.props.update(c.props)
            replace[c] = new
    if not replace:
        return list(outputs), list(updatetargs)
    return _rewire(outputs, updatetargs, replace)


def _conv_channels_ok(n):
    return n % 16 == 0 and (n <= 128 or n % 128 == 0)


def _direct_wgrad_with_relu(c, x, info, children, out_set, node2shape, replace):
    """The filter gradient c = Mul22{T,N}(Reshape(TupleIndex{0}(ReluGradNHWC(mask, g))), col) of a first layer: when the
    channels-last gradient has no other reader, c and the bias gradient TupleIndex{1} become the two outputs of one
    ConvDirectWgradRelu(x, mask, g). Returns True when it registered the replacements."""
    from .nn_ops import im2col as im2col_ops
    r2 = c.parents[0]
    if r2.is_input() or not isinstance(r2.op, core.Reshape) or r2 in out_set or len(children[r2]) != 1:
        return False
    t0 = r2.parents[0]
    if t0.is_input() or not isinstance(t0.op, core.TupleIndex) or t0.op.idx != 0 or t0 in out_set or len(children[t0]) != 1:
        return False
    rg = t0.parents[0]
    if rg.is_input() or not isinstance(rg.op, im2col_ops.ReluGradNHWC) or rg in out_set:
        return False
    others = [t for t in children[rg] if t is not t0]
    if any(t.is_input() or not isinstance(t.op, core.TupleIndex) or t.op.idx != 1 for t in others):
        return False
    (mask, g) = rg.parents
    gs = _static_shape(node2shape[g]) if g in node2shape else None
    xs = _static_shape(node2shape[x])
    if gs is None or gs != (xs[0], 32, xs[2], xs[3]) or mask.dtype != "i1" or g.dtype != "f4":
        return False
    new = core.Result(im2col_ops.ConvDirectWgradRelu(info, 32), [x, mask, g])
    node2shape[new] = (node2shape[c], node2shape[rg][1])
    new.props.update(c.props)
    dw = core.Result(core.TupleIndex(0), [new])
    node2shape[dw] = node2shape[c]
    replace[c] = dw
    for t in others:
        db = core.Result(core.TupleIndex(1), [new])
        node2shape[db] = node2shape[t]
        replace[t] = db
    return True


def fuse_conv_direct(outputs, updatetargs, node2shape):
    """Im2Col of an image with 3 channels (5 x 5 filters, pad 2, stride 1, 32 pixels wide, 32 filters) whose column matrix
    feeds only the layer's forward product (ConvBiasRelu) and its filter gradient (Mul22{T,N}(dy, col)): both are
    computed directly from the image (ConvDirectFwd, ConvDirectWgrad) and the column matrix, 25 times the image, is
    never formed. Runs before pad_conv_columns, which would otherwise widen that matrix."""
    from .nn_ops import im2col as im2col_ops
    all_out = list(outputs) + list(updatetargs)
    nodes = core.topsorted(all_out)
    children = defaultdict(list)
    for node in nodes:
        for par in node.parents:
            children[par].append(node)
    out_set = set(all_out)
    replace = {}
    for im in nodes:
        if im.is_input() or not isinstance(im.op, im2col_ops.Im2Col) or im.op.pitch or im.dtype != "f4" or im in out_set:
            continue
        info = im.op.info
        if tuple(info) != (5, 5, 2, 2, 1, 1) or len(children[im]) != 1:
            continue
        x = im.parents[0]
        xs = _static_shape(node2shape[x]) if x in node2shape else None
        if xs is None or len(xs) != 4 or xs[1] != 3 or xs[3] != 32 or xs[2] % 8 != 0 or x.dtype != "f4":
            continue
        r = children[im][0]
        if not isinstance(r.op, core.Reshape) or r in out_set or r.ndim != 2 or r.parents[0] is not im:
            continue
        fwd = [c for c in children[r] if isinstance(c.op, im2col_ops.ConvBiasRelu) and c.parents[0] is r and r not in c.parents[1:]]
        wgs = [c for c in children[r] if isinstance(c.op, core.Mul22) and c.op.tA and not c.op.tB and c.parents[1] is r
               and c.parents[0] is not r and c.dtype == "f4" and c not in out_set]
        if len(fwd) != 1 or len(fwd) + len(wgs) != len(children[r]) or len(wgs) > 1:
            continue
        f = fwd[0]
        wshape = _static_shape(node2shape[f.parents[1]])
        if wshape != (32, 75):
            continue
        new_f = core.Result(im2col_ops.ConvDirectFwd(info), [x] + list(f.parents[1:]))
        node2shape[new_f] = node2shape[f]
        new_f.props.update(f.props)
        replace[f] = new_f
        for c in wgs:
            fused = _direct_wgrad_with_relu(c, x, info, children, out_set, node2shape, replace)
            if fused:
                continue
            new_w = core.Result(im2col_ops.ConvDirectWgrad(info, 32), [x, c.parents[0]])
            node2shape[new_w] = node2shape[c]
            new_w.props.update(c.props)
            replace[c] = new_w
    if not replace:
        return list(outputs), list(updatetargs)
    return _rewire(outputs, updatetargs, replace)


def hoist_filter_splits(outputs, updatetargs, node2shape):
    """ConvFwdBiasRelu / ConvDgrad on a layer's stored filter bank each start with a small kernel that writes the
    bank's K-major [w_hi | w_lo] copy. All such copies of the step (at most eight per node) are made by one
    SplitFilterBanks node instead, and the convolutions take their copy as an extra input: four launches become one in
    the CIFAR-shape step. Applies to banks of static shape; needs at least two convolutions to pay."""
    from .nn_ops import im2col as im2col_ops
    all_out = list(outputs) + list(updatetargs)
    nodes = core.topsorted(all_out)
    jobs_nodes = []
    for node in nodes:
        if node.is_input() or not isinstance(node.op, (im2col_ops.ConvFwdBiasRelu, im2col_ops.ConvDgrad)):
            continue
        if not node.op.w_bank or node.op.pre:
            continue
        bank = node.parents[1]
        shp = _static_shape(node2shape[bank]) if bank in node2shape else None
        if shp is None or len(shp) != 4 or bank.dtype != "f4":
            continue
        taps = shp[2] * shp[3]
        if isinstance(node.op, im2col_ops.ConvFwdBiasRelu):
            job = (shp[0], shp[1], taps, 1)        # bank [Cout, Cin, kh, kw]: rows = Cout, source channels = Cin
        else:
            job = (shp[1], shp[0], taps, 2)        # the same bank read for the data gradient: rows = Cin, source channels = Cout
        jobs_nodes.append((node, bank, job))
    if len(jobs_nodes) < 2:
        return list(outputs), list(updatetargs)
    replace = {}
    const = lambda v: core.cgt.constant(np.array(v, "i8"))
    for lo in range(0, len(jobs_nodes), im2col_ops.SplitFilterBanks.MAX_JOBS):
        chunk = jobs_nodes[lo:lo + im2col_ops.SplitFilterBanks.MAX_JOBS]
        banks = []
        for (_node, bank, _job) in chunk:
            if bank not in banks:
                banks.append(bank)
        split = core.Result(im2col_ops.SplitFilterBanks([(banks.index(bank),) + job for (_node, bank, job) in chunk]), banks)
        node2shape[split] = tuple([const(2), const(job[0]), const(job[2] * job[1])] for (_node, _bank, job) in chunk)
        for (j, (node, _bank, job)) in enumerate(chunk):
            piece = core.Result(core.TupleIndex(j), [split])
            node2shape[piece] = [const(2), const(job[0]), const(job[2] * job[1])]
            new = core.Result(type(node.op)(node.op.info, w_bank=True, pre=True), list(node.parents) + [piece])
            node2shape[new] = node2shape[node]
            new.props.update(node.props)
            replace[node] = new
    return _rewire(outputs, updatetargs, replace)


def pad_conv_columns(outputs, updatetargs, node2shape):
    """Widen the rows of a float32 column matrix whose length Z = C*kh*kw is not a multiple of four (a 3-channel
    5x5 convolution: 75) to the next multiple, so that every row starts on a 16-byte boundary and the products
    that read it can be fed by the tensor-memory accelerator. Applies when Im2Col feeds exactly one
    Reshape to [M, Z] whose consumers are the forward product (ConvBiasRelu) and / or the filter gradient
    (Mul22{T,N}(dy, col)); those become ConvBiasRelu on the padded matrix and ConvWgrad{Z}. Runs last."""
    from .nn_ops import im2col as im2col_ops
    all_out = list(outputs) + list(updatetargs)
    nodes = core.topsorted(all_out)
    children = defaultdict(list)
    for node in nodes:
        for par in node.parents:
            children[par].append(node)
    out_set = set(all_out)
    replace = {}
    for im in nodes:
        if im.is_input() or not isinstance(im.op, im2col_ops.Im2Col) or im.op.pitch or im.dtype != "f4" or im in out_set:
            continue
        if len(children[im]) != 1:
            continue
        r = children[im][0]
        if not isinstance(r.op, core.Reshape) or r in out_set or r.ndim != 2 or r.parents[0] is not im:
            continue
        im_s = _static_shape(node2shape[im]) if im in node2shape else None
        r_s = _static_shape(node2shape[r]) if r in node2shape else None
        if im_s is None or r_s is None:
            continue
        z = im_s[3]
        if z % 4 == 0 or r_s != (im_s[0] * im_s[1] * im_s[2], z):
            continue
        ok = bool(children[r])
        for c in children[r]:
            if isinstance(c.op, im2col_ops.ConvBiasRelu) and c.parents[0] is r and r not in c.parents[1:]:
                continue
            if (isinstance(c.op, core.Mul22) and c.op.tA and not c.op.tB and c.parents[1] is r and c.parents[0] is not r
                    and c.dtype == "f4" and c not in out_set):
                continue
            ok = False
        if not ok:
            continue
        pitch = (z + 3) // 4 * 4
        pitch_node = core.cgt.constant(pitch)
        im2 = core.Result(im2col_ops.Im2Col(im.op.info, pitch=pitch), list(im.parents))
        node2shape[im2] = list(node2shape[im][:3]) + [pitch_node]
        im2.props.update(im.props)
        r2 = core.Result(core.Reshape(), [im2, r.parents[1], pitch_node])
        node2shape[r2] = [node2shape[r][0], pitch_node]
        r2.props.update(r.props)
        replace[r] = r2
        for c in children[r]:
            if isinstance(c.op, core.Mul22):
                wg = core.Result(im2col_ops.ConvWgrad(z), [c.parents[0], r2])
                node2shape[wg] = node2shape[c]
                wg.props.update(c.props)
                replace[c] = wg
    if not replace:
        return list(outputs), list(updatetargs)
    return _rewire(outputs, updatetargs, replace)


def prebuild_fused_kernels(builders):
    """Generate and compile the fused-chain kernels of the given configurations into the library cache
    (no GPU needed: nvcc cross-compiles), so that a later run finds them instead of compiling."""
    from . import codegen
    n = 0
    for build in builders:
        cfg = build()
        outs, _usrc, utargs, analysis = simplify_for_execution([cfg.loss] + list(cfg.extra_outputs), cfg.updates)
        o2, u2 = apply_graph_rewrites(outs, utargs, analysis["node2shape"])
        for node in core.topsorted(o2 + u2):
            if node.is_input():
                continue
            if isinstance(node.op, core.FusedElwise) and codegen.fused_launcher(node.op):
                n += 1
            if isinstance(node.op, core.FusedRows) and codegen.rows_launcher(node.op):
                n += 1
    return n


# ================================================================
# Phase 2: devices and transports
# ================================================================

def _meta_inputs(op, n):
    f = getattr(op, "meta_inputs", None)
    return tuple(f(n)) if f else ((0,) if isinstance(op, core.Size) else ())


def determine_devices(nodes_sorted, updatetarg2src):
    """Reference rule (cgt/compilation.py:45-80)."""
    node2dev = {}
    home_device = core.Device(devtype="cpu", idx=0)
    for node in nodes_sorted:
        default_device = node.props.get("default_device", home_device)
        if node.is_scalar():
            device = home_device
        elif node in updatetarg2src:
            device = node2dev[updatetarg2src[node]]
            assert "native_" + device.devtype in node.op.available_impls, \
                "update only works if final operation can be performed on target device"
        elif node.is_data():
            device = node.op.device
        elif node.is_argument():
            device = home_device
        else:
            impls = node.op.available_impls
            if ("native_gpu" in impls) and ((default_device.devtype == "gpu") or ("native_cpu" not in impls)):
                device = core.Device("gpu", default_device.idx)
            else:
                device = core.Device(devtype="cpu", idx=default_device.idx)
        node2dev[node] = device
    return node2dev


def add_transports(nodelist, node2dev, node2shape):
    """One Transport per (node, consumer device) pair (cgt/compilation.py:285-304); operands that an
    Op reads on the host stay on the host, operands of which only the shape is used are not moved."""
    node2child = defaultdict(list)
    for node in nodelist:
        for (pos, par) in enumerate(node.parents):
            node2child[par].append((node, pos))
    home = core.Device("cpu", 0)
    for node in nodelist:
        dev = node2dev[node]
        dev2copy = {}
        for (child, pos) in node2child[node]:
            if child.is_input():
                continue
            n = len(child.parents)
            if pos in _meta_inputs(child.op, n):
                continue
            want = home if pos in child.op.host_inputs(n) else node2dev[child]
            if isinstance(child.op, core.Transport):
                continue
            if want.devtype != dev.devtype or (want.devtype == "gpu" and want.idx != dev.idx):
                if want not in dev2copy:
                    nodecopy = core.Result(core.Transport(want), [node])
                    node2dev[nodecopy] = want
                    dev2copy[want] = nodecopy
                    node2shape[nodecopy] = node2shape[node]
                child.parents[pos] = dev2copy[want]


# ================================================================
# Phase 3: ordering, memory owners, execution graph
# ================================================================

def is_tensor(x):
    return isinstance(x.typ, core.TensorType)


def is_tuple(x):
    return isinstance(x.typ, core.TupleType)


def _update_control_deps(outputs_all, updates):
    """after -> nodes that must run before it: every other reader of the variable it overwrites."""
    if not updates:
        return {}
    nodelist = core.topsorted(outputs_all)
    children = defaultdict(list)
    for node in nodelist:
        for p in node.parents:
            children[p].append(node)
    extra = {}
    for (before, after) in updates:
        # descendants of `after` cannot be ordered before it
        desc = set([after])
        for node in nodelist:
            if any(p in desc for p in node.parents):
                desc.add(node)
        readers = []
        stack = list(children[before])
        seen = set()
        while stack:
            c = stack.pop()
            if c in seen or c in desc:
                continue
            seen.add(c)
            readers.append(c)
            # views of the variable alias its memory: their readers count too
            if c.op.return_type == "byval":
                stack.extend(children[c])
        extra[after] = readers
    return extra


def _transport_schedule(outputs_all, updatetargs, node2dev):
    """Copies at the edges of a step, so that the device work between them is one uninterrupted span (one CUDA
    graph): (first) the host->device Transports of function arguments, which depend on nothing else, are
    scheduled before everything; (last) a device->host Transport whose descendants all live on the host and
    include no update (the loss and the host arithmetic that finishes it) is scheduled after every update."""
    nodelist = core.topsorted(outputs_all)
    children = defaultdict(list)
    for node in nodelist:
        for p in node.parents:
            children[p].append(node)
    targs = set(updatetargs)
    first, last = [], []
    for node in nodelist:
        if node.is_input() or not isinstance(node.op, core.Transport):
            continue
        src = node.parents[0]
        if src.is_argument() and node2dev[node].devtype == "gpu":
            first.append(node)
        elif node2dev[node].devtype == "cpu" and node2dev[src].devtype == "gpu" and node not in targs:
            ok, seen, stack = True, set(), list(children[node])
            while stack and ok:
                c = stack.pop()
                if c in seen:
                    continue
                seen.add(c)
                ok = node2dev[c].devtype == "cpu" and c not in targs
                stack.extend(children[c])
            if ok:
                last.append(node)
    return first, last


def topsorted_shapes_first(outputs, node2shape, extra_parents=None):
    """Topological order in which the shape components of a byref node precede it
    (cgt/compilation.py:109-148), plus the control dependencies in `extra_parents`."""
    extra_parents = extra_parents or {}
    marks = {}
    out = []
    stack = []
    for x in outputs:
        stack.append((x, 0))
        while stack:
            (i, jidx) = stack.pop()
            if jidx == 0:
                m = marks.get(i, 0)
                if m == 0:
                    marks[i] = 1
                elif m == 1:
                    raise ValueError("not a dag")
                else:
                    continue
            ps = list(i.parents)
            if i.ndim > 0 and not i.is_input() and i.op.return_type == "byref":
                ps = ps + list(node2shape[i])
            elif is_tuple(i) and not i.is_input():
                for arrshp in node2shape[i]:
                    ps = ps + list(arrshp)
            ps = ps + extra_parents.get(i, [])
            if jidx == len(ps):
                marks[i] = 2
                out.append(i)
            else:
                stack.append((i, jidx + 1))
                stack.append((ps[jidx], 0))
    return out


def _same_shape(shp1, shp2):
    if isinstance(shp1, tuple) or isinstance(shp2, tuple) or len(shp1) != len(shp2):
        return False
    for (a, b) in zip(shp1, shp2):
        if a is b:
            continue
        if isinstance(a.op, core.Constant) and isinstance(b.op, core.Constant) and a.op.value == b.op.value:
            continue
        return False
    return True


def compute_const_nodes(nodes_sorted):
    """Nodes whose value is the same on every run: constants and pure functions of constants."""
    const = set()
    for node in nodes_sorted:
        if node.is_input():
            continue
        if isinstance(node.op, core.Constant):
            const.add(node)
        elif node.op.is_random_op:
            continue
        elif len(node.parents) > 0 and all(p in const for p in node.parents):
            const.add(node)
        elif isinstance(node.op, core.Fill) and len(node.parents) == 0:
            const.add(node)
    return const


def determine_memowner(nodes_sorted, updates, node2dev, outputs, node2shape, const_nodes):
    """Which node's memory each node writes into (cgt/compilation.py:150-189).

    In-place reuse of a parent's buffer is limited to elementwise Ops (safe to run in place), to parents
    with one consumer, equal shape and dtype, and never touches constants (they are computed once).
    """
    node2child = defaultdict(list)
    for node in nodes_sorted:
        for parent in node.parents:
            node2child[parent].append(node)
    node2memowner = {}
    after2before = {after: before for (before, after) in updates}
    enable_inplace_opt = core.get_config()["enable_inplace_opt"]
    outputs = set(outputs)
    for node in nodes_sorted:
        base = node
        if node.is_argument():
            pass
        elif node.op.writes_to_input >= 0:
            base = node2memowner[node.parents[node.op.writes_to_input]]
        elif node in after2before:
            base = after2before[node]
        elif enable_inplace_opt and node.op.return_type == "byref" and isinstance(node.op, (core.ElwiseUnary, core.ElwiseBinary)):
            for parent in node.parents:
                parentowner = node2memowner[parent]
                if (len(node2child[parent]) == 1 and node.dtype == parent.dtype and is_tensor(parent)
                        and node2dev[node] == node2dev[parent]
                        and _is_data_mutable(parentowner) and parentowner is parent
                        and parent not in outputs and parent not in const_nodes
                        and _same_shape(node2shape[node], node2shape[parent])):
                    base = parentowner
                    break
        node2memowner[node] = base
    return node2memowner


def _is_data_mutable(node):
    return not node.is_input() and node.op.return_type == "byref"


class MemCounter(object):
    def __init__(self):
        self.count = 0

    def new_memloc(self, devtype):
        out = MemLocation(self.count, devtype)
        self.count += 1
        return out


def _static_shape(shp):
    """tuple of ints when every extent is a compile-time constant, else None"""
    if isinstance(shp, tuple):
        parts = [_static_shape(s) for s in shp]
        return None if any(p is None for p in parts) else tuple(parts)
    out = []
    for s in shp:
        if not isinstance(s.op, core.Constant):
            return None
        out.append(int(s.op.value))
    return tuple(out)


def create_execution_graph(inputs, nodes_sorted, node2shape, node2memowner, node2dev, once_nodes=()):
    """Instruction list (cgt/compilation.py:204-248): Argument -> LoadArgument; byref tensor ->
    Alloc + ReturnByRef; byref tuple -> Alloc per component + BuildTup + ReturnByRef; byval ->
    ReturnByVal; a node that writes into another node's memory re-uses that location."""
    instrs = []
    counter = MemCounter()
    node2memloc = {}
    for node in nodes_sorted:
        if node not in node2dev:
            node2dev[node] = core.Device("cpu", 0)
        devtype = node2dev[node].devtype
        if node.is_argument():
            write_loc = counter.new_memloc(devtype)
            instrs.append(LoadArgument(inputs.index(node), write_loc))
        else:
            read_locs = [node2memloc[parent] for parent in node.parents]
            once = node in once_nodes
            if node.op.return_type == "byref":
                if node2memowner[node] is node:
                    if is_tensor(node):
                        nodeshape = node2shape[node] if node.ndim > 0 else []
                        shape_locs = [node2memloc[shpel] for shpel in nodeshape]
                        write_loc = counter.new_memloc(devtype)
                        instrs.append(Alloc(node.dtype, shape_locs, write_loc))
                    else:
                        nodeshape = node2shape[node]
                        assert isinstance(nodeshape, tuple)
                        arr_locs = []
                        for (arrshp, arrtyp) in utils.safezip(nodeshape, node.typ):
                            arr_loc = counter.new_memloc(devtype)
                            shape_locs = [node2memloc[shpel] for shpel in arrshp]
                            instrs.append(Alloc(arrtyp.dtype, shape_locs, arr_loc))
                            arr_locs.append(arr_loc)
                        write_loc = counter.new_memloc(devtype)
                        instrs.append(BuildTup(node.typ, arr_locs, write_loc))
                else:
                    assert node2dev[node] == node2dev[node2memowner[node]], \
                        "a node that writes into another node's memory must live on the same device"
                    write_loc = node2memloc[node2memowner[node]]
                instrs.append(ReturnByRef(node.op, [par.typ for par in node.parents], read_locs, write_loc,
                                          node_props=node.props, once=once))
            else:
                assert node.op.return_type == "byval"
                write_loc = counter.new_memloc(devtype)
                instrs.append(ReturnByVal(node.op, [par.typ for par in node.parents], read_locs, write_loc,
                                          node_props=node.props, once=once))
            # static shapes and dtypes, for profiling reports (algorithmic bytes per instruction)
            instrs[-1].in_shapes = [_static_shape(node2shape[p]) if p in node2shape else None for p in node.parents]
            instrs[-1].in_dtypes = [p.dtype for p in node.parents]
            instrs[-1].out_shape = _static_shape(node2shape[node]) if node in node2shape else None
            instrs[-1].out_dtype = node.dtype
            instrs[-1].out_dtypes = [t.dtype for t in node.typ] if is_tuple(node) else None
        node2memloc[node] = write_loc
    return ExecutionGraph(instrs, len(inputs), counter.count), node2memloc


def merge_parameter_updates(eg, update_locs):
    """Instruction-list pass: the update instructions of a step that run one and the same single-output FusedElwise
    program on float32 tensors / scalars (SGD: p - lr * g for every parameter) become ONE MultiFusedElwise instruction
    at the position of the last of them. `update_locs`: indices of the memory locations that updates write (the
    variables' own storage). An update is moved only if no instruction between its old and its new position touches its
    result location, so every reader still sees the value it saw before."""
    instrs = eg.instrs
    groups = defaultdict(list)
    for (i, ins) in enumerate(instrs):
        if not isinstance(ins, ReturnByRef) or not isinstance(ins.op, core.FusedElwise) or ins.once:
            continue
        op = ins.op
        if len(op.out_regs) != 1 or op.out_dtypes != ["f4"] or len(op.in_kinds) > 4 or any(k not in (0, 2, 3) for k in op.in_kinds):
            continue
        if ins.write_loc.index not in update_locs or ins.write_loc.devtype != "gpu":
            continue
        key = (tuple(op.program), tuple(op.in_kinds), tuple(op.out_regs))
        groups[key].append(i)
    # groups whose last member comes latest first: once the chains that READ a state variable's new value (the
    # parameter's own update) have moved to the end, the chains that write it can move past their old readers
    for (key, idxs) in sorted(groups.items(), key=lambda kv: -kv[1][-1]):
        last = idxs[-1]
        movable = []
        for i in idxs:
            w = instrs[i].write_loc.index
            ok = True
            for j in range(i + 1, last + 1):
                other = instrs[j]
                if j in idxs:
                    if any(r.index == w for r in other.read_locs if j != i) and w != other.write_loc.index:
                        ok = False
                    continue
                locs = [r.index for r in getattr(other, "read_locs", [])] + [other.write_loc.index]
                if w in locs:
                    ok = False
                    break
            if ok:
                movable.append(i)
        movable = movable[:24]
        if len(movable) < 2:
            continue
        first = instrs[movable[0]]
        reads, types, in_shapes, in_dtypes = [], [], [], []
        for i in movable:
            reads += list(instrs[i].read_locs)
            types += list(instrs[i].input_types)
            in_shapes += list(instrs[i].in_shapes)
            in_dtypes += list(instrs[i].in_dtypes)
        extra = [instrs[i].write_loc for i in movable[1:]]
        merged = ReturnByRef(core.MultiFusedElwise(first.op, len(movable)), types + [None] * len(extra), reads + extra, first.write_loc,
                             node_props=first.node_props)
        merged.in_shapes, merged.in_dtypes = in_shapes, in_dtypes
        merged.out_shape, merged.out_dtype, merged.out_dtypes = None, "f4", None
        merged.extra_out_shapes = [instrs[i].out_shape for i in movable]
        pos = movable[-1]
        drop = set(movable)
        new_instrs = []
        for (j, ins) in enumerate(instrs):
            if j == pos:
                new_instrs.append(merged)
            elif j not in drop:
                new_instrs.append(ins)
        instrs = new_instrs
        eg.instrs = instrs
        # indices changed: recompute the remaining groups on the new list
        return merge_parameter_updates(eg, update_locs)
    return eg


def apply_graph_rewrites(outputs_simple, updatetargs_simple, node2shape):
    """The graph rewrites that run after simplification and differentiation, in their fixed order, each under its
    configuration switch. Returns the new (outputs, update targets)."""
    config = core.get_config()
    if config["fuse_conv_dgrad"]:
        outputs_simple, updatetargs_simple = fuse_conv_dgrad(outputs_simple, updatetargs_simple, node2shape)
    if config["fuse_conv_grad_input"]:
        outputs_simple, updatetargs_simple = fuse_conv_grad_input(outputs_simple, updatetargs_simple, node2shape)
    if config["fuse_slice_views"]:
        outputs_simple, updatetargs_simple = view_leading_slices(outputs_simple, updatetargs_simple, node2shape)
    if config["fuse_slice_sums"]:
        outputs_simple, updatetargs_simple = fuse_slice_sums(outputs_simple, updatetargs_simple, node2shape)
    if config["fuse_slice_sums"] and config["split_gate_columns"]:
        outputs_simple, updatetargs_simple = split_gate_columns(outputs_simple, updatetargs_simple, node2shape)
    if config["batch_summed_products"]:
        outputs_simple, updatetargs_simple = batch_summed_products(outputs_simple, updatetargs_simple, node2shape)
        outputs_simple, updatetargs_simple = batch_shared_weight_products(outputs_simple, updatetargs_simple, node2shape)
        outputs_simple, updatetargs_simple = batch_scalar_sums(outputs_simple, updatetargs_simple, node2shape)
    if config["fuse_product_sums"]:    # after the batching: the products over all time steps are views by now
        outputs_simple, updatetargs_simple = fuse_product_sums(outputs_simple, updatetargs_simple, node2shape)
    if config["fuse_elementwise"]:
        if config["fuse_rows"] and config["fuse_flat_index_rows"]:
            outputs_simple, updatetargs_simple = fuse_flat_index_rows(outputs_simple, updatetargs_simple, node2shape)
        if config["fuse_rows"]:
            outputs_simple, updatetargs_simple = fuse_elementwise(outputs_simple, updatetargs_simple, node2shape, rows=True)
        outputs_simple, updatetargs_simple = fuse_elementwise(outputs_simple, updatetargs_simple, node2shape)
        if config["fuse_conv_output"]:
            outputs_simple, updatetargs_simple = fuse_conv_output(outputs_simple, updatetargs_simple, node2shape)
        if config["fuse_conv_output"] and config["fuse_conv_implicit"]:
            outputs_simple, updatetargs_simple = fuse_conv_implicit(outputs_simple, updatetargs_simple, node2shape)
        if config["fuse_conv_output"] and config["fuse_conv_direct"]:
            outputs_simple, updatetargs_simple = fuse_conv_direct(outputs_simple, updatetargs_simple, node2shape)
        if config["pad_conv_columns"]:
            outputs_simple, updatetargs_simple = pad_conv_columns(outputs_simple, updatetargs_simple, node2shape)
    if config["hoist_filter_splits"]:
        outputs_simple, updatetargs_simple = hoist_filter_splits(outputs_simple, updatetargs_simple, node2shape)
    return outputs_simple, updatetargs_simple


def run_compilation_pipeline(inputs, outputs, updates, givens):
    config = core.get_config()
    outputs_simple, updatesrcs, updatetargs_simple, analysis = simplify_for_execution(outputs, updates, givens)
    node2shape = analysis["node2shape"]
    outputs_simple, updatetargs_simple = apply_graph_rewrites(outputs_simple, updatetargs_simple, node2shape)
    all_out = outputs_simple + updatetargs_simple

    nodelist = core.topsorted(all_out)
    node2dev = determine_devices(nodelist, dict(zip(updatetargs_simple, updatesrcs)))
    add_transports(nodelist, node2dev, node2shape)

    updates_simple = list(zip(updatesrcs, updatetargs_simple))
    extra = _update_control_deps(all_out, updates_simple)
    first, last = _transport_schedule(all_out, updatetargs_simple, node2dev)
    for node in last:
        extra[node] = extra.get(node, []) + [t for t in updatetargs_simple if t is not node]
    nodes_sorted = topsorted_shapes_first(first + all_out, node2shape, extra)
    const_nodes = compute_const_nodes(nodes_sorted)
    node2memowner = determine_memowner(nodes_sorted, updates_simple, node2dev, outputs_simple, node2shape, const_nodes)
    written_into = set(owner for (n, owner) in node2memowner.items() if owner is not n)
    once_nodes = set(n for n in const_nodes if n not in written_into)
    eg, node2memloc = create_execution_graph(inputs, nodes_sorted, node2shape, node2memowner, node2dev, once_nodes)
    if config["merge_parameter_updates"] and updates_simple:
        merge_parameter_updates(eg, set(node2memloc[t].index for t in updatetargs_simple))

    if config["verbose"]:
        sys.stderr.write("begin\n" + "\n".join("%i.) \t%r" % (i, instr) for (i, instr) in enumerate(eg.instrs)) + "\nend\n")
    return create_interpreter(inputs, outputs_simple, eg, node2memloc)


def create_interpreter(inputs, outputs, eg, node2memloc):
    from . import runtime
    config = core.get_config()
    if config["backend"] != "native":
        raise NotImplementedError("this package only has the native GPU interpreter (backend=native)")
    input_types = [inp.typ for inp in inputs]
    output_locs = [node2memloc[node] for node in outputs]
    flags = 0
    if config["use_cuda_graphs"]:
        flags |= runtime.INTERP_CUDA_GRAPHS
    if config["profile"] or profiler.on:
        flags |= runtime.INTERP_PROFILE
    interp = runtime.InterpreterWrapper(eg, input_types, output_locs, flags)
    interp.eg = eg
    if flags & runtime.INTERP_PROFILE:
        profiler.register(interp)
    return interp


# ================================================================
# numeric_eval: evaluate without building a function object
# ================================================================

def numeric_eval(output, arg2val):
    """Evaluate `output` (Node or list) given values for its arguments. Compiles a throw-away function."""
    single = isinstance(output, core.Node)
    outs = [output] if single else list(output)
    args = list(arg2val.keys())
    f = function(args, outs)
    vals = f(*[arg2val[a] for a in args])
    return vals[0] if single else vals


# ================================================================
# Execution graph and instructions (cgt/compilation.py:425-517)
# ================================================================

class ExecutionGraph(object):
    def __init__(self, instrs, n_args, n_locs):
        self.instrs = instrs
        self.n_args = n_args
        self.n_locs = n_locs


class MemLocation(object):
    def __init__(self, idx, devtype):
        assert isinstance(idx, int) and devtype in ["cpu", "gpu"]
        self.index = idx
        self.devtype = devtype

    def __repr__(self):
        return "%%%i/%s" % (self.index, self.devtype)


class Instr(object):
    pass


class LoadArgument(Instr):
    def __init__(self, ind, write_loc):
        self.ind = ind
        self.write_loc = write_loc

    def __repr__(self):
        return "%s = LoadArg ind:%i" % (self.write_loc, self.ind)


class Alloc(Instr):
    def __init__(self, dtype, read_locs, write_loc):
        self.dtype = dtype
        self.read_locs = read_locs
        self.write_loc = write_loc

    def __repr__(self):
        return "%s = Alloc shp:%s dtype:%s" % (self.write_loc, str(self.read_locs), self.dtype)


class BuildTup(Instr):
    def __init__(self, typ, read_locs, write_loc):
        self.typ = typ
        self.read_locs = read_locs
        self.write_loc = write_loc

    def __repr__(self):
        return "%s = BuildTup args:%s" % (self.write_loc, str(self.read_locs))


class _Return(Instr):
    kindname = "Return"

    def __init__(self, op, input_types, read_locs, write_loc, node_props=None, once=False):
        self.op = op
        self.input_types = input_types
        self.read_locs = read_locs
        self.write_loc = write_loc
        self.node_props = node_props
        self.once = once
        self._callable = None

    def get_callable(self):
        if self._callable is None:
            self._callable = get_callable(self.op, self.input_types, self.write_loc.devtype)
        return self._callable

    def __repr__(self):
        return "%s = %s op:%s args:%s" % (self.write_loc, self.kindname, str(self.op), str(self.read_locs))


class ReturnByRef(_Return):
    kindname = "ReturnByRef"


class ReturnByVal(_Return):
    kindname = "ReturnByVal"


_QUICK_OPS = (core.Size, core.Reshape, core.LeadingSlice, core.MakeTuple, core.TupleIndex, core.GetData)


def instr_flags(instr):
    """Interpreter flags of a Return instruction (quick: host bookkeeping only, cf. cycgt.pyx:356-358)."""
    from . import runtime
    flags = 0
    if isinstance(instr.op, _QUICK_OPS):
        flags |= runtime.INSTR_QUICK
    if isinstance(instr.op, core.Transport):
        flags |= runtime.INSTR_TRANSPORT
    if getattr(instr, "once", False):
        flags |= runtime.INSTR_ONCE
    return flags


# ================================================================
# Callables
# ================================================================

def get_callable(op, input_types, devtype, prefer_python=False):
    """Native callable when the Op has one for `devtype`, else its Python function (run through a
    host trampoline; only valid for host-resident values)."""
    assert op.available_impls, "need to set op.available_impls"
    config = core.get_config()
    if (prefer_python or config["force_python_impl"]) and "python" in op.available_impls:
        return op.get_py_callable(input_types)
    if "native_" + devtype in op.available_impls or (devtype == "cpu" and "native_gpu" in op.available_impls and _prebuilt(op, input_types)):
        return get_native_callable(op, input_types, devtype)
    if "python" in op.available_impls:
        if devtype == "gpu":
            raise RuntimeError("Tried to put Op %s on the GPU but I only have a python impl :(" % op)
        return op.get_py_callable(input_types)
    raise RuntimeError("Can't find an implementation of %s for devtype %s. available_impls=%s" % (op, devtype, op.available_impls))


def _prebuilt(op, input_types):
    try:
        return op.get_native_compile_info(input_types, "cpu").prebuilt is not None
    except Exception:
        return False


def get_native_callable(op, input_types, devtype):
    nci = op.get_native_compile_info(input_types, devtype)
    nci.op_str = str(op)
    nci.return_type = op.return_type
    nci.n_in = len(input_types)
    return nci2callable(nci)


CPP_ABI_VERSION = 1  # bump when include/cgt_common.h changes layout, to invalidate cached libraries


def nci2callable(nci):
    from . import runtime
    cldata = _build_closure(nci.closure_triples)
    if nci.prebuilt is not None:
        L = runtime.lib()
        try:
            fptr = getattr(L, nci.prebuilt)
        except AttributeError:
            raise runtime.BackendError("libcgt_b200.so does not export %s" % nci.prebuilt)
        return core.NativeCallable(nci.n_in, nci.return_type, nci.op_str, fptr, cldata=cldata,
                                   store_objects=nci.store_objects, flags=nci.flags)
    template_code = gen_templated_code(nci.includes, nci.closure_triples, nci.func_code)
    compile_info = get_compile_info()
    prefix = utils.hash_seq1(template_code, compile_info["CPP_FLAGS"], str(CPP_ABI_VERSION), *(src.code for src in nci.extra_srcs))
    d = dict(function=_funcname(prefix), closure=_closurename(prefix), setup=_setupname(prefix), teardown=_teardownname(prefix))
    srcfiles = [core.SrcFile("c++", string.Template(template_code).substitute(d))]
    srcfiles.extend(core.SrcFile(sf.lang, string.Template(sf.code).substitute(d)) for sf in nci.extra_srcs)
    libpath = osp.join(compile_info["CACHE_ROOT"], prefix + ".so")
    if not osp.exists(libpath):
        TranslationUnit(srcfiles, nci.link_flags).compile(prefix, libpath)
    lib = get_or_load_lib(libpath)
    fptr = getattr(lib, _funcname(prefix))
    setup_fptr = getattr(lib, _setupname(prefix)) if nci.setup else None
    teardown_fptr = getattr(lib, _teardownname(prefix)) if nci.teardown else None
    return core.NativeCallable(nci.n_in, nci.return_type, nci.op_str, fptr, cldata=cldata, setup_fptr=setup_fptr,
                               teardown_fptr=teardown_fptr, store_objects=nci.store_objects, flags=nci.flags)


def _funcname(prefix):
    return "call_" + prefix


def _setupname(prefix):
    return "setup_" + prefix


def _teardownname(prefix):
    return "teardown_" + prefix


def _closurename(prefix):
    return "closure_" + prefix


def gen_templated_code(includes, closure_info, func_code):
    s = StringIO()
    for fname in ["cgt_common.h"] + list(includes):
        s.write('#include "%s"\n' % fname)
    gen_struct_code(closure_info, s)
    s.write(func_code)
    return s.getvalue()


def gen_struct_code(triples, outstream):
    if triples is None:
        return
    outstream.write("typedef struct $closure {\n")
    for (fieldname, fieldtype, _val) in triples:
        outstream.write("%s %s;\n" % (_ctypes2str[fieldtype], fieldname))
    outstream.write("} $closure;\n")


_LIBRARIES = {}


def get_or_load_lib(libname):
    if libname not in _LIBRARIES:
        _LIBRARIES[libname] = ctypes.cdll.LoadLibrary(libname)
    return _LIBRARIES[libname]


class TranslationUnit(object):
    """Sources of one native Op: compiled with c++ (lang "c++") or nvcc for sm_100a (lang "cuda"),
    linked against libcgt_b200.so into <cache>/<hash>.so."""

    def __init__(self, srcfiles, link_flags):
        self.srcfiles = srcfiles
        self.link_flags = link_flags

    def compile(self, prefix, libpath):
        info = get_compile_info()
        cache = info["CACHE_ROOT"]
        objs = []
        for (i, (lang, code)) in enumerate(self.srcfiles):
            if lang == "c++":
                srcpath = osp.join(cache, prefix + "_%i.cpp" % i)
                cmd = "c++ %s %s -c -o %s.o %s" % (info["CPP_FLAGS"], srcpath, srcpath, info["INCLUDES"])
            elif lang == "cuda":
                srcpath = osp.join(cache, prefix + "_%i.cu" % i)
                from .build import _nvcc
                cmd = ("%s %s -c -o %s.o -gencode arch=compute_100a,code=sm_100a -lineinfo -O3 -std=c++17 "
                       "-Xcompiler -fPIC %s" % (_nvcc(), srcpath, srcpath, info["INCLUDES"]))
            else:
                raise NotImplementedError(lang)
            with open(srcpath, "w") as fh:
                fh.write(code)
            _call(cmd)
            objs.append(srcpath + ".o")
        _call("c++ %s %s %s %s -o %s" % (info["CPP_FLAGS"], " ".join(objs), info["LINK_FLAGS"], self.link_flags, libpath))


def _call(cmd):
    if core.get_config()["verbose"]:
        sys.stderr.write("\x1b[32m%s\x1b[0m\n" % cmd)
    p = subprocess.run(cmd, shell=True, capture_output=True, text=True)
    if p.returncode != 0:
        raise RuntimeError("native compilation failed:\n%s\n%s" % (cmd, p.stdout + p.stderr))


_COMPILE_CONFIG = None


def get_compile_info():
    global _COMPILE_CONFIG
    if _COMPILE_CONFIG is None:
        from . import runtime
        config = core.get_config()
        cache = osp.join(runtime.HERE, "_cache") if config["cache_dir"].startswith("~") else osp.expanduser(config["cache_dir"])
        os.makedirs(cache, exist_ok=True)
        includes = "-I%s -I/usr/local/cuda/include" % runtime.INCLUDE_DIR
        link_flags = "-shared -rdynamic -L%s -l:libcgt_b200.so -Wl,-rpath,%s -L/usr/local/cuda/lib64 -lcudart" % (runtime.HERE, runtime.HERE)
        cpp_flags = "-fvisibility=hidden -std=c++17 -fPIC" + (" -O0 -g" if config["debug_cpp"] else " -O3 -DNDEBUG")
        _COMPILE_CONFIG = dict(CACHE_ROOT=cache, INCLUDES=includes, LINK_FLAGS=link_flags, CPP_FLAGS=cpp_flags,
                               CGT_INCLUDE_DIR=runtime.INCLUDE_DIR, CGT_ENABLE_CUDA=True, CGT_ENABLE_CUDNN=False)
    return _COMPILE_CONFIG


_ctypes2str = {
    ctypes.c_byte: "uint8_t", ctypes.c_bool: "bool", ctypes.c_char: "char", ctypes.c_int: "int",
    ctypes.c_long: "long", ctypes.c_void_p: "void*", ctypes.c_double: "double", ctypes.c_float: "float",
}

_struct_cache = {}


def _build_closure(triples):
    if triples is None:
        return ctypes.c_void_p(0)
    fields = [(name, typ) for (name, typ, _val) in triples]
    key = tuple((name, typ.__name__) for (name, typ) in fields)
    S = _struct_cache.get(key)
    if S is None:
        S = type("closure", (ctypes.Structure,), {"_fields_": fields})
        _struct_cache[key] = S
    return S(*[val for (_n, _t, val) in triples])


# ================================================================
# Profiler: per-instruction CUDA-event timing in the native interpreter, aggregated per Op
# (the reference's profiler only works with its Python interpreter, cgt/compilation.py:821-858)
# ================================================================

class _Profiler(object):
    def __init__(self):
        self.on = False
        self.interps = []

    def start(self):
        self.on = True

    def stop(self):
        self.on = False

    def register(self, interp):
        self.interps.append(interp)

    def clear_stats(self):
        self.interps = []

    def op_stats(self):
        """{op string: (count, total ms)} over every profiled function"""
        out = {}
        for interp in self.interps:
            for (instr, (r, ms, count)) in zip(interp.eg.instrs, interp.profile()):
                if count == 0:
                    continue
                key = str(instr.op) if isinstance(instr, _Return) else type(instr).__name__
                c0, t0 = out.get(key, (0, 0.0))
                out[key] = (c0 + count, t0 + ms)
        return out

    def print_stats(self):
        stats = self.op_stats()
        total = sum(t for (_c, t) in stats.values()) or 1.0
        rows = sorted(stats.items(), key=lambda kv: -kv[1][1])
        sys.stdout.write("Total device time in profiled instructions: %.3f ms\n" % total)
        sys.stdout.write("%-50s %8s %12s %8s\n" % ("Op", "Count", "Time (ms)", "Frac"))
        for (k, (c, t)) in rows:
            sys.stdout.write("%-50s %8d %12.4f %8.3f\n" % (k[:50], c, t, t / total))


profiler = _Profiler()
