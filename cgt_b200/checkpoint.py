"""Checkpoint / resume of a training job's state: every ``shared`` variable a set of update expressions
touches (parameters, optimizer slots, step counters) goes to one ``.npz`` file and comes back with ``set_value``.

The reference has no checkpoint format; what it offers is ``InMemoryData.get_value`` / ``set_value``
(cgt/core.py:569-582) and the flat-vector helpers of ``ParamCollection`` (examples/param_collection.py:37-56).
This module is the file format on top of those two calls. Restoring writes into the variables' existing device
buffers (``set_value`` keeps the address when the shape is unchanged), so compiled functions and their captured
CUDA graphs stay valid across a ``load_state``.
"""
import json

import numpy as np

from . import core

FORMAT_VERSION = 1


def state_variables(updates=(), outputs=(), params=()):
    """All ``shared`` variables of a training step, in a deterministic order: `params` first (as given), then every
    Data node that is the target of an update, then every Data node the update expressions and `outputs` read."""
    seen, order = set(), []

    def add(node):
        if node not in seen and node.is_data():
            seen.add(node)
            order.append(node)

    for p in params:
        add(p)
    roots = list(outputs)
    for (before, after) in updates:
        add(before)
        roots.append(after)
    for node in core.topsorted(roots):
        add(node)
    return order


def save_state(path, variables, extra=None):
    """Write the values of `variables` (a list of ``shared`` nodes) and the JSON-serialisable dict `extra`
    (step counter, RNG seed, learning rate ...) to `path` (``.npz``). Device values are copied to the host first."""
    arrays, meta = {}, []
    for (i, v) in enumerate(variables):
        assert v.is_data(), "save_state takes shared variables"
        val = np.asarray(v.op.get_value())
        key = "v%05d" % i
        arrays[key] = val
        meta.append({"key": key, "name": getattr(v, "name", None), "shape": list(val.shape), "dtype": val.dtype.str})
    header = {"format": FORMAT_VERSION, "variables": meta, "extra": extra or {}}
    arrays["__header__"] = np.frombuffer(json.dumps(header).encode("utf-8"), dtype=np.uint8)
    with open(path, "wb") as fh:
        np.savez(fh, **arrays)


def load_state(path, variables):
    """Restore `variables` (same list, same order as at ``save_state``) from `path`; returns the saved `extra` dict.
    Shapes and dtypes must match: a mismatch raises before any variable is touched."""
    with np.load(path, allow_pickle=False) as z:
        header = json.loads(bytes(z["__header__"].tobytes()).decode("utf-8"))
        if header.get("format") != FORMAT_VERSION:
            raise ValueError("unknown checkpoint format %r" % header.get("format"))
        meta = header["variables"]
        if len(meta) != len(variables):
            raise ValueError("checkpoint holds %d variables, %d were given" % (len(meta), len(variables)))
        vals = []
        for (m, v) in zip(meta, variables):
            val = z[m["key"]]
            if tuple(val.shape) != tuple(v.op.get_shape()) or np.dtype(m["dtype"]) != np.dtype(v.dtype):
                raise ValueError("checkpoint variable %s %s %s does not match %s %s" % (
                    m["name"], m["shape"], m["dtype"], tuple(v.op.get_shape()), v.dtype))
            vals.append(val)
    for (v, val) in zip(variables, vals):
        v.op.set_value(val)
    return header["extra"]


class ParamCollection(object):
    """Flat-vector view of a list of float parameters (the helper of examples/param_collection.py:4-56)."""

    def __init__(self, params):
        assert all(p.is_data() and p.dtype == core.cgt.floatX for p in params)
        self._params = list(params)

    @property
    def params(self):
        return self._params

    def get_values(self):
        return [p.op.get_value() for p in self._params]

    def get_shapes(self):
        return [tuple(p.op.get_shape()) for p in self._params]

    def get_total_size(self):
        return int(sum(int(np.prod(s)) for s in self.get_shapes()))

    def num_vars(self):
        return len(self._params)

    def set_values(self, parvals):
        assert len(parvals) == len(self._params)
        for (p, v) in zip(self._params, parvals):
            p.op.set_value(v)

    def set_value_flat(self, theta):
        theta = np.asarray(theta).astype(core.cgt.floatX)
        assert theta.ndim == 1 and theta.size == self.get_total_size()
        vals, n = [], 0
        for s in self.get_shapes():
            k = int(np.prod(s))
            vals.append(theta[n:n + k].reshape(s))
            n += k
        self.set_values(vals)

    def get_value_flat(self):
        if not self._params:
            return np.zeros((0,), core.cgt.floatX)
        return np.concatenate([np.asarray(v).reshape(-1) for v in self.get_values()]).astype(core.cgt.floatX)
