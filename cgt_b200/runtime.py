"""ctypes binding of ``libcgt_b200.so`` (declared in ``include/cgt_b200.h``).

Plays the role of the reference's Cython bridge ``src/cycgt.pyx``: numpy <-> cgtArray conversion,
the persistent array behind ``cgt.shared`` (CppArrayWrapper there, ArrayWrapper here) and the
interpreter wrapper. There is no Python or CPU execution path behind these calls: if the library is
missing, or no B200 is present when device work is requested, they raise.
"""
import ctypes
import os
import os.path as osp

import numpy as np

HERE = osp.dirname(osp.abspath(__file__))
LIB_PATH = osp.join(HERE, "libcgt_b200.so")
INCLUDE_DIR = osp.normpath(osp.join(HERE, "..", "include"))

CPU, GPU = 0, 1
INSTR_QUICK, INSTR_TRANSPORT, INSTR_NOCAPTURE, INSTR_ONCE = 1, 2, 4, 8
INTERP_CUDA_GRAPHS, INTERP_PROFILE = 1, 2

DTYPE_NUM = {"i1": 1, "i2": 3, "i4": 5, "i8": 7, "f4": 11, "f8": 12}
NUM_DTYPE = {v: k for (k, v) in DTYPE_NUM.items()}

c_long_p = ctypes.POINTER(ctypes.c_long)
c_int_p = ctypes.POINTER(ctypes.c_int)


class BackendError(RuntimeError):
    pass


_lib = None


def _declare(lib):
    vp, ci, cl, cd = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_double
    sig = {
        "cgtb_init": (ci, [ci]), "cgtb_initialized": (ci, []), "cgtb_device": (ci, []),
        "cgtb_last_error": (ctypes.c_char_p, []), "cgtb_clear_error": (None, []), "cgtb_synchronize": (ci, []),
        "cgtb_stream": (vp, []), "cgtb_pool_stats": (ci, [c_long_p] * 4), "cgtb_pool_trim": (ci, []),
        "cgtb_kernel_launches": (cl, []), "cgtb_sm_count": (ci, []),
        "cgtb_event_new": (vp, []), "cgtb_event_record": (ci, [vp]),
        "cgtb_event_elapsed_ms": (ci, [vp, vp, ctypes.POINTER(ctypes.c_float)]), "cgtb_event_free": (None, [vp]),
        "cgtb_l2_flush": (ci, []), "cgtb_selftest_refused_launch": (ci, []),
        "cgtb_prefetch_h2d": (ci, [vp, vp, cl]),
        "cgtb_prefetch_begin": (ci, [ci]), "cgtb_prefetch_mark": (ci, [ci]), "cgtb_prefetch_join": (ci, [ci]),
        "cgtb_prefetch_release": (ci, [ci]),
        "cgtb_comm_load": (ci, [ctypes.c_char_p]), "cgtb_comm_unique_id": (ci, [ctypes.c_char_p]),
        "cgtb_comm_init": (ci, [ctypes.c_char_p, ci, ci]), "cgtb_comm_world": (ci, []), "cgtb_comm_rank": (ci, []),
        "cgtb_comm_check": (ci, []), "cgtb_comm_abort": (ci, []), "cgtb_comm_destroy": (ci, []),
        "cgtb_allreduce_sum": (ci, [ci, ci, ctypes.POINTER(vp), ctypes.POINTER(vp), c_long_p]),
        "cgtb_peer_alloc": (ci, [cl, ctypes.c_char_p]), "cgtb_peer_open": (ci, [ctypes.c_char_p, ci, ci]),
        "cgtb_peer_close": (ci, []), "cgtb_peer_world": (ci, []), "cgtb_peer_slot_bytes": (cl, []),
        "cgtb_peer_set_wait_cycles": (ci, [cl]), "cgtb_peer_timing": (ci, [c_long_p]), "cgtb_peer_set_two_phase_bytes": (ci, [cl]),
        "cgtb_peer_allreduce_sum": (ci, [ci, ctypes.POINTER(vp), ctypes.POINTER(vp), c_long_p]),
        "cgtb_peer_selftest_open": (ci, [cl]), "cgtb_peer_selftest_post": (ci, [vp, cl]),
        "cgtb_alloc": (vp, [ci, cl]), "cgtb_free": (None, [ci, vp]), "cgtb_memcpy": (ci, [ci, ci, vp, vp, cl, ci]),
        "cgtb_memset": (ci, [vp, ci, cl]),
        "cgtb_array_new": (vp, [ci, c_long_p, ci, ci]), "cgtb_array_from_host": (vp, [ci, c_long_p, ci, ci, vp, ci]),
        "cgtb_array_view_device": (vp, [ci, c_long_p, ci, vp]),
        "cgtb_array_to_host": (ci, [vp, vp]), "cgtb_array_set_from_host": (ci, [vp, vp]),
        "cgtb_array_ndim": (ci, [vp]), "cgtb_array_shape": (c_long_p, [vp]), "cgtb_array_dtype": (ci, [vp]),
        "cgtb_array_devtype": (ci, [vp]), "cgtb_array_data": (vp, [vp]), "cgtb_array_nbytes": (cl, [vp]),
        "cgtb_tuple_new": (vp, [ci]), "cgtb_tuple_len": (ci, [vp]), "cgtb_tuple_get": (vp, [vp, ci]),
        "cgtb_tuple_set": (ci, [vp, ci, vp]), "cgtb_object_kind": (ci, [vp]), "cgtb_retain": (None, [vp]),
        "cgtb_release": (None, [vp]),
        "cgtb_graph_new": (vp, [cl, cl]), "cgtb_graph_free": (None, [vp]),
        "cgtb_graph_add_load_argument": (ci, [vp, ctypes.c_char_p, ci, cl, ci]),
        "cgtb_graph_add_alloc": (ci, [vp, ctypes.c_char_p, ci, ci, c_long_p, cl, ci]),
        "cgtb_graph_add_build_tup": (ci, [vp, ctypes.c_char_p, ci, c_long_p, cl, ci]),
        "cgtb_graph_add_return_byref": (ci, [vp, ctypes.c_char_p, ci, c_long_p, c_int_p, cl, ci, vp, vp, ci]),
        "cgtb_graph_add_return_byval": (ci, [vp, ctypes.c_char_p, ci, c_long_p, c_int_p, cl, ci, vp, vp, ci]),
        "cgtb_interp_new": (vp, [vp, ci, c_long_p, ci]), "cgtb_interp_free": (None, [vp]),
        "cgtb_interp_set_before_sync": (ci, [vp, vp, vp]),
        "cgtb_interp_run": (ci, [vp, vp, ctypes.POINTER(vp)]), "cgtb_interp_stats": (ci, [vp, c_long_p, ci]), "cgtb_state_version_bump": (None, []),
        "cgtb_interp_profile": (ci, [vp, ctypes.POINTER(cd), c_long_p, ci]),
        "cgtb_interp_instr_repr": (ctypes.c_char_p, [vp, ci]),
        "cgtb_apply_byref": (ci, [vp, vp, ci, ctypes.POINTER(vp), vp]),
        "cgtb_sgemm": (ci, [ci, ci, cl, cl, cl, vp, cl, vp, cl, vp, cl, ci]),
        "cgtb_sgemm_batched": (ci, [ci, ci, cl, cl, cl, cl, vp, cl, cl, vp, cl, cl, vp, cl, cl, ci]),
        "cgtb_sgemm_bias_add": (ci, [ci, ci, cl, cl, cl, vp, cl, vp, cl, vp, vp, cl, vp, vp, cl]),
        "cgtb_dgemm": (ci, [ci, ci, cl, cl, cl, vp, cl, vp, cl, vp, cl]),
        "cgtb_im2col": (ci, [ci, vp, cl] + [ci] * 9 + [vp]), "cgtb_col2im": (ci, [ci, vp, cl] + [ci] * 9 + [vp]),
        "cgtb_max_pool": (ci, [ci, vp, cl] + [ci] * 11 + [vp, vp]),
        "cgtb_max_pool_pullback": (ci, [ci, vp, vp, cl] + [ci] * 11 + [vp]),
        "cgtb_lrn_forward": (ci, [ci, vp, cl, ci, ci, ci, ci, cd, cd, vp, vp]),
        "cgtb_lrn_backward": (ci, [ci, vp, vp, vp, vp, cl, ci, ci, ci, ci, cd, cd, vp]),
        "cgtb_conv_dgrad": (ci, [vp, cl, ci, ci, ci, vp] + [ci] * 7 + [vp]),
        "cgtb_conv_fwd_bias_relu": (ci, [vp, cl, ci, ci, ci, vp] + [ci] * 7 + [vp, vp, vp]),
        "cgtb_conv_wgrad": (ci, [vp, cl, ci, ci, ci, vp] + [ci] * 7 + [vp]),
        "cgtb_conv_dgrad_bank": (ci, [vp, cl, ci, ci, ci, vp] + [ci] * 7 + [vp]),
        "cgtb_conv_fwd_bias_relu_bank": (ci, [vp, cl, ci, ci, ci, vp] + [ci] * 7 + [vp, vp, vp]),
        "cgtb_conv_fwd_bias_relu_pre": (ci, [vp, cl, ci, ci, ci, vp, vp] + [ci] * 7 + [vp, vp, vp]),
        "cgtb_conv_dgrad_pre": (ci, [vp, cl, ci, ci, ci, vp, vp] + [ci] * 7 + [vp]),
        "cgtb_split_filter_banks": (ci, [ci, ctypes.POINTER(vp), c_int_p, c_int_p, c_int_p, c_int_p, ctypes.POINTER(vp)]),
        "cgtb_conv_bias_relu": (ci, [vp, cl, cl, vp, ci, vp, cl, vp, vp]),
        "cgtb_conv_bias_relu_ld": (ci, [vp, cl, cl, cl, vp, ci, vp, cl, vp, vp]),
        "cgtb_relu_grad_nhwc": (ci, [vp, vp, cl, ci, cl, vp, vp]),
        "cgtb_im2col_ld": (ci, [ci, vp, cl] + [ci] * 9 + [cl, vp]),
        "cgtb_unary": (ci, [ci, ci, ci, cl, vp, vp]), "cgtb_binary": (ci, [ci, ci, ci, ci, cl, vp, vp, vp, ci, ci]),
        "cgtb_reduce": (ci, [ci, ci, ci, c_long_p, c_int_p, vp, vp]),
        "cgtb_repeat": (ci, [ci, ci, c_long_p, c_int_p, vp, vp]),
        "cgtb_transpose": (ci, [ci, ci, c_long_p, c_int_p, vp, vp]),
        "cgtb_getsli": (ci, [ci, cl, cl, cl, cl, cl, cl, vp, vp]),
        "cgtb_incsli": (ci, [ci, cl, cl, cl, cl, cl, cl, vp, vp, vp]),
        "cgtb_getflat": (ci, [ci, cl, vp, vp, vp]), "cgtb_incflat": (ci, [ci, cl, cl, vp, vp, vp, vp]),
        "cgtb_concat_part": (ci, [ci, cl, cl, cl, cl, cl, vp, vp]), "cgtb_fill": (ci, [ci, cl, cd, cl, vp]),
        "cgtb_fused_elwise": (ci, [vp, cl, vp, c_long_p, c_long_p, vp]),
        "cgtb_fused_elwise_multi": (ci, [vp, ci, c_long_p, vp, vp]),
        "cgtb_fused_rows": (ci, [vp, cl, cl, vp, vp]),
        "cgtb_onehot_rows": (ci, [vp, cl, cl, vp]),
        "cgtb_masked_row_sum": (ci, [vp, vp, cl, cl, vp]),
        "cgtb_scatter_cols": (ci, [cl, cl, ci, c_long_p, c_long_p, vp, vp]),
        "cgtb_concat_rows": (ci, [ci, vp, c_long_p, vp]),
        "cgtb_conv_direct_fwd_bias_relu": (ci, [vp, cl, ci, ci, ci, vp, ci, ci, ci, ci, ci, vp, vp, vp]),
        "cgtb_conv_direct_wgrad": (ci, [vp, cl, ci, ci, ci, vp, ci, ci, ci, ci, ci, vp]),
        "cgtb_conv_direct_wgrad_relu": (ci, [vp, cl, ci, ci, ci, vp, vp, ci, ci, ci, ci, ci, vp, vp]),
        "cgtb_reduce_rkr_f32_static": (ci, [ci, cl, cl, cl, vp, vp]), "cgtb_reduce_static_max_k": (cl, []),
    }
    for (name, (restype, argtypes)) in sig.items():
        f = getattr(lib, name)
        f.restype = restype
        f.argtypes = argtypes
    return sig


C_ABI_SYMBOLS = None


def lib():
    """The loaded library. Raises BackendError when it has not been built."""
    global _lib, C_ABI_SYMBOLS
    if _lib is None:
        if not osp.exists(LIB_PATH):
            raise BackendError("%s is missing: build it with `python -m cgt_b200.build` (there is no CPU fallback)" % LIB_PATH)
        _lib = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
        C_ABI_SYMBOLS = sorted(_declare(_lib).keys())
    return _lib


def last_error():
    return lib().cgtb_last_error().decode("utf-8", "replace")


def check(rc, what=""):
    if rc != 0:
        raise BackendError("%s%s" % (what + ": " if what else "", last_error()))


def gpu_available():
    """True when cgtb_init can bind a B200 (tries once)."""
    try:
        ensure_init()
        return True
    except BackendError:
        return False


_init_error = None


def ensure_init(device=None):
    """Bind this process to one GPU (config device_index unless given). Raises without a GPU."""
    global _init_error
    L = lib()
    if L.cgtb_initialized():
        return
    if _init_error is not None:
        raise BackendError(_init_error)
    if device is None:
        from . import core
        device = int(core.get_config()["device_index"])
    if L.cgtb_init(int(device)) != 0:
        _init_error = last_error()
        raise BackendError(_init_error)


def synchronize():
    check(lib().cgtb_synchronize(), "synchronize")


def kernel_launches():
    return int(lib().cgtb_kernel_launches())


def pool_stats():
    vals = [ctypes.c_long(0) for _ in range(4)]
    lib().cgtb_pool_stats(*[ctypes.byref(v) for v in vals])
    return dict(zip(("reserved_bytes", "in_use_bytes", "high_water_bytes", "n_device_mallocs"), [v.value for v in vals]))


class Event(object):
    """CUDA event on the runtime stream."""

    def __init__(self):
        ensure_init()
        self.h = lib().cgtb_event_new()
        if not self.h:
            raise BackendError(last_error())

    def record(self):
        check(lib().cgtb_event_record(self.h), "event record")

    def elapsed_ms(self, later):
        ms = ctypes.c_float(0)
        check(lib().cgtb_event_elapsed_ms(self.h, later.h, ctypes.byref(ms)), "event elapsed")
        return float(ms.value)

    def __del__(self):
        try:
            if _lib is not None and self.h:
                _lib.cgtb_event_free(self.h)
        except Exception:
            pass


def l2_flush():
    check(lib().cgtb_l2_flush(), "l2 flush")


def _shape_arg(shape):
    return (ctypes.c_long * max(len(shape), 1))(*[int(s) for s in shape])


def _dtype_code(dtype):
    dt = np.dtype(dtype)
    key = ("f" if dt.kind == "f" else "i") + str(dt.itemsize)
    if dt.kind not in "fiub" or key not in DTYPE_NUM:
        raise BackendError("dtype %s is not supported by the backend" % dt)
    return DTYPE_NUM[key]


# ------------------------------------------------------------------------------------------------
# object conversion (src/cycgt.pyx:92-140)
# ------------------------------------------------------------------------------------------------
def py2cgt_array(arr, devtype=CPU, view=True):
    """numpy array -> new reference to a cgtArray. view=True wraps host memory without copying
    (the caller keeps `arr` alive); otherwise the data is copied to `devtype`."""
    L = lib()
    arr = np.asarray(arr)
    if not arr.flags.c_contiguous:
        arr = np.ascontiguousarray(arr)
        view = view and devtype == CPU
    if devtype == GPU:
        ensure_init()
        view = False
    h = L.cgtb_array_from_host(arr.ndim, _shape_arg(arr.shape), _dtype_code(arr.dtype), devtype,
                               ctypes.c_void_p(arr.ctypes.data), 0 if view else 1)
    if not h:
        raise BackendError(last_error())
    return h, arr


def py2cgt_object(o, view=True):
    """numpy array, ArrayWrapper or tuple of them -> (new reference, objects to keep alive)"""
    L = lib()
    if isinstance(o, ArrayWrapper):
        L.cgtb_retain(o.handle)
        return o.handle, o
    if isinstance(o, tuple):
        t = L.cgtb_tuple_new(len(o))
        keep = []
        for (i, el) in enumerate(o):
            h, k = py2cgt_object(el, view)
            L.cgtb_tuple_set(t, i, h)
            L.cgtb_release(h)
            keep.append(k)
        return t, keep
    return py2cgt_array(o, CPU, view)


def cgt2py_object(h):
    """cgtObject -> numpy array (always a copy; device arrays are copied to the host) or tuple"""
    L = lib()
    kind = L.cgtb_object_kind(h)
    if kind == 1:
        ndim = L.cgtb_array_ndim(h)
        shp = L.cgtb_array_shape(h)
        shape = tuple(shp[i] for i in range(ndim))
        out = np.empty(shape, NUM_DTYPE[L.cgtb_array_dtype(h)])
        check(L.cgtb_array_to_host(h, ctypes.c_void_p(out.ctypes.data)), "copy to host")
        return out
    elif kind == 2:
        return tuple(cgt2py_object(L.cgtb_tuple_get(h, i)) for i in range(L.cgtb_tuple_len(h)))
    raise BackendError("cgt object seems to be invalid")


class ArrayWrapper(object):
    """Persistent runtime array (host or device) behind ``cgt.shared``; counterpart of
    CppArrayWrapper (src/cycgt.pyx:371-401). A device array is created lazily, at the first use that
    needs the GPU, so graphs can be built on a machine without one."""

    def __init__(self):
        self.handle = None
        self._host = None
        self._devtype = CPU
        self._ptr_box = None

    @staticmethod
    def from_numpy(nparr, pydevtype="cpu", view=False):
        out = ArrayWrapper()
        out._devtype = GPU if pydevtype == "gpu" else CPU
        out._host = np.array(nparr, copy=True, order="C")
        return out

    def materialize(self):
        if self.handle is None:
            self.handle, _ = py2cgt_array(self._host, self._devtype, view=False)
            self._host_shape = self._host.shape
            self._host_dtype = self._host.dtype
        return self.handle

    def to_numpy(self):
        if self.handle is None:
            return self._host.copy()
        return cgt2py_object(self.handle)

    def set_from_numpy(self, value):
        value = np.ascontiguousarray(value, dtype=self._host.dtype)
        assert value.shape == self._host.shape
        if self.handle is None:
            self._host = value.copy()
        else:
            check(lib().cgtb_array_set_from_host(self.handle, ctypes.c_void_p(value.ctypes.data)), "set_value")

    @property
    def ndim(self):
        return self._host.ndim

    @property
    def shape(self):
        return tuple(self._host.shape)

    @property
    def size(self):
        return int(self._host.size)

    @property
    def dtype(self):
        return self._host.dtype.str[1:]

    @property
    def ptr(self):
        """Address of the cgtArray object (creates the runtime array)."""
        return int(self.materialize())

    @property
    def data(self):
        return int(lib().cgtb_array_data(self.materialize()))

    def __del__(self):
        try:
            if self.handle is not None and _lib is not None:
                _lib.cgtb_release(self.handle)
        except Exception:  # interpreter shutdown
            pass


def device_array(nparr):
    """Copy a numpy array to the GPU; the returned ArrayWrapper can be passed as a function argument."""
    w = ArrayWrapper.from_numpy(nparr, "gpu")
    w.materialize()
    return w


def pinned_empty(shape, dtype):
    """numpy array backed by pinned (page-locked) host memory owned by the runtime pool, so that
    host->device copies of function arguments are truly asynchronous."""
    ensure_init()
    dt = np.dtype(dtype)
    n = int(np.prod(shape, dtype=np.int64)) * dt.itemsize
    p = lib().cgtb_alloc(CPU, max(n, 8192))  # above the small-slab limit -> its own pinned block
    if not p:
        raise BackendError(last_error())
    buf = (ctypes.c_char * max(n, 1)).from_address(p)
    arr = np.frombuffer(buf, dtype=dt, count=int(np.prod(shape, dtype=np.int64))).reshape(shape)
    return arr


def apply_byref(fptr, cldata, inputs, output):
    """Run one native byref callable on numpy arrays / ArrayWrappers (src/cycgt.pyx:439-449)."""
    L = lib()
    handles, keep = [], []
    for x in inputs:
        h, k = py2cgt_object(x, True)
        handles.append(h)
        keep.append(k)
    ho, ko = py2cgt_object(output, True)
    arr = (ctypes.c_void_p * max(len(handles), 1))(*handles)
    clptr = ctypes.c_void_p(ctypes.addressof(cldata)) if isinstance(cldata, ctypes.Structure) else ctypes.c_void_p(0)
    rc = L.cgtb_apply_byref(ctypes.cast(fptr, ctypes.c_void_p), clptr, len(handles), arr, ho)
    for h in handles:
        L.cgtb_release(h)
    L.cgtb_release(ho)
    check(rc, "apply_byref")


# ------------------------------------------------------------------------------------------------
# interpreter wrapper (src/cycgt.pyx:404-434)
# ------------------------------------------------------------------------------------------------
_BYREF_T = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p)
_BYVAL_T = ctypes.CFUNCTYPE(ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p))


def _host_view(h):
    """numpy view of a HOST cgtArray (no copy)"""
    L = lib()
    if L.cgtb_array_devtype(h) != CPU:
        raise BackendError("a Python-implemented Op received a device array; Python Ops run on host values only")
    ndim = L.cgtb_array_ndim(h)
    shp = L.cgtb_array_shape(h)
    shape = tuple(shp[i] for i in range(ndim))
    dt = np.dtype(NUM_DTYPE[L.cgtb_array_dtype(h)])
    n = int(np.prod(shape, dtype=np.int64))
    buf = (ctypes.c_char * max(n * dt.itemsize, 1)).from_address(L.cgtb_array_data(h))
    return np.frombuffer(buf, dtype=dt, count=n).reshape(shape)


def _obj_view(h):
    L = lib()
    if L.cgtb_object_kind(h) == 2:
        return tuple(_obj_view(L.cgtb_tuple_get(h, i)) for i in range(L.cgtb_tuple_len(h)))
    return _host_view(h)


class InterpreterWrapper(object):
    """Builds the native execution graph from the Python one and runs it."""

    def __init__(self, pyeg, input_types, output_locs, flags):
        from . import compilation
        L = lib()
        self.storage = []  # keeps callables, closures and trampolines alive
        self.input_types = input_types
        self.n_instrs = len(pyeg.instrs)
        self.graph = L.cgtb_graph_new(pyeg.n_args, pyeg.n_locs)
        self.interp = None
        dev = {"cpu": CPU, "gpu": GPU}
        for instr in pyeg.instrs:
            r = repr(instr).encode()
            w = instr.write_loc
            if isinstance(instr, compilation.LoadArgument):
                rc = L.cgtb_graph_add_load_argument(self.graph, r, instr.ind, w.index, dev[w.devtype])
            elif isinstance(instr, compilation.Alloc):
                locs = _shape_arg([m.index for m in instr.read_locs])
                rc = L.cgtb_graph_add_alloc(self.graph, r, DTYPE_NUM[instr.dtype], len(instr.read_locs), locs, w.index,
                                            dev[w.devtype])
            elif isinstance(instr, compilation.BuildTup):
                locs = _shape_arg([m.index for m in instr.read_locs])
                rc = L.cgtb_graph_add_build_tup(self.graph, r, len(instr.read_locs), locs, w.index, dev[w.devtype])
            else:
                callable_ = instr.get_callable()
                fptr, clptr, flags_i = self._marshal(callable_, instr)
                locs = _shape_arg([m.index for m in instr.read_locs])
                devs = (ctypes.c_int * max(len(instr.read_locs), 1))(*[dev[m.devtype] for m in instr.read_locs])
                add = L.cgtb_graph_add_return_byref if isinstance(instr, compilation.ReturnByRef) else L.cgtb_graph_add_return_byval
                rc = add(self.graph, r, len(instr.read_locs), locs, devs, w.index, dev[w.devtype], fptr, clptr, flags_i)
            check(rc, "building execution graph")
        olocs = _shape_arg([m.index for m in output_locs])
        self.interp = L.cgtb_interp_new(self.graph, len(output_locs), olocs, flags)
        if not self.interp:
            raise BackendError(last_error())

    def _marshal(self, callable_, instr):
        from . import compilation
        self.storage.append(callable_)
        flags = compilation.instr_flags(instr)
        if callable_.kind == "native":
            flags |= callable_.flags
            cl = callable_.cldata
            clptr = ctypes.c_void_p(ctypes.addressof(cl)) if isinstance(cl, ctypes.Structure) else ctypes.c_void_p(0)
            return ctypes.cast(callable_.fptr, ctypes.c_void_p), clptr, flags
        # Python-implemented Op: trampoline on host values, never captured into a CUDA graph
        n_in, func = callable_.n_in, callable_.func
        L = lib()
        if callable_.return_type == "byref":
            def tramp(_cl, reads, write):
                try:
                    func([_obj_view(reads[i]) for i in range(n_in)], _obj_view(write))
                except Exception as e:  # reported through the error channel, not abort()
                    L.cgt_set_error(b"%s", ("Python Op raised: %r" % (e,)).encode())
            cfun = _BYREF_T(tramp)
        else:
            def tramp(_cl, reads):
                try:
                    out = func([_obj_view(reads[i]) for i in range(n_in)])
                    h, _ = py2cgt_object(out if isinstance(out, tuple) else np.asarray(out), view=False)
                    # ownership passes to the interpreter slot: drop our reference once it has taken its own
                    self._pending_release.append(h)
                    return h
                except Exception as e:
                    L.cgt_set_error(b"%s", ("Python Op raised: %r" % (e,)).encode())
                    return None
            cfun = _BYVAL_T(tramp)
        self.storage.append(cfun)
        return ctypes.cast(cfun, ctypes.c_void_p), ctypes.c_void_p(0), flags | INSTR_NOCAPTURE

    _pending_release = []

    def prefetch(self, *pyargs):
        """Announce the array arguments of a later call f(*pyargs) so that their host->device copy overlaps a step
        instead of running inside one. The upload is issued on the copy stream by the next call of f right after
        that call's own work has been queued (or at once by that call, if it is the one that uses the arrays); the
        call that receives the same array objects waits on the device for the upload and reads the staged copies.
        Typical loop: ``f.prefetch(*batch[i + 1]); loss = f(*batch[i])``. Two staging slots alternate. The arrays
        must not be written between prefetch and the call that uses them. Page-locked arrays
        (runtime.pinned_empty) make the copy asynchronous. Not part of the reference's API, whose Transport
        copies inside the step (cgt/core.py:1419-1430)."""
        assert len(pyargs) == len(self.input_types), "expected %d arguments, got %d" % (len(self.input_types), len(pyargs))
        self._pf_request = pyargs
        if not hasattr(self, "_pf_hook"):
            def hook(_ctx):
                try:
                    if self._pf_request is not None:
                        self._pf_issue()
                except Exception as e:  # surfaces after the run; an exception cannot cross the C frames
                    self._pf_error = e
            self._pf_hook = ctypes.CFUNCTYPE(None, ctypes.c_void_p)(hook)
            check(lib().cgtb_interp_set_before_sync(self.interp, ctypes.cast(self._pf_hook, ctypes.c_void_p), None), "prefetch")

    def _pf_issue(self):
        """Queue the uploads of the announced arguments into the next staging slot."""
        from . import core
        L = lib()
        pyargs, self._pf_request = self._pf_request, None
        if not hasattr(self, "_pf_bufs"):
            self._pf_bufs, self._pf_slot, self._pf = ({}, {}), 0, {}
        self._pf_slot ^= 1
        slot, bufs = self._pf_slot, self._pf_bufs[self._pf_slot]
        check(L.cgtb_prefetch_begin(slot), "prefetch")
        staged = {}
        for (i, (arg, typ)) in enumerate(zip(pyargs, self.input_types)):
            if isinstance(arg, (ArrayWrapper, tuple)):
                continue
            a = core.as_valid_array(arg, typ.dtype)
            if a.ndim != typ.ndim:
                raise ValueError("argument %d has %d dimensions, expected %d" % (i, a.ndim, typ.ndim))
            w = bufs.get(i)
            if w is None or w.shape != a.shape or np.dtype(w.dtype) != a.dtype:
                w = bufs[i] = device_array(np.zeros(a.shape, a.dtype))
            check(L.cgtb_prefetch_h2d(ctypes.c_void_p(w.data), ctypes.c_void_p(a.ctypes.data), ctypes.c_long(a.nbytes)), "prefetch")
            staged[i] = (arg, a, w)  # `a` stays referenced until the call that consumes the upload
        check(L.cgtb_prefetch_mark(slot), "prefetch")
        self._pf[slot] = staged  # replaces an unconsumed upload that used this slot

    def __call__(self, *pyargs):
        from . import core
        L = lib()
        assert len(pyargs) == len(self.input_types), "expected %d arguments, got %d" % (len(self.input_types), len(pyargs))
        request = getattr(self, "_pf_request", None)
        if request is not None and any(r is a for (r, a) in zip(request, pyargs) if not isinstance(a, (ArrayWrapper, tuple))):
            self._pf_issue()  # announced for this very call: upload now
        used_slot = None
        for (slot, staged) in list(getattr(self, "_pf", {}).items()):
            hits = [i for (i, (arg, _a, _w)) in staged.items() if pyargs[i] is arg]
            if hits:
                pyargs = list(pyargs)
                for i in hits:
                    pyargs[i] = staged[i][2]
                check(L.cgtb_prefetch_join(slot), "prefetch join")
                # consumed: a later call with the same arrays copies again; the host sources stay referenced
                # until this call has returned (its result read-back waits for the stream)
                self._pf_keep = self._pf.pop(slot)
                used_slot = slot
                break
        cargs = L.cgtb_tuple_new(len(pyargs))
        keep = []
        for (i, (arg, typ)) in enumerate(zip(pyargs, self.input_types)):
            if isinstance(arg, ArrayWrapper):
                h = arg.materialize()
                L.cgtb_tuple_set(cargs, i, h)
                keep.append(arg)
            elif isinstance(arg, tuple):
                h, k = py2cgt_object(tuple(core.as_valid_array(a) for a in arg), True)
                L.cgtb_tuple_set(cargs, i, h)
                L.cgtb_release(h)
                keep.append(k)
            else:
                a = core.as_valid_array(arg, typ.dtype)
                if a.ndim != typ.ndim:
                    L.cgtb_release(cargs)
                    raise ValueError("argument %d has %d dimensions, expected %d" % (i, a.ndim, typ.ndim))
                h, k = py2cgt_array(a, CPU, view=True)
                L.cgtb_tuple_set(cargs, i, h)
                L.cgtb_release(h)
                keep.append(k)
        out = ctypes.c_void_p(0)
        rc = L.cgtb_interp_run(self.interp, cargs, ctypes.byref(out))
        L.cgtb_release(cargs)
        if used_slot is not None:
            L.cgtb_prefetch_release(used_slot)  # the slot's buffers are free once this step has run
        for h in self._pending_release:
            L.cgtb_release(h)
        del self._pending_release[:]
        check(rc, "running compiled function")
        try:
            err = getattr(self, "_pf_error", None)
            if err is not None:
                self._pf_error = None
                raise err
            return list(cgt2py_object(out.value))
        finally:
            L.cgtb_release(out)

    def stats(self):
        vals = (ctypes.c_long * 8)()
        lib().cgtb_interp_stats(self.interp, vals, 8)
        return dict(zip(("runs", "last_kernel_launches", "last_graph_launches", "segments_captured", "graph_kernels",
                         "device_instructions", "last_host_ns", "steady_runs"), list(vals)))

    def profile(self):
        """[(instruction repr, total ms, count)] when the interpreter was created with profiling on"""
        L = lib()
        n = self.n_instrs
        ms = (ctypes.c_double * max(n, 1))()
        counts = (ctypes.c_long * max(n, 1))()
        L.cgtb_interp_profile(self.interp, ms, counts, n)
        return [(L.cgtb_interp_instr_repr(self.interp, i).decode(), ms[i], counts[i]) for i in range(n)]

    def __del__(self):
        try:
            if _lib is not None:
                if self.interp:
                    _lib.cgtb_interp_free(self.interp)
                if self.graph:
                    _lib.cgtb_graph_free(self.graph)
        except Exception:
            pass
