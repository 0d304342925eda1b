"""Minibatch-sharded data parallelism: one process per GPU, identical graph and parameters on every
rank, each rank's gradients summed across ranks by an ``AllReduce`` Op placed between ``cgt.grad``'s
outputs and the update expressions.

The reference has no multi-device collective; its documented data parallelism splits the batch
across CPU threads inside one graph (doc/index.rst:212-238). Here the batch is split across
processes. ``torch.distributed`` (gloo) carries the rendezvous, the NCCL unique id and barriers; the
gradient bytes move through NCCL over NVLink, queued on the runtime's CUDA stream by the Op's
native callable.
"""
import ctypes
import os
import os.path as osp

import numpy as np

from . import core

_state = {"world": 1, "rank": 0, "local_rank": 0, "comm": False, "peer": False}

# Payloads up to this size go through the peer-memory kernels instead of NCCL. Default 4 MiB: every configuration but the
# wide one (21 MB of gradients). CGTB_PEER_SLOT_MB=32 sends that one through the two-phase peer kernel as well (one graph
# launch per step, no NCCL); measured on B200s it equals NCCL at two GPUs (0.846 vs 0.840 ms per step) and is 17 us
# slower at four (0.890 vs 0.873 ms), so NCCL stays the default for large payloads.
PEER_SLOT_BYTES = int(os.environ.get("CGTB_PEER_SLOT_MB", "4")) << 20


def world_size():
    return _state["world"]


def rank():
    return _state["rank"]


def _find_nccl():
    cands = []
    try:
        import torch
        base = osp.dirname(osp.dirname(torch.__file__))
        cands.append(osp.join(base, "nvidia", "nccl", "lib", "libnccl.so.2"))
    except ImportError:
        pass
    cands += ["/usr/lib/x86_64-linux-gnu/libnccl.so.2"]
    for c in cands:
        if osp.exists(c):
            return c
    raise RuntimeError("no NCCL library found (looked in %s)" % cands)


def init_process_group(with_gpu=True):
    """Join the job described by RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT.

    with_gpu=False sets up only the host-side group (gloo); the AllReduce Op can then be evaluated by
    the CPU oracle, which is how the multi-rank logic is tested without GPUs."""
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rk = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rk)))
    _state.update(world=world, rank=rk, local_rank=local)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group(backend="gloo", rank=rk, world_size=world)
    if with_gpu:
        from . import runtime
        core.update_config(device_index=local, default_device=core.Device("gpu", local))
        runtime.ensure_init(local)
        if world > 1 and not _state["comm"]:
            L = runtime.lib()
            runtime.check(L.cgtb_comm_load(_find_nccl().encode()), "loading NCCL")
            idbuf = ctypes.create_string_buffer(128)
            if rk == 0:
                runtime.check(L.cgtb_comm_unique_id(idbuf), "ncclGetUniqueId")
            box = [bytes(idbuf.raw)]
            dist.broadcast_object_list(box, src=0)
            runtime.check(L.cgtb_comm_init(box[0], rk, world), "ncclCommInitRank")
            _state["comm"] = True
            if os.environ.get("CGTB_PEER_ALLREDUCE", "1") != "0" and world <= 8:
                _open_peer_group(L, rk, world)
    return rk, world


def _open_peer_group(L, rk, world):
    """Symmetric buffers for the peer-memory all-reduce: every rank allocates one, the 64-byte IPC handles travel
    through the host group, every rank maps the others'. Ranks must share a node (NVLink / PCIe peer access)."""
    import torch.distributed as dist
    from . import runtime
    h = ctypes.create_string_buffer(64)
    runtime.check(L.cgtb_peer_alloc(PEER_SLOT_BYTES, h), "cgtb_peer_alloc")
    handles = [None] * world
    dist.all_gather_object(handles, bytes(h.raw))
    runtime.check(L.cgtb_peer_open(b"".join(handles), rk, world), "cgtb_peer_open")
    if os.environ.get("CGTB_PEER_TWO_PHASE_BYTES"):   # payload size above which the two-phase kernel runs (default 1 MiB)
        runtime.check(L.cgtb_peer_set_two_phase_bytes(int(os.environ["CGTB_PEER_TWO_PHASE_BYTES"])), "cgtb_peer_set_two_phase_bytes")
    dist.barrier()
    _state["peer"] = True


def barrier():
    if _state["world"] > 1:
        import torch.distributed as dist
        dist.barrier()


def device_barrier():
    """Queues, on the runtime's stream, a collective that completes only when every rank's stream has reached the same
    point (an NCCL all-reduce of one float, outside any captured graph): what follows it on the streams starts on all
    GPUs within a few microseconds, whatever the skew between the host processes. False (and nothing queued) with one
    process. Every rank must call it the same number of times."""
    if not _state["comm"]:
        return False
    from . import runtime
    if _state.get("barrier_word") is None:
        _state["barrier_word"] = runtime.device_array(np.zeros((1,), "f4"))
    w = _state["barrier_word"]
    ptrs = (ctypes.c_void_p * 1)(w.data)
    runtime.check(runtime.lib().cgtb_allreduce_sum(runtime._dtype_code(np.dtype("f4")), 1, ptrs, ptrs, (ctypes.c_long * 1)(1)),
                  "cgtb_allreduce_sum")
    return True


def all_max(value):
    """max over ranks of a host float (timing reduction)"""
    if _state["world"] == 1:
        return float(value)
    import torch
    import torch.distributed as dist
    t = torch.tensor([float(value)], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def check_health():
    """Raises when NCCL has reported an asynchronous error (a peer died or a link failed)."""
    if _state["comm"]:
        from . import runtime
        runtime.check(runtime.lib().cgtb_comm_check(), "communicator")


def shutdown():
    if _state["peer"]:
        from . import runtime
        barrier()   # nobody unmaps a buffer that a peer's kernel may still read
        runtime.lib().cgtb_peer_close()
        _state["peer"] = False
    if _state["comm"]:
        from . import runtime
        runtime.lib().cgtb_comm_destroy()
        _state["comm"] = False
    try:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()
    except ImportError:
        pass
    _state.update(world=1, rank=0)


class AllReduce(core.Op):
    """(g_1, ..., g_k) -> tuple of their sums over all ranks. All k reductions are queued as one group."""
    available_impls = ("native_gpu",)

    def __init__(self, n, peer=False):
        """peer=True: the exchange runs as one kernel over peer memory (small float32 payloads; an ordinary launch,
        so it stays inside the step's captured CUDA graph); otherwise through NCCL, outside captured graphs."""
        self.n = n
        self.peer = bool(peer)

    def get_diff(self, n):
        return [False] * n

    def typ_apply(self, input_types):
        return core.TupleType(*input_types)

    def shp_apply(self, inputs):
        return tuple(core.cgt.shape(x) for x in inputs)

    def get_native_compile_info(self, input_types, devtype):
        from . import runtime
        if self.peer:
            return core.NativeCompileInfo(None, prebuilt="cgtb_op_allreduce_peer", closure_triples=[("n", ctypes.c_int, self.n)])
        # stream-ordered, but issued outside captured CUDA graphs (same class as a Transport)
        return core.NativeCompileInfo(None, prebuilt="cgtb_op_allreduce", closure_triples=[("n", ctypes.c_int, self.n)],
                                      flags=runtime.INSTR_TRANSPORT)

    def oracle_eval(self, vals):
        """Host evaluation for the test oracle: torch.distributed (gloo) all_reduce on copies."""
        if _state["world"] == 1:
            return tuple(np.array(v, copy=True) for v in vals)
        import torch
        import torch.distributed as dist
        out = []
        for v in vals:
            t = torch.from_numpy(np.array(v, copy=True))
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
            out.append(t.numpy())
        return tuple(out)

    def __repr__(self):
        return "AllReduce{%d%s}" % (self.n, ",peer" if self.peer else "")


def allreduce_mean(grads):
    """Average a list of gradient nodes over the ranks; the identity when there is one rank."""
    grads = list(grads)
    w = world_size()
    if w == 1:
        return grads
    tup = core.Result(AllReduce(len(grads), peer=_fits_peer_path(grads)), grads)
    inv = np.array(1.0 / w, core.cgt.floatX)
    return [tup[i] * inv for i in range(len(grads))]


def _fits_peer_path(grads):
    """True when a peer group is open and the gradients are float32 tensors of static shape that fit its slot together."""
    if not _state["peer"] or len(grads) > 32:
        return False
    total = 0
    for g in grads:
        if g.dtype != "f4":
            return False
        try:
            shp = core.cgt.infer_shape(g)
        except Exception:
            return False
        if shp is None or any(s is None for s in shp):
            return False
        total += int(np.prod(shp)) * 4
    return total + 16 * 32 <= PEER_SLOT_BYTES   # in the slot every tensor starts on a 16-byte boundary


def shard(arrays, rank_=None, world=None):
    """This rank's slice of a global batch along axis 0."""
    rank_ = rank() if rank_ is None else rank_
    world = world_size() if world is None else world
    out = []
    for a in arrays:
        n = a.shape[0] // world
        out.append(np.ascontiguousarray(a[rank_ * n:(rank_ + 1) * n]))
    return out
