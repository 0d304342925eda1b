"""Worker of the world_size-2 data-parallel tests (launched by tests/test_parallel_cpu.py and
tests/test_parallel_gpu.py with RANK / WORLD_SIZE / MASTER_* set). Every rank builds the same model,
takes its shard of a global batch, and runs three update steps with the AllReduce Op between cgt.grad
and the updates: on the CPU oracle (DP_BACKEND unset: the Op is a gloo all_reduce) or on one GPU per
rank through the native interpreter (DP_BACKEND=gpu: the Op is an NCCL all-reduce)."""
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import cgt_b200 as cgt  # noqa: E402,F401
from cgt_b200 import configs, parallel  # noqa: E402
from oracle import cpu_backend  # noqa: E402

on_gpu = os.environ.get("DP_BACKEND") == "gpu"
build = getattr(configs, "build_" + os.environ.get("DP_CONFIG", "mlp"))
rank, world = parallel.init_process_group(with_gpu=on_gpu)
per_rank = 8
cfg = build(batch=per_rank, grad_hook=parallel.allreduce_mean)
if on_gpu:
    f = cgt.function(cfg.inputs, [cfg.loss], updates=cfg.updates)
    n_allreduce = sum(1 for instr in f.eg.instrs if "AllReduce" in repr(instr))
else:
    f = cpu_backend.function(cfg.inputs, [cfg.loss], updates=cfg.updates)
    n_allreduce = sum(1 for n in f.nodes if isinstance(n.op, parallel.AllReduce))
losses = []
for step in range(3):
    full = build(batch=per_rank * world).batch(step)  # the global batch, same on every rank
    shard = parallel.shard(full, rank, world)
    losses.append(float(f(*shard)[0]))
    parallel.check_health()  # raises (and ends this rank) when the communicator reported an asynchronous error
params = [p.op.get_value() for p in cfg.params] if on_gpu else [f.get_value(p) for p in cfg.params]
stats = f.stats() if on_gpu else {}
out = {"rank": rank, "world": world, "losses": losses, "n_allreduce": n_allreduce,
       "graph_launches": int(stats.get("last_graph_launches", 0)), "peer": bool(parallel._state["peer"]),
       "checksum": [float(np.abs(p).sum()) for p in params], "first": [float(p.ravel()[0]) for p in params]}
np.savez(os.environ["DP_OUT"] + ".%d.npz" % rank, *params)
print(json.dumps(out))
parallel.shutdown()
