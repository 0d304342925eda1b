"""Data-parallel host logic on CPU ranks (gloo, world_size 2): the AllReduce Op inserted between
cgt.grad's outputs and the updates averages the shard gradients, so two ranks with half a batch each
end with the same parameters as one process with the whole batch. No GPU involved: the graphs run on
the CPU oracle, whose evaluation of the Op is a gloo all_reduce."""
import json
import os
import os.path as osp
import socket
import subprocess
import sys

import numpy as np

import cgt_b200 as cgt  # noqa: F401
from cgt_b200 import configs, parallel
from oracle import cpu_backend

HERE = osp.dirname(osp.abspath(__file__))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def test_two_ranks_match_single_process(tmp_path):
    world, per_rank = 2, 8
    port = _free_port()
    procs = []
    for rank in range(world):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), DP_OUT=str(tmp_path / "params"), OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, osp.join(HERE, "dp_worker.py")], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.PIPE, text=True))
    outs = []
    try:
        for p in procs:
            so, se = p.communicate(timeout=240)
            assert p.returncode == 0, se[-3000:]
            outs.append(json.loads(so.strip().splitlines()[-1]))
    finally:
        # a rank that outlives the test (a stalled collective, a peer that failed first) must not keep a device
        for p in procs:
            if p.poll() is None:
                p.kill()
            try:
                p.wait(timeout=30)
            except subprocess.TimeoutExpired:
                pass
    assert [o["rank"] for o in outs] == [0, 1] and all(o["world"] == 2 for o in outs)
    assert all(o["n_allreduce"] == 1 for o in outs)  # one grouped exchange for all parameter gradients
    # replicas stay bit-identical: same averaged gradients applied to the same parameters
    p0 = np.load(str(tmp_path / "params") + ".0.npz")
    p1 = np.load(str(tmp_path / "params") + ".1.npz")
    for k in p0.files:
        assert np.array_equal(p0[k], p1[k])
    # single process, whole batch
    cfg = configs.build_mlp(batch=per_rank * world)
    f = cpu_backend.function(cfg.inputs, [cfg.loss], updates=cfg.updates)
    losses = [float(f(*cfg.batch(step))[0]) for step in range(3)]
    for (k, p) in zip(p0.files, cfg.params):
        np.testing.assert_allclose(p0[k], f.get_value(p), rtol=2e-5, atol=1e-7)
    # the global loss is the mean of the shard losses
    for step in range(3):
        np.testing.assert_allclose(np.mean([o["losses"][step] for o in outs]), losses[step], rtol=1e-5)


def test_single_rank_is_the_identity():
    x = cgt.matrix("x", fixed_shape=(2, 2))
    assert parallel.world_size() == 1
    g = [x * 2.0]
    assert parallel.allreduce_mean(g) == g
    assert [a.tolist() for a in parallel.shard([np.arange(8).reshape(4, 2)], 1, 2)] == [[[4, 5], [6, 7]]]
    # without a communicator there is nothing to line up with: the device-side barrier queues nothing
    assert parallel.device_barrier() is False
