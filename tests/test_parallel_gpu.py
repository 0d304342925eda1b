"""Data parallelism on real GPUs: two ranks, one B200 each, gradients summed by the NCCL AllReduce Op.
The two ranks with half a batch each must end with the same parameters as one GPU with the whole
batch (float32 tolerance: the mean of two half-batch gradients rounds differently), and the replicas
must stay bit-identical to each other. Skipped on a box with fewer than two GPUs."""
import json
import os
import os.path as osp
import subprocess
import sys

import numpy as np
import pytest

from cgt_b200 import configs
import cgt_b200 as cgt
from tests.test_parallel_cpu import _free_port

pytestmark = pytest.mark.gpu
HERE = osp.dirname(osp.abspath(__file__))


def _n_gpus():
    import torch
    return torch.cuda.device_count()


@pytest.mark.parametrize("config,two_phase", [("mlp", False), ("cifar", False), ("cifar", True)])
def test_two_gpu_ranks_match_one_gpu(rt, tmp_path, config, two_phase):
    """two_phase: every payload goes through the two-phase peer kernel (each rank sums one slice, all collect the slices),
    which otherwise serves payloads beyond a megabyte."""
    if _n_gpus() < 2:
        pytest.skip("needs two GPUs")
    world, per_rank = 2, 8
    port = _free_port()
    procs = []
    for rank in range(world):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), DP_OUT=str(tmp_path / "params"), DP_BACKEND="gpu", DP_CONFIG=config)
        if two_phase:
            env["CGTB_PEER_TWO_PHASE_BYTES"] = "0"
        procs.append(subprocess.Popen([sys.executable, osp.join(HERE, "dp_worker.py")], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.PIPE, text=True))
    outs = []
    try:
        for p in procs:
            so, se = p.communicate(timeout=300)
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
    assert all(o["n_allreduce"] == 1 for o in outs)
    # small gradients travel through the peer-memory kernel, which stays inside the step's captured graph
    assert all(o["peer"] and o["graph_launches"] == 1 for o in outs), outs
    p0 = np.load(str(tmp_path / "params") + ".0.npz")
    p1 = np.load(str(tmp_path / "params") + ".1.npz")
    for k in p0.files:
        assert np.array_equal(p0[k], p1[k])
    build = getattr(configs, "build_" + config)
    cfg = build(batch=per_rank * world)
    f = cgt.function(cfg.inputs, [cfg.loss], updates=cfg.updates)
    losses = [float(f(*cfg.batch(step))[0]) for step in range(3)]
    for (k, p) in zip(p0.files, cfg.params):
        np.testing.assert_allclose(p0[k], p.op.get_value(), rtol=1e-3, atol=1e-5)
    for step in range(3):
        np.testing.assert_allclose(np.mean([o["losses"][step] for o in outs]), losses[step], rtol=1e-3)
