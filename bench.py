"""Benchmark of the compiled-graph training step on B200: train examples/sec (forward + cgt.grad
backward + SGD update) of the CIFAR-shape convnet at batch 128 per GPU, on synthetic data.

    python bench.py --gpus N --steps K --warmup W            # this backend (one rank per GPU under torchrun)
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU path on the host cores

Prints ONE JSON line (rank 0). `value` is measured with the batch already resident in device memory;
`e2e` goes through the public API with pinned host buffers (host->device copy of the batch and
device->host read of the loss inside every timed step). Every timed step is bracketed by CUDA events on
the runtime stream and preceded by an L2 flush that is not timed; per-rank totals are reduced with max.
"""
import argparse
import json
import os
import os.path as osp
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = osp.dirname(osp.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "train examples/sec (fwd+bwd+SGD) CIFAR-shape convnet b128"
UNIT = "examples/s"
BATCH = 128


def load_peaks():
    p = osp.join(ROOT, "MEASURED_PEAKS.json")
    if osp.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], bf16_tflops_sustained=d.get("bf16_tflops_sustained"),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


# ------------------------------------------------------------------------------------------------
# clocks during the timed region
# ------------------------------------------------------------------------------------------------
class ClockSampler(object):
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device = device
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.device), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, reasons = [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    out["sm_max_mhz"] = float(f[2])
                except ValueError:
                    continue
                for (name, v) in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except OSError:
            pass
        if sm:
            out["sm_mhz"] = float(np.median(sm))
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


# algorithmic bytes / flops per instruction: every operand and result of an Op crosses HBM once; 2MNK flops per product
# algorithmic bytes / flops per instruction (per-op figures stated in DESIGN.md)
# ------------------------------------------------------------------------------------------------
def _nbytes(shape, dtype):
    if shape is None:
        return 0
    return int(np.prod(shape, dtype=np.int64)) * int(dtype[1:])


def algorithmic_cost(instr):
    """(bytes, flops) that the instruction must move / compute, from its static shapes."""
    from cgt_b200 import core
    op = instr.op
    name = type(op).__name__
    ins = [(s, d) for (s, d) in zip(instr.in_shapes, instr.in_dtypes)]
    out_shape, out_dtype = instr.out_shape, instr.out_dtype
    if name == "MaxPool":  # values + int32 mask
        top = out_shape[0]
        return _nbytes(ins[0][0], ins[0][1]) + _nbytes(top, ins[0][1]) + _nbytes(top, "i4"), 0
    if name == "CrossChannelLRNForward":
        return 3 * _nbytes(ins[0][0], ins[0][1]), 0
    if isinstance(out_shape, tuple) and out_shape and isinstance(out_shape[0], tuple):
        return sum(_nbytes(s, d) for (s, d) in ins) + sum(_nbytes(s, ins[0][1]) for s in out_shape), 0
    out_b = _nbytes(out_shape, out_dtype)
    if name == "MaxPoolPullback":  # mask + pooled gradient read, input gradient written; x and pooled give shapes only
        return _nbytes(ins[2][0], ins[2][1]) + _nbytes(ins[3][0], ins[3][1]) + out_b, 0
    if name in ("Mul22",):
        (sa, _), (sb, _) = ins[0], ins[1]
        M, N = out_shape
        K = sa[0] if op.tA else sa[1]
        return 4 * (M * K + K * N + M * N), 2 * M * N * K
    if name in ("Reshape", "Size", "TupleIndex", "InMemoryData", "Arange"):
        return 0, 0
    host = set(op.host_inputs(len(ins))) if hasattr(op, "host_inputs") else set()
    in_b = sum(_nbytes(s, d) for (i, (s, d)) in enumerate(ins) if i not in host)
    if name in ("IncSli", "IncFlatIndices"):  # in place: read the increment and the touched part, write it back
        return 3 * _nbytes(ins[-1][0], ins[-1][1]), 0
    return in_b + out_b, 0


def profile_ops(cfg_builder, batch_dev, steps=20):
    """Per-Op device time from a profiled pass (CUDA events around every instruction), with the
    algorithmic bytes / flops of each Op class per step."""
    import cgt_b200 as cgt
    from cgt_b200 import compilation, runtime
    with cgt.scoped_update_config(profile=True, use_cuda_graphs=False):
        cfg = cfg_builder()
        f = cfg.compile()
    for _ in range(3):
        f(*batch_dev)
    base = {i: (ms, c) for (i, (_r, ms, c)) in enumerate(f.profile())}
    for _ in range(steps):
        runtime.l2_flush()
        f(*batch_dev)
    table = {}
    for (i, (instr, (_r, ms, c))) in enumerate(zip(f.eg.instrs, f.profile())):
        ms -= base[i][0]
        c -= base[i][1]
        if c <= 0 or not isinstance(instr, compilation._Return):
            continue
        key = type(instr.op).__name__
        b, fl = algorithmic_cost(instr)
        t = table.setdefault(key, dict(ms=0.0, launches=0, bytes=0, flops=0))
        t["ms"] += ms / steps
        t["launches"] += c / steps
        t["bytes"] += b
        t["flops"] += fl
    return table


# ------------------------------------------------------------------------------------------------
# timed loops
# ------------------------------------------------------------------------------------------------
def timed_steps(f, batches, steps, warmup, flush=True, prefetch=False):
    """Returns (total device ms over `steps`, last loss). Each step: untimed L2 flush, event, step, event.
    prefetch: inside every timed step the NEXT step's batch is handed to f.prefetch before the step is called, so
    its host->device copy (one per step, like without prefetch) runs on the copy stream beside the step."""
    from cgt_b200 import parallel, runtime
    nb = len(batches)
    if prefetch:
        f.prefetch(*batches[0])
    for i in range(warmup):
        if prefetch:
            f.prefetch(*batches[(i + 1) % nb])
        f(*batches[i % nb])
    e0, e1 = runtime.Event(), runtime.Event()
    parallel.barrier()
    runtime.synchronize()
    total = 0.0
    loss = None
    for i in range(steps):
        if flush:
            runtime.l2_flush()
            runtime.synchronize()
        e0.record()
        if prefetch:
            f.prefetch(*batches[(warmup + i + 1) % nb])
        loss = f(*batches[(warmup + i) % nb])[0] if prefetch else f(*batches[i % nb])[0]
        e1.record()
        total += e0.elapsed_ms(e1)
    runtime.synchronize()
    parallel.barrier()
    return parallel.all_max(total), float(loss)


def run_b200(args):
    import cgt_b200 as cgt
    from cgt_b200 import configs, parallel, runtime
    rank, world = parallel.init_process_group() if int(os.environ.get("WORLD_SIZE", "1")) > 1 else (0, 1)
    if world == 1:
        runtime.ensure_init()
    assert world == args.gpus, "--gpus %d but WORLD_SIZE is %d (launch with torch.distributed.run)" % (args.gpus, world)

    def builder():
        return configs.build_cifar(batch=BATCH, grad_hook=parallel.allreduce_mean)
    cfg = builder()
    f = cfg.compile()
    # every rank draws its own 128-example shard (weak scaling); 4 batches are cycled
    host_batches, dev_batches = [], []
    for j in range(4):
        b = cfg.batch(seed=1000 * rank + j)
        pinned = []
        for a in b:
            p = runtime.pinned_empty(a.shape, a.dtype)
            p[...] = a
            pinned.append(p)
        host_batches.append(pinned)
        dev_batches.append([runtime.device_array(a) for a in b])
    h2d = int(sum(a.nbytes for a in host_batches[0]))

    sampler = ClockSampler(runtime.lib().cgtb_device())
    if rank == 0:
        sampler.start()
    ms_dev, loss = timed_steps(f, dev_batches, args.steps, args.warmup)
    st = f.stats()
    launches = int(st["last_kernel_launches"]) * args.steps
    ms_e2e_serial, _ = timed_steps(f, host_batches, args.steps, max(3, args.warmup // 4))
    ms_e2e, _ = timed_steps(f, host_batches, args.steps, max(3, args.warmup // 4), prefetch=True)
    clocks = sampler.stop() if rank == 0 else None

    out = None
    if rank == 0:
        n_examples = BATCH * world * args.steps
        out = {
            "metric": METRIC, "value": n_examples / (ms_dev / 1e3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32 (3xTF32 tensor-core GEMM where used, fp32 elsewhere)", "data": "synthetic",
            "config": {"workload": "CIFAR-shape convnet, batch 128 per GPU, fwd+bwd+SGD (BASELINE configs[1])",
                       "global_batch": BATCH * world, "parallelism": "dp%d" % world,
                       "l2": "flushed between timed steps (256 MiB memset, untimed)", "cuda_graphs": bool(st["segments_captured"]),
                       "kernels_per_step": int(st["last_kernel_launches"]), "graph_launches_per_step": int(st["last_graph_launches"])},
            "e2e": {"value": n_examples / (ms_e2e / 1e3), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                    "ms_per_step": ms_e2e / args.steps,
                    "input_upload": "pinned host batch -> f.prefetch: copied on the copy stream while the step before it runs; one copy per timed step",
                    "value_copy_inside_step": n_examples / (ms_e2e_serial / 1e3)},
            "gpu_launches": launches, "clocks": clocks, "final_loss": loss,
        }
    # roofline of the dominant kernel (rank 0, on the single-GPU graph: the per-GPU work is the same at every
    # N under weak scaling) and, at N = 1, the CPU baseline
    if rank == 0 and not args.no_extras:
        peaks = load_peaks()
        table = profile_ops(lambda: configs.build_cifar(batch=BATCH), dev_batches[0])
        total_ms = sum(t["ms"] for t in table.values())
        dom = max(table.items(), key=lambda kv: kv[1]["ms"])
        name, t = dom
        sec = t["ms"] / 1e3
        gbs = t["bytes"] / sec / 1e9 if sec > 0 else 0.0
        tfl = t["flops"] / sec / 1e12 if sec > 0 else 0.0
        tf32_peak = peaks["bf16_tflops"] / 2.0  # dense TF32 runs at half the bf16 rate on this part
        hbm_floor, tensor_floor = t["bytes"] / (peaks["hbm_gbs"] * 1e9), t["flops"] / (tf32_peak * 1e12)
        if t["flops"] and tensor_floor > hbm_floor:
            roof = {"bound": "tensor", "achieved": tfl, "peak": tf32_peak, "unit": "TFLOP/s", "frac": tfl / tf32_peak}
        else:
            roof = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"]}
        ratio = NCU_TRAFFIC_RATIO.get(name)
        roof.update({"kernel": name, "traffic": (ratio * t["bytes"]) if ratio else None,
                     "traffic_note": NCU_TRAFFIC_NOTE.get(name), "peak_source": peaks["source"],
                     "share_of_step": t["ms"] / total_ms, "launches_per_step": t["launches"],
                     "algorithmic_bytes_per_step": t["bytes"], "ms_per_step": t["ms"]})
        out["roofline"] = roof
        out["per_op"] = {k: {"ms": round(v["ms"], 4), "GB/s": round(v["bytes"] / (v["ms"] / 1e3) / 1e9, 1) if v["ms"] > 0 else None,
                             "share": round(v["ms"] / total_ms, 3)} for (k, v) in sorted(table.items(), key=lambda kv: -kv[1]["ms"])}
        step_bytes = sum(v["bytes"] for v in table.values())
        out["step_roofline"] = {"algorithmic_bytes_per_step": step_bytes, "hbm_floor_ms": step_bytes / (peaks["hbm_gbs"] * 1e9) * 1e3,
                                "frac": (step_bytes / (peaks["hbm_gbs"] * 1e9) * 1e3) / (ms_dev / args.steps)}
        if world == 1:
            out["cpu_baseline"] = cpu_baseline(sample_steps=5, warmup=2)
    parallel.barrier()
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        parallel.shutdown()


# DRAM traffic of the dominant Op class from an ncu capture (dram__bytes_read.sum + dram__bytes_write.sum of one
# launch, summary under profiles/), as a ratio to that launch's algorithmic bytes; `traffic` scales the class's
# algorithmic bytes per step by it (the captured launch streams its operands once, like every launch of the class).
NCU_TRAFFIC_RATIO = {"Mul22": 96.33 / 95.95, "ConvBiasRelu": 96.33 / 95.95}
NCU_TRAFFIC_NOTE = {"Mul22": "ncu capture of the conv2 forward product 28800x32x800 (sgemm_tma_kernel): 92.31 MB read + 4.02 MB "
                             "written against 95.95 MB algorithmic; scaled to the class's algorithmic bytes per step",
                    "ConvBiasRelu": "same kernel as Mul22 with the output stage in its epilogue. ncu captures of its products: conv2 "
                                    "28800x32x800 92.31 MB read + 4.02 MB written against 95.95 MB algorithmic; conv1 131072x32x76 "
                                    "39.90 MB read against 39.85 MB of operand (its 16.8 MB result was still in L2 when the kernel "
                                    "ended: 0.02 MB written). Operands are streamed once; the conv2 ratio scales the class's "
                                    "algorithmic bytes per step"}


# ------------------------------------------------------------------------------------------------
# CPU arm: the reference's CPU implementation of the path (its own im2col.h / pooling.h / lrn.cuh-as-C++
# when oracle/_ref is built, restated loops otherwise, OpenBLAS sgemm on all host cores)
# ------------------------------------------------------------------------------------------------
def _cpu_function(batch):
    import cgt_b200  # noqa: F401  (graph front-end only; nothing is placed on a GPU here)
    from cgt_b200 import configs
    from oracle import cpu_backend, oracle
    cfg = configs.build_cifar(batch=batch)
    kind = "reference" if oracle.have_ref() else "port"
    f = cpu_backend.function(cfg.inputs, [cfg.loss], updates=cfg.updates, impl="ref" if kind == "reference" else "port")
    return cfg, f, kind


def cpu_baseline(sample_steps=5, warmup=2):
    cfg, f, kind = _cpu_function(BATCH)
    b = cfg.batch(0)
    for _ in range(warmup):
        f(*b)
    ts = []
    for _ in range(sample_steps):
        t0 = time.perf_counter()
        f(*b)
        ts.append(time.perf_counter() - t0)
    med = float(np.median(ts))
    return {"value": BATCH / med, "unit": UNIT, "cores": os.cpu_count(), "kind": kind,
            "sample": "%d full training steps at batch %d after %d warm-ups, median step %.3f s; OpenBLAS sgemm on all host "
                      "threads, other ops single-threaded as in the reference's sequential interpreter" % (sample_steps, BATCH, warmup, med)}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    budget_s = 150.0
    cfg, f, kind = _cpu_function(BATCH)
    b = cfg.batch(0)
    t0 = time.perf_counter()
    f(*b)
    t1 = time.perf_counter() - t0
    batch = BATCH
    total_steps = args.steps + args.warmup
    if t1 * total_steps > budget_s:  # bounded sample: a smaller batch per step, same network
        batch = int(max(1, min(BATCH, BATCH * budget_s / (t1 * total_steps))))
        cfg, f, kind = _cpu_function(batch)
        b = cfg.batch(0)
    for _ in range(args.warmup):
        f(*b)
    t0 = time.perf_counter()
    loss = None
    for _ in range(args.steps):
        loss = f(*b)[0]
    dt = time.perf_counter() - t0
    value = batch * args.steps / dt
    sample = "each step is one full training step on %d of the %d examples of a batch (same network and op sequence)" % (batch, BATCH)
    out = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "CIFAR-shape convnet, fwd+bwd+SGD (BASELINE configs[1]) on the host cores", "batch_per_step": batch},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": os.cpu_count(), "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "final_loss": float(loss),
    }
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the per-Op profile pass and the CPU baseline (for ncu runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
