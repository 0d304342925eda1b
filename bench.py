"""Benchmark of the compiled-graph training step on B200: train examples/sec (forward + cgt.grad
backward + SGD update) of the CIFAR-shape convnet at batch 128 per GPU, on synthetic data.

    python bench.py --gpus N --steps K --warmup W            # this backend (one rank per GPU under torchrun)
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU path on the host cores
    python bench.py --config wide ...                        # the wide conv stack (128 examples per GPU) instead

Prints ONE JSON line (rank 0). `value` is measured with the batch already resident in device memory;
`e2e` goes through the public API with pinned host buffers (host->device copy of the batch and
device->host read of the loss inside every timed step). Every timed step is bracketed by CUDA events on
the runtime stream and preceded by an L2 flush that is not timed. The block of K steps is repeated R times
(--repeats, default 15) inside one invocation; each block is bracketed by a barrier and a synchronisation, its
time is the max over ranks, and the reported figure is the median block (`spread` gives the fastest and the
slowest one). `per_kernel` times every C-ABI entry point of the step at the step's own shapes in a loop of cold-L2
launches; `roofline` is the entry of that list with the largest share of the step.
"""
import argparse
import ctypes
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

UNIT = "examples/s"
BATCH = 128
CONFIGS = {
    "cifar": dict(builder="build_cifar", metric="train examples/sec (fwd+bwd+SGD) CIFAR-shape convnet b128",
                  workload="CIFAR-shape convnet, batch 128 per GPU, fwd+bwd+SGD (BASELINE configs[1])"),
    "wide": dict(builder="build_wide", metric="train examples/sec (fwd+bwd+SGD) wide conv stack b128 per GPU",
                 workload="wide conv stack 3x64x64 -> conv96/11/4 -> LRN -> pool -> conv256/5 -> pool -> fc4096 -> fc100, "
                          "batch 128 per GPU, fwd+bwd+SGD (BASELINE configs[4])"),
}


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


# ------------------------------------------------------------------------------------------------
# algorithmic bytes / flops per instruction: every operand and result of an Op crosses HBM once, each at its
# own element size; 2MNK flops per product
# ------------------------------------------------------------------------------------------------
def _nbytes(shape, dtype):
    if shape is None or not isinstance(dtype, str) or len(dtype) < 2 or not dtype[1:].isdigit():
        return 0  # unknown extent, or a tuple-typed operand (its members are counted where they are produced)
    if shape and isinstance(shape[0], tuple):
        return 0
    return int(np.prod(shape, dtype=np.int64)) * int(dtype[1:])


def algorithmic_cost(instr):
    """(bytes, flops) that the instruction must move / compute, from its static shapes."""
    op = instr.op
    name = type(op).__name__
    ins = [(s, d) for (s, d) in zip(instr.in_shapes, instr.in_dtypes)]
    out_shape, out_dtype = instr.out_shape, instr.out_dtype
    host = set(op.host_inputs(len(ins))) if hasattr(op, "host_inputs") else set()
    in_b = sum(_nbytes(s, d) for (i, (s, d)) in enumerate(ins) if i not in host)
    if name == "MaxPoolPullback":  # mask + pooled gradient read, input gradient written; x and pooled give shapes only
        return _nbytes(ins[2][0], ins[2][1]) + _nbytes(ins[3][0], ins[3][1]) + _nbytes(out_shape, out_dtype), 0
    if name in ("Reshape", "Size", "TupleIndex", "InMemoryData", "Arange"):
        return 0, 0
    if name in ("IncSli", "IncFlatIndices"):  # in place: read the increment and the touched part, write it back
        return 3 * _nbytes(ins[-1][0], ins[-1][1]), 0
    if isinstance(out_shape, tuple) and out_shape and isinstance(out_shape[0], tuple):  # tuple-valued: members at their own dtypes
        dts = getattr(instr, "out_dtypes", None) or [ins[0][1]] * len(out_shape)
        out_b = sum(_nbytes(s, d) for (s, d) in zip(out_shape, dts))
    else:
        out_b = _nbytes(out_shape, out_dtype)
    flops = 0
    if name == "Mul22":
        (sa, _), _ = ins[0], ins[1]
        M, N = out_shape
        K = sa[0] if op.tA else sa[1]
        flops = 2 * M * N * K
    elif name in ("ConvBiasRelu",):
        (M, ld), (C, K) = ins[0][0], ins[1][0]
        flops = 2 * M * C * K
    elif name in ("ConvFwdBiasRelu", "ConvDgrad"):
        (B, H, W, Cs), wshape = ins[0][0], ins[1][0]
        flops = 2 * B * H * W * int(np.prod(wshape))
    elif name in ("ConvWgradImplicit",):
        (B, H, W, Cs), (_b, Ho, Wo, N) = ins[0][0], ins[1][0]
        flops = 2 * B * Ho * Wo * N * int(out_shape[1])
    elif name == "ConvWgrad":
        (M, C), (_m, ld) = ins[0][0], ins[1][0]
        flops = 2 * M * C * int(out_shape[1])
    return in_b + out_b, flops


def step_algorithmic_bytes(f):
    from cgt_b200 import compilation
    total_b, total_f = 0, 0
    for instr in f.eg.instrs:
        if isinstance(instr, compilation._Return) and not getattr(instr, "once", False) and instr.write_loc.devtype == "gpu":
            b, fl = algorithmic_cost(instr)
            total_b += b
            total_f += fl
    return total_b, total_f


# ------------------------------------------------------------------------------------------------
# per-kernel loop: every tensor / stencil entry point of the step through the C ABI at the step's shapes
# ------------------------------------------------------------------------------------------------
def _dev(arr):
    from cgt_b200 import runtime
    return runtime.device_array(np.ascontiguousarray(arr))


def _ptr(w):
    return ctypes.c_void_p(w.data)


def cifar_kernel_table(B=BATCH):
    """[(name, shape string, per-step count, algorithmic bytes, flops, launcher)] of the CIFAR batch-B training step.
    The launchers call the same C-ABI entry points the Ops of the compiled step call, on synthetic operands."""
    from cgt_b200 import runtime
    L = runtime.lib()
    rs = np.random.RandomState(0)
    f4 = runtime._dtype_code(np.dtype("f4"))
    d = ctypes.c_double
    table = []

    def add(name, shape, nbytes, flops, fn):
        table.append(dict(name=name, shape=shape, bytes=int(nbytes), flops=int(flops), fn=fn))

    # conv1: 3 -> 32 channels, 32x32, direct convolution (no column matrix)
    x1 = _dev(rs.randn(B, 3, 32, 32).astype("f4"))
    w1, b1 = _dev((rs.randn(32, 75) * 0.1).astype("f4")), _dev(rs.randn(32).astype("f4"))
    y1, m1 = _dev(np.zeros((B, 32, 1024), "f4")), _dev(np.zeros((B, 32, 1024), "i1"))
    dw1 = _dev(np.zeros((32, 75), "f4"))
    M1 = B * 1024
    add("cgtb_conv_direct_fwd_bias_relu", "conv1 forward %dx3x32x32 * 32x3x5x5 + bias + relu -> NCHW" % B,
        4 * (B * 3 * 1024 + 32 * 75 + 32 + M1 * 32) + M1 * 32, 2 * M1 * 32 * 75,
        lambda: L.cgtb_conv_direct_fwd_bias_relu(_ptr(x1), B, 3, 32, 32, _ptr(w1), 32, 5, 5, 2, 2, _ptr(b1), _ptr(y1), _ptr(m1)))
    g1 = _dev(rs.randn(B, 32, 1024).astype("f4"))
    db1 = _dev(np.zeros((32,), "f4"))
    add("cgtb_conv_direct_wgrad_relu", "conv1 relu gradient + filter gradient 32x75 + bias gradient over %d pixels" % M1,
        4 * (B * 3 * 1024 + M1 * 32 + 32 * 75 + 32) + M1 * 32, 2 * M1 * 32 * 75,
        lambda: L.cgtb_conv_direct_wgrad_relu(_ptr(x1), B, 3, 32, 32, _ptr(m1), _ptr(g1), 32, 5, 5, 2, 2, _ptr(dw1), _ptr(db1)))

    # conv2 / conv3: stride-1 convolutions on 32-channel inputs, without a column matrix
    def conv_layer(tag, Cin, H, Cout):
        HW = H * H
        xn = _dev(rs.randn(B, H, H, Cin).astype("f4"))
        xc = _dev(rs.randn(B, Cin, H, H).astype("f4"))
        wb = _dev((rs.randn(Cout, Cin, 5, 5) * 0.05).astype("f4"))
        bias = _dev(rs.randn(Cout).astype("f4"))
        y, mask = _dev(np.zeros((B, Cout, HW), "f4")), _dev(np.zeros((B, Cout, HW), "i1"))
        dyn = _dev(rs.randn(B, H, H, Cout).astype("f4"))
        dx, dw = _dev(np.zeros((B, Cin, HW), "f4")), _dev(np.zeros((Cout, Cin * 25), "f4"))
        g = _dev(rs.randn(B, Cout, HW).astype("f4"))
        gt, bs = _dev(np.zeros((B, HW, Cout), "f4")), _dev(np.zeros((Cout,), "f4"))
        longs = (ctypes.c_long * 4)(B, Cin, H, H)
        axes = (ctypes.c_int * 4)(0, 2, 3, 1)
        nx, ny, nw = B * Cin * HW, B * Cout * HW, Cout * Cin * 25
        fl = 2 * B * HW * Cout * Cin * 25
        add("cgtb_transpose", "%s input NCHW -> NHWC %dx%dx%dx%d" % (tag, B, Cin, H, H), 8 * nx, 0,
            lambda: L.cgtb_transpose(f4, 4, longs, axes, _ptr(xc), _ptr(xn)))
        add("cgtb_conv_fwd_bias_relu_bank", "%s forward %dx%dx%dx%d * %dx%dx5x5 + bias + relu" % (tag, B, H, H, Cin, Cout, Cin),
            4 * (nx + nw + Cout + ny) + ny, fl,
            lambda: L.cgtb_conv_fwd_bias_relu_bank(_ptr(xn), B, H, H, Cin, _ptr(wb), Cout, H, H, 5, 5, 2, 2, _ptr(bias), _ptr(y), _ptr(mask)))
        add("cgtb_relu_grad_nhwc", "%s relu gradient + NHWC + bias gradient %dx%dx%d" % (tag, B, Cout, HW), ny + 4 * ny + 4 * ny + 4 * Cout, 0,
            lambda: L.cgtb_relu_grad_nhwc(_ptr(mask), _ptr(g), B, Cout, HW, _ptr(gt), _ptr(bs)))
        add("cgtb_conv_dgrad_bank", "%s data gradient %dx%dx%dx%d -> %dx%dx%dx%d" % (tag, B, H, H, Cout, B, Cin, H, H), 4 * (ny + nw + nx), fl,
            lambda: L.cgtb_conv_dgrad_bank(_ptr(dyn), B, H, H, Cout, _ptr(wb), Cin, H, H, 5, 5, 2, 2, _ptr(dx)))
        add("cgtb_conv_wgrad", "%s filter gradient %dx%d over %d pixels" % (tag, Cout, Cin * 25, B * HW), 4 * (nx + ny + nw), fl,
            lambda: L.cgtb_conv_wgrad(_ptr(xn), B, H, H, Cin, _ptr(dyn), H, H, Cout, 5, 5, 2, 2, _ptr(dw)))

    conv_layer("conv2", 32, 15, 32)
    conv_layer("conv3", 32, 6, 64)

    # pooling 3x3 / 2 (three layers), LRN on the first pooled activations, relu gradient of conv1
    def pool(tag, C, H, PH):
        x = _dev(rs.randn(B, C, H, H).astype("f4"))
        top, mask, gx = _dev(np.zeros((B, C, PH, PH), "f4")), _dev(np.zeros((B, C, PH, PH), "i4")), _dev(np.zeros((B, C, H, H), "f4"))
        nin, nout = B * C * H * H, B * C * PH * PH
        add("cgtb_max_pool", "%s %dx%dx%dx%d -> %dx%d" % (tag, B, C, H, H, PH, PH), 4 * nin + 8 * nout, 0,
            lambda: L.cgtb_max_pool(f4, _ptr(x), B, C, H, H, 3, 3, 0, 0, 2, 2, PH, PH, _ptr(top), _ptr(mask)))
        add("cgtb_max_pool_pullback", "%s %dx%dx%dx%d <- %dx%d" % (tag, B, C, H, H, PH, PH), 8 * nout + 4 * nin, 0,
            lambda: L.cgtb_max_pool_pullback(f4, _ptr(mask), _ptr(top), B, C, PH, PH, H, H, 3, 3, 0, 0, 2, 2, _ptr(gx)))

    pool("pool1", 32, 32, 15)
    pool("pool2", 32, 15, 6)
    pool("pool3", 64, 6, 2)
    xl = _dev(rs.randn(B, 32, 15, 15).astype("f4"))
    t, sc, gl = (_dev(np.zeros((B, 32, 15, 15), "f4")) for _ in range(3))
    nl = B * 32 * 225
    add("cgtb_lrn_forward", "LRN(5) %dx32x15x15" % B, 12 * nl, 0,
        lambda: L.cgtb_lrn_forward(f4, _ptr(xl), B, 32, 15, 15, 5, d(1e-4), d(0.75), _ptr(t), _ptr(sc)))
    add("cgtb_lrn_backward", "LRN(5) gradient %dx32x15x15" % B, 20 * nl, 0,
        lambda: L.cgtb_lrn_backward(f4, _ptr(xl), _ptr(t), _ptr(sc), _ptr(xl), B, 32, 15, 15, 5, d(1e-4), d(0.75), _ptr(gl)))
    return table


def measure_kernels(table, launches=200):
    """Median device time of each entry over `launches` cold-L2 launches: flush, event, call, event, all queued
    without a host synchronisation in between (so no launch gap is timed); one synchronisation at the end."""
    from cgt_b200 import runtime
    out = []
    for ent in table:
        for _ in range(3):
            runtime.check(ent["fn"](), ent["name"])
        runtime.synchronize()
        k0 = runtime.kernel_launches()
        runtime.check(ent["fn"](), ent["name"])
        n_kernels = runtime.kernel_launches() - k0
        evs = [(runtime.Event(), runtime.Event()) for _ in range(launches)]
        for (e0, e1) in evs:
            runtime.l2_flush()
            e0.record()
            runtime.check(ent["fn"](), ent["name"])
            e1.record()
        runtime.synchronize()
        ts = np.array([e0.elapsed_ms(e1) * 1e3 for (e0, e1) in evs])
        out.append(dict(name=ent["name"], shape=ent["shape"], us=float(np.median(ts)), us_min=float(ts.min()), kernels=int(n_kernels),
                        bytes=ent["bytes"], flops=ent["flops"]))
    return out


# ------------------------------------------------------------------------------------------------
# timed loops
# ------------------------------------------------------------------------------------------------
def timed_blocks(f, batches, steps, warmup, repeats, flush=True, prefetch=False):
    """`repeats` blocks of `steps` steps after `warmup` steps. Returns (list of block times in device ms, each the max
    over ranks; last loss). Each step: untimed L2 flush, event, step, event. prefetch: inside every timed step the
    NEXT step's batch is handed to f.prefetch before the step is called, so its host->device copy (one per step)
    runs on the copy stream beside the step."""
    from cgt_b200 import parallel, runtime
    nb = len(batches)
    if prefetch:
        f.prefetch(*batches[0])
    for i in range(warmup):
        if prefetch:
            f.prefetch(*batches[(i + 1) % nb])
        f(*batches[i % nb])
    e0, e1 = runtime.Event(), runtime.Event()
    blocks, loss, it = [], None, warmup
    for _ in range(repeats):
        parallel.barrier()
        runtime.synchronize()
        total = 0.0
        for _i in range(steps):
            if flush:
                runtime.l2_flush()
                runtime.synchronize()
            parallel.device_barrier()   # N > 1: the ranks' streams start the step together (outside the timed region)
            e0.record()
            if prefetch:
                f.prefetch(*batches[(it + 1) % nb])
            loss = f(*batches[it % nb])[0]
            e1.record()
            total += e0.elapsed_ms(e1)
            it += 1
        runtime.synchronize()
        parallel.barrier()
        blocks.append(parallel.all_max(total))
    return blocks, float(loss)


def _summary(blocks, n_examples_per_block):
    med = float(np.median(blocks))
    return dict(value=n_examples_per_block / (med / 1e3), ms_block=med,
                spread={"min": n_examples_per_block / (max(blocks) / 1e3), "max": n_examples_per_block / (min(blocks) / 1e3)})


def parity_check(config, steps=3):
    """`steps` update steps from a fresh seed on the GPU and on the CPU oracle: largest relative loss error."""
    from cgt_b200 import configs
    from oracle import cpu_backend, oracle
    build = getattr(configs, CONFIGS[config]["builder"])
    ref, cfg = build(batch=BATCH, seed=7), build(batch=BATCH, seed=7)
    f_cpu = cpu_backend.function(ref.inputs, [ref.loss], updates=ref.updates, impl="ref" if oracle.have_ref() else "port")
    f_gpu = cfg.compile()
    worst = 0.0
    for i in range(steps):
        b = ref.batch(100 + i)
        g, c = float(f_gpu(*b)[0]), float(f_cpu(*b)[0])
        worst = max(worst, abs(g - c) / max(abs(c), 1e-12))
    return {"loss_rel_err": worst, "steps": steps, "against": "CPU oracle (reference kernels where built)", "bar": 1e-3}


def replica_diff(params):
    """max over ranks and parameters of |param - rank 0's param| (0.0 when the replicas stayed identical)."""
    import torch
    import torch.distributed as dist
    worst = 0.0
    for p in params:
        mine = torch.from_numpy(np.ascontiguousarray(p.op.get_value()).copy())
        ref = mine.clone()
        dist.broadcast(ref, src=0)
        worst = max(worst, float((mine - ref).abs().max()))
    t = torch.tensor([worst], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def run_b200(args):
    from cgt_b200 import configs, parallel, runtime
    rank, world = parallel.init_process_group() if int(os.environ.get("WORLD_SIZE", "1")) > 1 else (0, 1)
    if world == 1:
        runtime.ensure_init()
    assert world == args.gpus, "--gpus %d but WORLD_SIZE is %d (launch with torch.distributed.run)" % (args.gpus, world)
    meta = CONFIGS[args.config]
    build = getattr(configs, meta["builder"])
    cfg = build(batch=BATCH, grad_hook=parallel.allreduce_mean)
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
    K, R = args.steps, args.repeats
    dev_blocks, loss = timed_blocks(f, dev_batches, K, args.warmup, R)
    st = f.stats()
    launches = int(st["last_kernel_launches"]) * K * R
    e2e_serial_blocks, _ = timed_blocks(f, host_batches, K, max(3, args.warmup // 4), max(3, R // 3))
    e2e_blocks, _ = timed_blocks(f, host_batches, K, max(3, args.warmup // 4), R, prefetch=True)
    clocks = sampler.stop() if rank == 0 else None
    rdiff = replica_diff(cfg.params) if world > 1 else None
    exchange = None
    if world > 1 and parallel._state["peer"]:
        # the peer-memory all-reduce kernel's own clock (block 0): how long it waited for the slower ranks' flags
        # and how long the whole kernel ran, averaged over all calls of this process
        import ctypes
        t = (ctypes.c_long * 3)()
        if runtime.lib().cgtb_peer_timing(t) == 0 and t[0] > 0:
            exchange = {"kernel": "peer_allreduce_kernel", "calls": int(t[0]), "us_until_all_flags_seen": t[1] / t[0] / 1e3,
                        "us_total": t[2] / t[0] / 1e3}

    out = None
    if rank == 0:
        n_block = BATCH * world * K
        dev, e2e, e2e_serial = _summary(dev_blocks, n_block), _summary(e2e_blocks, n_block), _summary(e2e_serial_blocks, n_block)
        out = {
            "metric": meta["metric"], "value": dev["value"], "unit": UNIT, "n_gpus": world, "steps": K, "repeats": R,
            "warmup": args.warmup, "ms_per_step": dev["ms_block"] / K, "spread": dev["spread"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32 (3xTF32 tensor-core GEMM where used, fp32 elsewhere)",
            "data": "synthetic",
            "config": {"workload": meta["workload"], "global_batch": BATCH * world, "parallelism": "dp%d" % world,
                       "l2": "flushed between timed steps (256 MiB memset, untimed)",
                       "rank_alignment": ("one-float NCCL all-reduce queued before the start event of every timed step (untimed)"
                                          if world > 1 else None), "cuda_graphs": bool(st["segments_captured"]),
                       "timing": "median of %d blocks of %d steps; every block between a barrier and a synchronisation, max over ranks" % (R, K),
                       "kernels_per_step": int(st["last_kernel_launches"]), "graph_launches_per_step": int(st["last_graph_launches"])},
            "e2e": {"value": e2e["value"], "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                    "ms_per_step": e2e["ms_block"] / K, "spread": e2e["spread"],
                    "input_upload": "pinned host batch -> f.prefetch: copied on the copy stream while the step before it runs; one copy per timed step",
                    "value_copy_inside_step": e2e_serial["value"]},
            "gpu_launches": launches, "clocks": clocks, "final_loss": loss,
        }
        if rdiff is not None:
            out["replica_max_abs_diff"] = rdiff
        if exchange is not None:
            out["exchange"] = exchange
    # roofline of the dominant kernel (rank 0; the per-GPU work is the same at every N under weak scaling) and, at
    # N = 1, parity against the CPU oracle and the CPU baseline
    if rank == 0 and not args.no_extras:
        peaks = load_peaks()
        tf32_peak = peaks["bf16_tflops"] / 2.0  # dense TF32 runs at half the bf16 rate on this part
        step_b, step_f = step_algorithmic_bytes(f)
        ms_step = out["ms_per_step"]
        out["step_roofline"] = {"algorithmic_bytes_per_step": step_b, "algorithmic_flops_per_step": step_f,
                                "hbm_floor_ms": step_b / (peaks["hbm_gbs"] * 1e9) * 1e3,
                                "frac": (step_b / (peaks["hbm_gbs"] * 1e9) * 1e3) / ms_step}
        if args.config == "cifar":
            per = measure_kernels(cifar_kernel_table(), launches=args.kernel_launches)
            total_us = sum(k["us"] for k in per)
            for k in per:
                sec = k["us"] * 1e-6
                hbm_floor, tensor_floor = k["bytes"] / (peaks["hbm_gbs"] * 1e9), k["flops"] / (tf32_peak * 1e12)
                k["GB/s"] = k["bytes"] / sec / 1e9
                k["TFLOP/s"] = k["flops"] / sec / 1e12
                k["bound"] = "tensor" if tensor_floor > hbm_floor else "hbm"
                k["frac"] = (k["TFLOP/s"] / tf32_peak) if k["bound"] == "tensor" else (k["GB/s"] / peaks["hbm_gbs"])
                k["share"] = k["us"] / total_us
            dom = max(per, key=lambda k: k["us"])
            out["roofline"] = {
                "bound": dom["bound"], "achieved": dom["TFLOP/s"] if dom["bound"] == "tensor" else dom["GB/s"],
                "peak": tf32_peak if dom["bound"] == "tensor" else peaks["hbm_gbs"],
                "unit": "TFLOP/s" if dom["bound"] == "tensor" else "GB/s", "frac": dom["frac"], "kernel": dom["name"], "shape": dom["shape"],
                "us_per_launch": dom["us"], "algorithmic_bytes": dom["bytes"], "algorithmic_flops": dom["flops"],
                "traffic": NCU_TRAFFIC.get(dom["name"]), "traffic_note": NCU_TRAFFIC_NOTE.get(dom["name"]),
                "peak_source": peaks["source"], "share_of_listed_kernels": dom["share"],
                "timing": "median of %d cold-L2 launches through the C ABI, CUDA events on the launching stream" % args.kernel_launches,
                "tf32_peak_note": "dense TF32 peak taken as half of the measured bf16 peak; 3xTF32 issues three tensor MACs per algorithmic MAC",
            }
            out["per_kernel"] = [{"name": k["name"], "shape": k["shape"], "us": round(k["us"], 2), "kernels": k["kernels"], "bytes": k["bytes"],
                                  "GB/s": round(k["GB/s"], 1), "TFLOP/s": round(k["TFLOP/s"], 2), "bound": k["bound"],
                                  "frac": round(k["frac"], 4), "share": round(k["share"], 4)} for k in sorted(per, key=lambda k: -k["us"])]
        if world == 1:
            out["parity"] = parity_check(args.config)
            if args.config == "cifar":
                out["cpu_baseline"] = cpu_baseline(sample_steps=5, warmup=2)
    parallel.barrier()
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        parallel.shutdown()


# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum, bytes per launch) of an entry point's main kernel from an
# ncu capture (--set full, cold launches) at the shape listed in `per_kernel`.
NCU_TRAFFIC = {
    "cgtb_conv_wgrad": 7418112 + 1024,
    "cgtb_conv_fwd_bias_relu_bank": 3941888,
    "cgtb_conv_direct_fwd_bias_relu": 1626368,
}
NCU_TRAFFIC_NOTE = {
    "cgtb_conv_direct_fwd_bias_relu": "conv_direct_fwd_kernel at the CIFAR conv1 shape, one cold launch under ncu --set full: the "
                                      "image is read from DRAM once; the 21 MB of results had not left L2 when the launch ended",
    "cgtb_conv_wgrad": "sgemm_tma_kernel<1,1,2> at the conv2 shape, one cold launch under ncu --set full: every operand "
                       "byte is read from DRAM once; the 0.1 MB result had not left L2 when the launch ended",
    "cgtb_conv_fwd_bias_relu_bank": "conv_tsa_kernel at the conv2 shape, one cold launch under ncu --set full: the input "
                                    "is read once; the 4.6 MB of results had not left L2 when the launch ended",
}


# ------------------------------------------------------------------------------------------------
# CPU arm: the reference's CPU implementation of the path (its own im2col.h / pooling.h / lrn.cuh-as-C++
# when oracle/_ref is built, restated loops otherwise, OpenBLAS sgemm on all host cores)
# ------------------------------------------------------------------------------------------------
def _cpu_function(batch, config="cifar"):
    import cgt_b200  # noqa: F401  (graph front-end only; nothing is placed on a GPU here)
    from cgt_b200 import configs
    from oracle import cpu_backend, oracle
    cfg = getattr(configs, CONFIGS[config]["builder"])(batch=batch)
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
    meta = CONFIGS[args.config]
    cfg, f, kind = _cpu_function(BATCH, args.config)
    b = cfg.batch(0)
    t0 = time.perf_counter()
    f(*b)
    t1 = time.perf_counter() - t0
    batch = BATCH
    total_steps = args.steps + args.warmup
    if t1 * total_steps > budget_s:  # bounded sample: a smaller batch per step, same network
        batch = int(max(1, min(BATCH, BATCH * budget_s / (t1 * total_steps))))
        cfg, f, kind = _cpu_function(batch, args.config)
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
        "impl": "reference", "metric": meta["metric"], "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": meta["workload"] + " on the host cores", "batch_per_step": batch},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": os.cpu_count(), "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "final_loss": float(loss),
    }
    print(json.dumps(out))


def run_only_kernel(args):
    from cgt_b200 import runtime
    runtime.ensure_init(0)
    table = [e for e in cifar_kernel_table() if args.only_kernel in e["name"] or args.only_kernel in e["shape"]]
    if not table:
        raise SystemExit("no entry of the per-kernel list matches %r" % args.only_kernel)
    for k in measure_kernels(table, launches=args.kernel_launches):
        print(json.dumps({"name": k["name"], "shape": k["shape"], "us_median": round(k["us"], 2), "us_min": round(k["us_min"], 2),
                          "kernels_per_call": k["kernels"], "algorithmic_bytes": k["bytes"], "algorithmic_flops": k["flops"],
                          "launches": args.kernel_launches}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--repeats", type=int, default=15, help="timed blocks of --steps steps; the median block is reported")
    ap.add_argument("--kernel-launches", type=int, default=200, help="cold-L2 launches per entry of the per-kernel list")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--config", default="cifar", choices=sorted(CONFIGS))
    ap.add_argument("--no-extras", action="store_true", help="skip the per-kernel loop, parity and the CPU baseline (for ncu runs)")
    ap.add_argument("--only-kernel", default=None, metavar="TEXT",
                    help="run only the entries of the per-kernel list whose name or shape contains TEXT, --kernel-launches "
                         "times each on one GPU, print their times and exit (the command that ncu captures wrap)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    args.repeats = max(args.repeats, 1)
    if args.only_kernel is not None:
        run_only_kernel(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
