"""Builds ``cgt_b200/libcgt_b200.so`` in-tree with nvcc for sm_100a.

One object file per source under ``csrc/``, rebuilt only when the source or a header is newer, then
one link step. ``python -m cgt_b200.build`` forces nothing; pass ``--force`` to rebuild everything.
"""
import concurrent.futures
import glob
import os
import os.path as osp
import subprocess
import sys

HERE = osp.dirname(osp.abspath(__file__))
CSRC = osp.join(HERE, "csrc")
INCLUDE = osp.join(HERE, "..", "include")
OBJDIR = osp.join(HERE, "csrc", "build")
LIB = osp.join(HERE, "libcgt_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
    "-I" + INCLUDE,
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (osp.exists(cand) or cand == "nvcc"):
            return cand
    raise RuntimeError("nvcc not found")


def _deps():
    return glob.glob(osp.join(CSRC, "*.h")) + glob.glob(osp.join(INCLUDE, "*.h"))


def _stale(target, sources):
    if not osp.exists(target):
        return True
    t = osp.getmtime(target)
    return any(osp.getmtime(s) > t for s in sources)


def build(force=False, verbose=False):
    os.makedirs(OBJDIR, exist_ok=True)
    nvcc = _nvcc()
    srcs = sorted(glob.glob(osp.join(CSRC, "*.cu")))
    deps = _deps()
    jobs = []
    objs = []
    for src in srcs:
        obj = osp.join(OBJDIR, osp.basename(src)[:-3] + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + deps):
            extra = os.environ.get("CGTB_NVCC_EXTRA", "").split()  # e.g. -DCGTB_TMA_TRACE for a tracing build
            cmd = [nvcc] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
            jobs.append(cmd)

    def run(cmd):
        p = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, p.returncode, p.stdout + p.stderr

    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for cmd, rc, out in ex.map(run, jobs):
                if verbose or rc != 0:
                    sys.stderr.write(" ".join(cmd) + "\n" + out + "\n")
                if rc != 0:
                    raise RuntimeError("nvcc failed for %s" % cmd[-3])
    if jobs or not osp.exists(LIB):
        cmd = [nvcc, "-shared", "-o", LIB] + objs + ["-lcudart", "-ldl", "-lpthread"]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            sys.stderr.write(p.stdout + p.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
