"""TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Build recipe for the two CPU checker libraries:

* ``oracle/liboracle.so``      -- the restatement in ``cgt_oracle.cpp`` (always built);
* ``oracle/_ref/libcgt_ref.so`` -- the reference's own headers behind ``ref_shim.cpp``, compiled from
  the reference tree where it lies (only when that tree is present; nothing is copied).

Both are compiled with ``-ffp-contract=off`` so that no fused multiply-add changes the rounding.
Run as ``python oracle/build_oracle.py [reference_root]``.
"""
import os
import os.path as osp
import subprocess
import sys

HERE = osp.dirname(osp.abspath(__file__))
CXXFLAGS = ["-O2", "-ffp-contract=off", "-fPIC", "-shared", "-fvisibility=hidden"]


def _newer(target, sources):
    if not osp.exists(target):
        return False
    t = osp.getmtime(target)
    return all(osp.getmtime(s) <= t for s in sources)


def build_restatement(force=False):
    src = osp.join(HERE, "cgt_oracle.cpp")
    hdr = osp.join(HERE, "..", "include", "cgt_b200_ops.h")
    out = osp.join(HERE, "liboracle.so")
    if force or not _newer(out, [src, hdr]):
        subprocess.check_call(["g++", "-std=c++17"] + CXXFLAGS + [src, "-o", out])
    return out


def default_reference_root():
    """The reference checkout: $CGT_REFERENCE_ROOT, else a directory `reference` beside this repository."""
    env = os.environ.get("CGT_REFERENCE_ROOT")
    if env:
        return env
    return osp.join(osp.dirname(osp.dirname(HERE)), "reference")


def build_reference(reference_root=None, force=False):
    """Returns the path of the built library, or None when the reference tree is absent."""
    if reference_root is None:
        reference_root = default_reference_root()
    inc = osp.join(reference_root, "include")
    common = osp.join(reference_root, "src", "cgt_common.cpp")
    if not (osp.isdir(inc) and osp.exists(common)):
        return None
    outdir = osp.join(HERE, "_ref")
    os.makedirs(outdir, exist_ok=True)
    src = osp.join(HERE, "ref_shim.cpp")
    out = osp.join(outdir, "libcgt_ref.so")
    if force or not _newer(out, [src]):
        subprocess.check_call(["g++", "-std=c++11"] + CXXFLAGS + ["-DNDEBUG", "-I" + inc, src, common, "-o", out])
    return out


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else default_reference_root()
    print(build_restatement(force=True))
    print(build_reference(root, force=True))
