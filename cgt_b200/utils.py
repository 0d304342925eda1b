"""Small helpers shared by the graph core (counterpart of the reference's cgt/utils.py)."""
import hashlib
import sys
import time

import numpy as np


def warn(msg):
    sys.stderr.write("\x1b[33m%s\x1b[0m\n" % msg)


def error(msg):
    sys.stderr.write("\x1b[31m%s\x1b[0m\n" % msg)


def is_singleton(x):
    return isinstance(x, np.ndarray) and int(np.prod(x.shape)) == 1


def safezip(x, y):
    x, y = list(x), list(y)
    assert len(x) == len(y)
    return list(zip(x, y))


def safezip3(x, y, z):
    x, y, z = list(x), list(y), list(z)
    assert len(x) == len(y) == len(z)
    return list(zip(x, y, z))


def invert_perm(x):
    return [int(i) for i in np.argsort(x)]


def hash_seq1(*args):
    h = hashlib.md5()
    for a in args:
        h.update(a.encode() if isinstance(a, str) else a)
    return h.hexdigest()


class Message(object):
    """``with Message("compiling"):`` prints the elapsed time of the block."""
    depth = 0

    def __init__(self, msg):
        self.msg = msg

    def __enter__(self):
        sys.stderr.write("\t" * Message.depth + "=: " + self.msg + "\n")
        self.tstart = time.time()
        Message.depth += 1

    def __exit__(self, etype, *args):
        Message.depth -= 1
        maybe_exc = "" if etype is None else " (with exception)"
        sys.stderr.write("\t" * Message.depth + "done%s in %.3f seconds\n" % (maybe_exc, time.time() - self.tstart))
