"""Log-likelihood helpers (counterpart of the reference's cgt/distributions.py)."""
from . import core


class Distribution(object):
    def loglik(self, x, p):
        raise NotImplementedError


class _Categorical(Distribution):
    def crossent(self, p, q):
        assert p.ndim == 2 and q.ndim == 2
        return -(p * core.cgt.log(q)).sum(axis=1)

    def loglik(self, labels, p):
        """log p[i, labels[i]] through flat indexing (cgt/distributions.py:28-29)."""
        cgt = core.cgt
        return cgt.log(p[cgt.arange(cgt.size(labels, 0)), labels])


categorical = _Categorical()
