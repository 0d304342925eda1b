"""cgt_b200: a B200 (sm_100a) execution backend behind the operator API of the Computation Graph
Toolkit. The module namespace plays the role of the reference's ``cgt`` package: symbolic API,
``function``, ``grad``, configuration.
"""
import sys as _sys

from . import core, utils
from . import api as _api

floatX = "f4"
complexX = "c8"

core.cgt = _sys.modules[__name__]
_api.cgt = _sys.modules[__name__]

from .api import *  # noqa: F401,F403,E402
from .api import (abs, max, sum, shape, size, scalar, vector, matrix, tensor3, tensor4, tensor)  # noqa: F401,E402
from .core import (grad, get_config, update_config, simplify, reset_config, Device, scoped_update_config,  # noqa: E402
                   infer_shape, count_nodes)
from .compilation import function, numeric_eval, profiler  # noqa: E402
from . import nn, distributions  # noqa: E402
from .checkpoint import save_state, load_state, state_variables, ParamCollection  # noqa: E402,F401

get_config()
