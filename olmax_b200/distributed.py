"""Alias of :mod:`olmax_b200.parallel` under the reference's package name (``olmax.distributed``)."""
from .parallel import *  # noqa: F401,F403
from .parallel import collectives, dist_utils, mesh, param_store  # noqa: F401
