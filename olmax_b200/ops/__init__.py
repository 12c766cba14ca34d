"""sm_100a kernels (``kernels``), the differentiable ops built on them (``functional``) and the PyTorch restatement
used as oracle and CPU path (``reference``)."""
from . import reference
