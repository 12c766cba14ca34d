from .distributed import run_distributed_test
from .utils import allclose, rel_err
