from .callback import Callback
from .console import JSONLMetricsCallback
from .profiler import ProfilerCallback
