from . import collectives, dist_utils
from .dist_utils import (
    DistConfig,
    allgather_value,
    barrier,
    get_global_device_count,
    get_local_device_count,
    get_local_rank,
    get_process_filesystem_rank,
    get_rank,
    get_reduce_divide_factor,
    get_world_size,
    init_distributed,
    is_distributed,
    synchronize_array,
    synchronize_value,
    teardown_distributed,
)
from .mesh import (
    ContextParallelConfig,
    DataParallelConfig,
    DataParallelType,
    DeviceMesh,
    ExpertParallelConfig,
    MeshResource,
    PipelineParallelConfig,
    TensorParallelConfig,
    TPStyle,
    get_mesh,
    set_mesh,
    shard_map,
)
from .context import (CPStrategy, context_parallel_attention, cp_local_positions,
                      inverse_reorder_causal_load_balancing, reorder_causal_load_balancing, shard_sequence_for_cp)
from .param_store import FSDPUnit, ParamHandle, ParamMeta, ParamStore
