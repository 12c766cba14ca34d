from . import ocdbt, orbax_layout
from .utils import (
    AsyncSaveHandle,
    get_metadata,
    restore,
    restore_from_metadata,
    restore_sharded,
    save,
    save_sharded,
)
