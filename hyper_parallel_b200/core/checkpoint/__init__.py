from .api import AsyncSaveHandle, async_save, load, save  # noqa: F401
from .filesystem_storage import FileSystemReader, FileSystemWriter  # noqa: F401
from .layout import combine_layout, get_current_layout, get_global_layout, load_layout, save_layout  # noqa: F401
from .loader import load_checkpoint  # noqa: F401
from .metadata import (BytesStorageMetadata, ChunkStorageMetadata, Metadata, MetadataIndex,  # noqa: F401
                       TensorProperties, TensorStorageMetadata)
from .planner import (LoadItemType, LoadPlan, LoadPlanner, ReadItem, SavePlan, SavePlanner, WriteItem,  # noqa: F401
                      WriteItemType)
from .reshard import ReshardHandler, infer_intersection, infer_slice_area_by_rank  # noqa: F401
from .saver import save_checkpoint  # noqa: F401
from .standard_planner import StandardLoadPlanner, StandardSavePlanner  # noqa: F401
from .storage import StorageInfo, StorageReader, StorageWriter, WriteResult  # noqa: F401
