"""Planner interfaces and plan records (hyper_parallel/core/checkpoint/planner.py:26-318)."""
from __future__ import annotations

import enum
from abc import ABC, abstractmethod
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .metadata import ChunkStorageMetadata, Metadata, MetadataIndex, TensorProperties


class WriteItemType(enum.Enum):
    TENSOR = "tensor"
    BYTE_IO = "byte_io"


class LoadItemType(enum.Enum):
    TENSOR = "tensor"
    BYTE_IO = "byte_io"


@dataclass(frozen=True)
class TensorWriteData:
    chunk: ChunkStorageMetadata
    properties: TensorProperties
    size: tuple


@dataclass(frozen=True)
class WriteItem:
    index: MetadataIndex
    type: WriteItemType
    tensor_data: Optional[TensorWriteData] = None
    # bytes (or any picklable object) a planner attaches to a BYTE_IO item itself, as the reference's
    # planner does; without it the writer asks ``planner.resolve_data``
    bytes_io_data: Any = field(default=None, compare=False, hash=False)


@dataclass
class SavePlan:
    items: List[WriteItem] = field(default_factory=list)
    storage_data: Any = None
    planner_data: Any = None
    rank: int = 0


@dataclass(frozen=True)
class ReadItem:
    type: LoadItemType
    dest_index: MetadataIndex            # which entry of the state_dict
    dest_offsets: tuple                  # where inside the destination local tensor
    storage_index: MetadataIndex         # which saved chunk
    storage_offsets: tuple               # where inside the saved chunk
    lengths: tuple


@dataclass
class LoadPlan:
    items: List[ReadItem] = field(default_factory=list)
    storage_data: Any = None
    planner_data: Any = None


class SavePlanner(ABC):
    @abstractmethod
    def set_up_planner(self, state_dict: Dict[str, Any], is_coordinator: bool = False, **kw) -> None: ...

    @abstractmethod
    def create_local_plan(self) -> SavePlan: ...

    @abstractmethod
    def create_global_plan(self, all_plans: List[SavePlan]): ...

    @abstractmethod
    def finish_plan(self, new_plan: SavePlan) -> SavePlan: ...

    @abstractmethod
    def resolve_data(self, write_item: WriteItem): ...


class LoadPlanner(ABC):
    @abstractmethod
    def set_up_planner(self, state_dict: Dict[str, Any], metadata: Optional[Metadata] = None,
                       is_coordinator: bool = False, **kw) -> None: ...

    @abstractmethod
    def create_local_plan(self) -> LoadPlan: ...

    @abstractmethod
    def create_global_plan(self, all_plans: List[LoadPlan]) -> List[LoadPlan]: ...

    @abstractmethod
    def finish_plan(self, new_plan: LoadPlan) -> LoadPlan: ...

    @abstractmethod
    def load_bytes(self, read_item: ReadItem, value: Any) -> None: ...

    @abstractmethod
    def resolve_tensor(self, read_item: ReadItem): ...

    @abstractmethod
    def commit_tensor(self, read_item: ReadItem, tensor) -> None: ...
