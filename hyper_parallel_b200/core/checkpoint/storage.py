"""Storage interfaces (hyper_parallel/core/checkpoint/storage.py)."""
from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import List, Optional

from .metadata import Metadata, MetadataIndex
from .planner import LoadPlan, LoadPlanner, SavePlan, SavePlanner

_metadata_file_name = ".metadata"


@dataclass
class StorageInfo:
    relative_path: str
    offset: int = 0
    length: int = -1


@dataclass
class WriteResult:
    index: MetadataIndex
    size_in_bytes: int
    storage_data: StorageInfo


class StorageWriter(ABC):
    @abstractmethod
    def initialize_writer(self, checkpoint_id) -> None: ...

    @abstractmethod
    def configure_writer(self, is_coordinator: bool, rank: int, use_collectives: bool = True) -> None: ...

    @abstractmethod
    def optimize_local_plan(self, plan: SavePlan) -> SavePlan: ...

    @abstractmethod
    def optimize_global_plan(self, plans: List[SavePlan]) -> List[SavePlan]: ...

    @abstractmethod
    def execute_write(self, plan: SavePlan, planner: SavePlanner) -> List[WriteResult]: ...

    @abstractmethod
    def finalize_checkpoint(self, metadata: Metadata, results: List[List[WriteResult]]) -> None: ...


class StorageReader(ABC):
    @abstractmethod
    def initialize_reader(self, checkpoint_id) -> None: ...

    @abstractmethod
    def load_metadata(self, rank: Optional[int] = None) -> Metadata: ...

    @abstractmethod
    def configure_reader(self, metadata: Metadata, is_coordinator: bool, rank: int = 0) -> None: ...

    @abstractmethod
    def optimize_local_plan(self, plan: LoadPlan) -> LoadPlan: ...

    @abstractmethod
    def optimize_global_plan(self, plans: List[LoadPlan]) -> List[LoadPlan]: ...

    @abstractmethod
    def execute_read(self, plan: LoadPlan, planner: LoadPlanner) -> None: ...
