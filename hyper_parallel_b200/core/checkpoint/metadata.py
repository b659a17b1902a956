"""Checkpoint metadata records.

Field-for-field the records of hyper_parallel/core/checkpoint/metadata.py:20-102 of the
reference (version ``"1.0"``), so that ``.metadata`` files interchange: ``MetadataIndex(fqn,
offset, index)``, ``ChunkStorageMetadata(offsets, sizes)``, ``TensorProperties(dtype str,
requires_grad, memory_format)``, ``TensorStorageMetadata(properties, size, chunks)``,
``BytesStorageMetadata``, ``Metadata(state_dict_metadata, planner_data, storage_data, version)``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Union


@dataclass(frozen=True)
class MetadataIndex:
    fqn: str
    offset: tuple = field(default_factory=tuple)
    index: Optional[int] = None


@dataclass(frozen=True)
class ChunkStorageMetadata:
    offsets: tuple
    sizes: tuple


@dataclass(frozen=True)
class TensorProperties:
    dtype: str
    requires_grad: bool = False
    memory_format: Optional[str] = None


@dataclass
class BytesStorageMetadata:
    pass


@dataclass(frozen=True)
class TensorStorageMetadata:
    properties: TensorProperties
    size: tuple
    chunks: List[ChunkStorageMetadata] = field(default_factory=list)


@dataclass
class Metadata:
    state_dict_metadata: Dict[str, Union[TensorStorageMetadata, BytesStorageMetadata]]
    planner_data: Any = None
    storage_data: Optional[Dict[MetadataIndex, Any]] = None
    version: str = "1.0"
