"""``save`` / ``load`` of sharded state dicts (hyper_parallel/core/checkpoint/api.py:53-268).

``save``: local plan -> ``all_gather_object`` of the plans -> every rank derives the same global
plan (replica de-duplication, chunk indices, metadata) -> each rank writes its files -> the write
results are gathered -> rank 0 writes ``.metadata``.  ``load`` works in place: every rank reads
the metadata, intersects its own chunks with the saved ones and copies the overlaps, so a
checkpoint written on N ranks loads on any other number of ranks / layout.
With ``use_collectives=False`` each rank plans and writes on its own (``.rank{r}_metadata``).
"""
from __future__ import annotations

from typing import Any, Dict, Optional

from ...collectives import cc
from .filesystem_storage import FileSystemReader, FileSystemWriter
from .metadata import Metadata
from .planner import LoadPlanner, SavePlanner
from .standard_planner import StandardLoadPlanner, StandardSavePlanner
from .storage import StorageReader, StorageWriter


def _gather(obj, no_dist: bool):
    if no_dist or not cc.is_initialized():
        return [obj]
    return cc.all_gather_object(obj)


def save(state_dict: Dict[str, Any], *, checkpoint_id=None, storage_writer: Optional[StorageWriter] = None,
         planner: Optional[SavePlanner] = None, no_dist: bool = False, use_collectives: bool = True,
         remove_redundancy: bool = True, save_to_minimum_rank: bool = False) -> Metadata:
    """Write ``state_dict`` (DTensors, tensors, arbitrary picklable objects) to ``checkpoint_id``."""
    if not isinstance(state_dict, dict):
        raise TypeError(f"state_dict must be a dict, got {type(state_dict)}")
    dist_on = cc.is_initialized() and not no_dist
    rank = cc.get_rank() if dist_on else 0
    collectives = use_collectives and dist_on
    writer = storage_writer or FileSystemWriter()
    writer.initialize_writer(checkpoint_id)
    writer.configure_writer(is_coordinator=(rank == 0), rank=rank, use_collectives=use_collectives or not dist_on)
    planner = planner or StandardSavePlanner(remove_redundancy and collectives, save_to_minimum_rank)
    planner.set_up_planner(state_dict, is_coordinator=(rank == 0), rank=rank)
    local_plan = writer.optimize_local_plan(planner.create_local_plan())
    if collectives:
        all_plans = _gather(local_plan, no_dist)
        global_plans, metadata = planner.create_global_plan(all_plans)
        global_plans = writer.optimize_global_plan(global_plans)
        my_plan = planner.finish_plan(global_plans[rank])
        results = writer.execute_write(my_plan, planner)
        all_results = _gather(results, no_dist)
        writer.finalize_checkpoint(metadata, all_results)
        if dist_on:
            import torch.distributed as dist
            dist.barrier()
        return metadata
    local_plan.rank = rank
    plans, metadata = planner.create_global_plan([local_plan])
    # keep this rank's real index in the plan so that file names carry it
    my_plan = planner.finish_plan(plans[0])
    results = writer.execute_write(my_plan, planner)
    writer.finalize_checkpoint(metadata, [results])
    return metadata


def load(state_dict: Dict[str, Any], *, checkpoint_id=None, storage_reader: Optional[StorageReader] = None,
         planner: Optional[LoadPlanner] = None, no_dist: bool = False, use_collectives: bool = True) -> None:
    """Fill ``state_dict`` in place from ``checkpoint_id`` (resharding as needed)."""
    if not isinstance(state_dict, dict):
        raise TypeError(f"state_dict must be a dict, got {type(state_dict)}")
    dist_on = cc.is_initialized() and not no_dist
    rank = cc.get_rank() if dist_on else 0
    reader = storage_reader or FileSystemReader()
    reader.initialize_reader(checkpoint_id)
    try:
        metadata = reader.load_metadata()
    except FileNotFoundError:
        metadata = reader.load_metadata(rank=rank)      # rank-local metadata (use_collectives=False save)
    reader.configure_reader(metadata, is_coordinator=(rank == 0), rank=rank)
    planner = planner or StandardLoadPlanner()
    planner.set_up_planner(state_dict, metadata, is_coordinator=(rank == 0))
    plan = reader.optimize_local_plan(planner.create_local_plan())
    plan = planner.finish_plan(plan)
    reader.execute_read(plan, planner)
    if dist_on and use_collectives:
        import torch.distributed as dist
        dist.barrier()
