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
    # No collective here: every rank plans from the metadata and reads on its own, so a subset of the
    # job's ranks may load (onto a mesh of their own) while the others do something else -- the
    # reference's resharding test loads on ranks 0-3 of an 8-rank job.  Callers that overwrite the
    # checkpoint right after loading synchronise themselves.


class AsyncSaveHandle:
    """Result of :func:`async_save`; ``wait()`` returns the metadata (and re-raises a write error)."""

    def __init__(self, thread, box):
        self._thread, self._box = thread, box

    def done(self) -> bool:
        return not self._thread.is_alive()

    def wait(self) -> Metadata:
        self._thread.join()
        if "error" in self._box:
            raise self._box["error"]
        return self._box["metadata"]


def async_save(state_dict: Dict[str, Any], *, checkpoint_id=None, storage_writer: Optional[StorageWriter] = None,
               planner: Optional[SavePlanner] = None) -> AsyncSaveHandle:
    """Checkpoint without stalling the training loop (the reference only saves synchronously).

    Every tensor is first copied to host memory (pinned for CUDA tensors, on a side stream that the
    call waits for, so the caller may overwrite the parameters as soon as this returns); the files
    are then written by a background thread.  The thread must not issue collectives next to the
    training loop's, so each rank plans and writes on its own (``.rank{r}_metadata``, the layout of
    ``save(use_collectives=False)``), which ``load`` reads on any number of ranks.
    """
    import threading

    import torch

    from ..dtensor import DTensor

    def stage(t):
        local = t.to_local() if isinstance(t, DTensor) else t
        if local.is_cuda:
            host = torch.empty(local.shape, dtype=local.dtype, device="cpu", pin_memory=True)
            host.copy_(local.detach(), non_blocking=True)
        else:
            host = local.detach().clone()
        return DTensor._wrap(host, t.layout) if isinstance(t, DTensor) else host

    side = None
    if torch.cuda.is_available() and any(
            (v.to_local() if isinstance(v, DTensor) else v).is_cuda for v in state_dict.values()
            if isinstance(v, torch.Tensor)):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
    staged: Dict[str, Any] = {}
    ctx = torch.cuda.stream(side) if side is not None else None
    if ctx is not None:
        ctx.__enter__()
    try:
        for k, v in state_dict.items():
            staged[k] = stage(v) if isinstance(v, torch.Tensor) else v
    finally:
        if ctx is not None:
            ctx.__exit__(None, None, None)
    if side is not None:
        side.synchronize()
    box: Dict[str, Any] = {}

    def work():
        try:
            box["metadata"] = save(staged, checkpoint_id=checkpoint_id, storage_writer=storage_writer,
                                   planner=planner, use_collectives=False)
        except BaseException as e:  # noqa: BLE001 - re-raised by wait()
            box["error"] = e

    th = threading.Thread(target=work, name="hpb-async-save", daemon=True)
    th.start()
    return AsyncSaveHandle(th, box)
