"""Helpers to run a function as N CPU ranks (gloo) in child processes."""
import os
import socket
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn, args, errq):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    try:
        torch.set_num_threads(1)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        fn(rank, world, *args)
        dist.barrier()
    except Exception:  # noqa: BLE001
        errq.put((rank, traceback.format_exc()))
        raise
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def run_distributed(fn, world_size: int, *args, timeout: float = 240.0):
    """Run ``fn(rank, world_size, *args)`` on ``world_size`` gloo ranks; raise on any failure."""
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world_size, port, fn, args, errq)) for r in range(world_size)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    failed = []
    for r, p in enumerate(procs):
        if p.is_alive():
            p.kill()
            failed.append(f"rank {r}: timeout")
        elif p.exitcode != 0:
            failed.append(f"rank {r}: exit code {p.exitcode}")
    msgs = []
    while not errq.empty():
        msgs.append("rank %d:\n%s" % errq.get())
    if failed or msgs:
        raise AssertionError("distributed run failed: " + "; ".join(failed) + "\n" + "\n".join(msgs))
