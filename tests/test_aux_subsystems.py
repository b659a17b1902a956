"""Auxiliary subsystems on CPU: heartbeat failure detection with host-made failures (a rank that
stops taking part between steps), a short process-group timeout ending a collective with an error,
resume after the loss of a rank on fewer ranks from a distributed checkpoint, metrics / tracing."""
import datetime
import json
import os
import time

import pytest
import torch
import torch.distributed as dist
from torch import nn

from dist_utils import _free_port


def _spawn(fn, world, *args):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    port = _free_port()
    q = ctx.SimpleQueue()
    procs = [ctx.Process(target=fn, args=(r, world, port, q) + args) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    out = {}
    while not q.empty():
        k, v = q.get()
        out[k] = v
    for p in procs:
        if p.is_alive():
            p.kill()
            raise AssertionError("worker did not finish")
    return out, [p.exitcode for p in procs]


def _hb_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    from hyper_parallel_b200.utils.failure import Heartbeat
    hb = Heartbeat()
    t = torch.ones(1)
    dead = []
    for step in range(40):
        if rank == 2 and step == 3:
            # host-made failure: this rank leaves between steps, with no collective in flight
            q.put((f"left{rank}", step))
            os._exit(0)
        hb.beat()
        dead = hb.dead_ranks(timeout=0.6)
        if dead:
            break                              # the survivors learn of it on the host, before the next collective
        if step < 3:
            dist.all_reduce(t)                 # the job makes progress while everybody is alive
        time.sleep(0.1)
    q.put((f"dead{rank}", dead))
    time.sleep(1.5)                            # rank 0 hosts the store: let the others finish reading it
    os._exit(0)                                # no collective teardown with a missing rank


def test_heartbeat_detects_a_rank_that_left_between_steps():
    out, codes = _spawn(_hb_worker, 3)
    assert out["left2"] == 3
    assert out["dead0"] == [2] and out["dead1"] == [2]


def _timeout_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=2))
    t = torch.ones(1)
    dist.all_reduce(t)
    if rank == 1:
        time.sleep(6)                          # never joins the second collective in time
        os._exit(0)
    try:
        dist.all_reduce(t)
        q.put((f"r{rank}", "no error"))
    except Exception as e:  # noqa: BLE001
        q.put((f"r{rank}", type(e).__name__))
    os._exit(0)


def test_short_process_group_timeout_ends_the_collective_with_an_error():
    out, _ = _spawn(_timeout_worker, 2)
    assert out["r0"] != "no error"


class _Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.a = nn.Linear(8, 16, bias=False)
        self.b = nn.Linear(16, 4, bias=False)

    def forward(self, x):
        return self.b(torch.relu(self.a(x)))


def _save_worker(rank, world, port, q, ckpt):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from hyper_parallel_b200 import Layout, distribute_tensor
    from hyper_parallel_b200.core import checkpoint as dcp
    torch.manual_seed(7)
    net = _Net()
    lay = Layout((world,), ("dp",))
    sd = {"a.weight": distribute_tensor(net.a.weight.detach(), lay("dp", "None")),
          "b.weight": distribute_tensor(net.b.weight.detach(), lay("None", "dp")), "step": 12}
    dcp.save(sd, checkpoint_id=ckpt)
    dist.barrier()
    dist.destroy_process_group()


def _resume_worker(rank, world, port, q, ckpt):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from hyper_parallel_b200 import Layout, distribute_tensor
    from hyper_parallel_b200.core import checkpoint as dcp
    lay = Layout((world,), ("dp",))
    sd = {"a.weight": distribute_tensor(torch.zeros(16, 8), lay("dp", "None")),
          "b.weight": distribute_tensor(torch.zeros(4, 16), lay("None", "dp")), "step": 0}
    dcp.load(sd, checkpoint_id=ckpt)
    torch.manual_seed(7)
    ref = _Net()
    ok = torch.allclose(sd["a.weight"].full_tensor(), ref.a.weight.detach()) and \
        torch.allclose(sd["b.weight"].full_tensor(), ref.b.weight.detach()) and sd["step"] == 12
    q.put((f"ok{rank}", bool(ok)))
    dist.barrier()
    dist.destroy_process_group()


def test_resume_on_fewer_ranks_after_a_rank_loss(tmp_path):
    ckpt = str(tmp_path / "ckpt")
    _, codes = _spawn(_save_worker, 4, ckpt)
    assert codes == [0, 0, 0, 0]
    # a rank is gone: the job restarts on 3... the shapes divide by 2, so on 2 ranks
    out, codes = _spawn(_resume_worker, 2, ckpt)
    assert codes == [0, 0] and out == {"ok0": True, "ok1": True}
    # a missing shard file is reported, not silently ignored
    victim = [f for f in os.listdir(ckpt) if f.startswith("_rank1_")][0]
    os.remove(os.path.join(ckpt, victim))
    out, codes = _spawn(_resume_worker, 2, ckpt)
    assert any(c != 0 for c in codes)


def test_metrics_writer_and_layer_timer(tmp_path):
    from hyper_parallel_b200.utils.logging import MetricsWriter, get_logger
    from hyper_parallel_b200.utils.tracing import CudaTimer, LayerTimer, nvtx_range
    path = str(tmp_path / "m" / "metrics.jsonl")
    w = MetricsWriter(path)
    w.write(1, tokens_per_s=123.0, loss=torch.tensor(2.5))
    w.write(2, tokens_per_s=125.0, loss=2.25)
    recs = [json.loads(l) for l in open(path)]
    assert [r["step"] for r in recs] == [1, 2] and recs[0]["loss"] == 2.5
    get_logger().info("logger works")
    net = _Net()
    lt = LayerTimer(net, lambda name, mod: "dense" if isinstance(mod, nn.Linear) else None)
    with nvtx_range("step"):
        net(torch.randn(4, 8)).sum().backward()
    t = CudaTimer()
    with t.time("x"):
        torch.randn(64, 64) @ torch.randn(64, 64)
    assert t.resolve()["x"] >= 0.0
    assert lt is not None


def test_reserved_sms_shrink_the_persistent_grids(monkeypatch):
    """``native.reserve_sms`` leaves an even number of SMs out of what persistent kernels may fill."""
    from hyper_parallel_b200.ops import native
    monkeypatch.setitem(native._sm_count, 0, 148)
    monkeypatch.setattr(native, "_sm_reserve", 0)
    import torch
    dev = torch.device("cuda", 0)
    assert native.sm_count(dev) == 148
    native.reserve_sms(16)
    assert native.sm_count(dev) == 132
    native.reserve_sms(7)                       # CTA pairs: rounded down to an even number
    assert native.sm_count(dev) == 142
    native.reserve_sms(1000)
    assert native.sm_count(dev) == 2            # never below one CTA pair
    native.reserve_sms(0)
    assert native.sm_count(dev) == 148
