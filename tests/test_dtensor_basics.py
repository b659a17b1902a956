"""DTensor basics, one pytest id per case, all cases in ONE launch of 8 gloo ranks: the factory
functions (even, uneven and empty shapes), ``numel`` / ``to`` / ``float``, a two-step SGD run through
redistributions, process groups (ranks, backend, ``split_group`` with ranks left out), the distributed
RNG tracker in both call forms, and random operators on DTensors.  Case list after the reference's
``tests/torch/shard/base_dtensor_init.py:24-140``, ``tests/torch/dtensor/dtensor_api.py:24-100``,
``tests/torch/shard/base_dtensor.py:47-150``, ``tests/torch/process_group/process_group.py:23-75`` and
``tests/torch/shard/base_random.py:33-160``."""
import json
import os
import traceback

import pytest
import torch

from dist_utils import run_distributed

WORLD = 8
CASES = {}


def case(fn):
    CASES[fn.__name__] = fn
    return fn


def _mesh(shape, names):
    import hyper_parallel_b200 as hp
    return hp.init_device_mesh("cpu", shape, mesh_dim_names=names)


def _factory_check(dist_op, torch_op, same, *args):
    import torch.distributed as dist
    from hyper_parallel_b200 import Replicate, Shard
    world, rank = dist.get_world_size(), dist.get_rank()
    mesh = _mesh((world,), ("dp",))
    plist = [[Shard(0)], [Shard(1)], [Shard(2)], [Replicate()]]
    for placements in plist:                                   # even
        size = [8, 16, 24]
        local = list(size)
        if isinstance(placements[0], Shard):
            local[placements[0].dim] //= world
        d = dist_op(size, *args, device_mesh=mesh, placements=placements)
        same(torch_op(local, *args), d.to_local())
        assert tuple(d.shape) == tuple(size)
    for placements in plist:                                   # uneven: torch.chunk semantics
        size = [5, 10, 15]
        d = dist_op(size, *args, device_mesh=mesh, placements=placements)
        if isinstance(placements[0], Shard):
            chunks = list(torch.chunk(torch_op(size, *args), world, dim=placements[0].dim))
            if rank < len(chunks):
                same(chunks[rank], d.to_local())
            else:
                assert d.to_local().numel() == 0
        else:
            same(torch_op(size, *args), d.to_local())
    d = dist_op([], *args, device_mesh=mesh, placements=[Replicate()])   # empty shape = a scalar
    same(torch_op([], *args), d.to_local())


def _eq(a, b):
    assert a.shape == b.shape and a.dtype == b.dtype and torch.equal(a, b), (a.shape, b.shape)


def _same_meta(a, b):
    assert a.shape == b.shape and a.dtype == b.dtype and a.layout == b.layout


@case
def factory_ones(rank):
    from hyper_parallel_b200.core.dtensor import ones
    _factory_check(ones, torch.ones, _eq)


@case
def factory_zeros(rank):
    from hyper_parallel_b200.core.dtensor import zeros
    _factory_check(zeros, torch.zeros, _eq)


@case
def factory_full(rank):
    from hyper_parallel_b200.core.dtensor import full
    _factory_check(full, torch.full, _eq, 123.4)


@case
def factory_empty(rank):
    from hyper_parallel_b200.core.dtensor import empty
    _factory_check(empty, torch.empty, _same_meta)


@case
def local_shape_and_offset_helper(rank):
    from hyper_parallel_b200 import Replicate, Shard
    from hyper_parallel_b200.core.utils import compute_local_shape_and_global_offset as f
    mesh = _mesh((2, 4), ("dp", "tp"))
    dp, tp = divmod(rank, 4)
    assert f((8, 16), mesh, (Shard(0), Shard(1))) == ((4, 4), (dp * 4, tp * 4))
    assert f((8, 16), mesh, (Replicate(), Shard(0))) == ((2, 16), (tp * 2, 0))
    assert f((16, 3), mesh, (Shard(0), Shard(0))) == ((2, 3), (dp * 8 + tp * 2, 0))      # two axes on one dim
    shape, off = f((10, 5), mesh, (Replicate(), Shard(0)))                                # 10 rows over 4: 3 3 3 1
    assert shape == ((3, 5) if tp < 3 else (1, 5)) and off == (tp * 3, 0)
    shape, off = f((2, 5), mesh, (Replicate(), Shard(0)))                                 # 2 rows over 4: 1 1 0 0
    assert shape == ((1, 5) if tp < 2 else (0, 5)) and off == (min(tp, 2), 0)


@case
def numel_is_global(rank):
    from hyper_parallel_b200 import DTensor, Replicate, Shard
    mesh = _mesh((2, 4), ("dp", "tp"))
    local = torch.ones(8, 8)
    for placements, factor in (([Replicate(), Replicate()], 1), ([Shard(0), Replicate()], 2),
                               ([Replicate(), Shard(1)], 4), ([Shard(0), Shard(1)], 8)):
        d = DTensor.from_local(local, mesh, placements)
        assert d.numel() == local.numel() * factor, (placements, d.numel())


@case
def to_keeps_mesh_and_placements(rank):
    from hyper_parallel_b200 import DTensor, Replicate, Shard
    mesh = _mesh((2, 4), ("dp", "tp"))
    placements = [Shard(0), Replicate()]
    d = DTensor.from_local(torch.ones(8, 8), mesh, placements)
    h = d.to(torch.float16)
    assert isinstance(h, DTensor) and h.dtype == torch.float16 and h.to_local().dtype == torch.float16
    assert h.device_mesh == mesh and tuple(h.placements) == tuple(placements) and h.shape == d.shape
    c = d.to(torch.device("cpu"))
    assert isinstance(c, DTensor) and c.device.type == "cpu" and c.device_mesh == mesh
    m = d.to(device=torch.device("cpu"), dtype=torch.int32)
    assert isinstance(m, DTensor) and m.dtype == torch.int32 and tuple(m.placements) == tuple(placements)


@case
def float_converts_the_local_shard(rank):
    from hyper_parallel_b200 import DTensor, Replicate, Shard
    mesh = _mesh((1, 8), ("dp", "tp"))
    local = torch.ones(8, 8).half()
    f = DTensor.from_local(local, mesh, (Replicate(), Shard(0))).float()
    assert isinstance(f, DTensor) and f.to_local().dtype == torch.float32
    assert torch.equal(f.to_local(), local.float()) and tuple(f.shape) == (64, 8)


@case
def sgd_through_redistributions_matches_single_process(rank):
    """x @ w with a column-sharded weight, two layout changes, a sum: loss and weight gradient of two
    SGD steps equal the single-process run."""
    from torch import nn, optim
    from hyper_parallel_b200 import DTensor, Replicate, Shard, SkipDTensorDispatch

    class Net(nn.Module):
        def __init__(self, mesh=None):
            super().__init__()
            self.mesh = mesh
            self.weight = nn.Parameter(torch.ones(8, 8))

        def forward(self, x):
            x = torch.matmul(x, self.weight)
            if self.mesh is not None:
                x = x.redistribute(self.mesh, (Shard(0), Shard(1)))
                x = x.redistribute(self.mesh, (Shard(1), Shard(0)))
            return torch.sum(x)

    ref = Net()
    ropt = optim.SGD(ref.parameters(), lr=0.01)
    for _ in range(2):
        rloss = ref(torch.ones(8, 8))
        rloss.backward()
        rgrad = ref.weight.grad.clone()
        ropt.step()
        ropt.zero_grad()

    mesh = _mesh((1, 8), ("dp", "tp"))
    net = Net(mesh)
    net.register_parameter("weight", nn.Parameter(DTensor.from_local(torch.ones(8, 1), mesh, (Replicate(), Shard(1)))))
    opt = optim.SGD(net.parameters(), lr=0.01)
    x = DTensor.from_local(torch.ones(8, 8), mesh, (Replicate(), Replicate()))
    for _ in range(2):
        loss = net(x).reduce_partial()
        loss.backward(torch.tensor(1.0 / loss.layout.repeat_num()))
        grad = net.weight.grad
        grad = grad.to_local().clone() if isinstance(grad, DTensor) else grad.clone()
        with SkipDTensorDispatch():
            opt.step()
            opt.zero_grad()
    assert torch.allclose(loss.to_local(), rloss, rtol=1e-3, atol=1e-3), (loss.to_local(), rloss)
    assert torch.allclose(grad, rgrad[:, rank:rank + 1], rtol=1e-3, atol=1e-3)


@case
def process_groups_and_split_group(rank):
    import torch.distributed as dist
    from hyper_parallel_b200.collectives import cc
    world = dist.get_world_size()
    cc.init_process_group()                                        # already initialised: a no-op
    assert cc.get_process_group_ranks() == list(range(world))
    assert cc.get_backend() == "gloo"
    group = cc.group_for_ranks(list(range(world)))
    assert cc.get_process_group_ranks(group) == list(range(world)) and cc.get_backend(group) == "gloo"
    pairs = [[r, r + 1] for r in range(0, world, 2)]
    pairs.pop()                                                    # the last pair gets no group
    sub = cc.split_group(group, pairs)
    mine = [rank, rank + 1] if rank % 2 == 0 else [rank - 1, rank]
    if world - 1 in mine:
        assert sub is None
    else:
        assert sub is not None and cc.get_process_group_ranks(sub) == mine and cc.get_backend(sub) == "gloo"
        t = torch.tensor([float(rank)])
        dist.all_reduce(t, group=sub)
        assert t.item() == float(sum(mine))
    with pytest.raises(ValueError):
        cc.split_group(sub if sub is not None else group, [[0, world + 3]])


@case
def size_one_mesh_axis_has_a_group_of_its_own(rank):
    """``None`` means "the world" to torch.distributed: an axis of size one must hand out a real
    one-member group, on the mesh and on its sub-mesh."""
    import torch.distributed as dist
    mesh = _mesh((1, 8), ("dp", "tp"))
    for group in (mesh.get_group("dp"), mesh["dp"].get_group()):
        assert group is not None and dist.get_process_group_ranks(group) == [rank]
        t = torch.ones(1) * rank
        dist.all_reduce(t, group=group)
        assert t.item() == rank
    t = torch.ones(1)
    dist.all_reduce(t, group=mesh.get_group("tp"))
    assert t.item() == 8


@case
def rng_tracker_construction_and_switch(rank):
    from hyper_parallel_b200.core.random import OffsetBasedRNGTracker, is_rng_supported_mesh
    assert is_rng_supported_mesh()
    torch.manual_seed(1000 + rank)
    synced = OffsetBasedRNGTracker(device="cpu", run_state_sync=True, seed=rank)
    assert synced.get_seed() == 0 and synced.distribute_region_enabled is True     # rank 0's seed everywhere
    plain = OffsetBasedRNGTracker(device="cpu", run_state_sync=False, seed=rank)
    assert plain.get_seed() == rank


@case
def rng_region_disabled_leaves_generator_and_offset(rank):
    from hyper_parallel_b200 import Replicate
    from hyper_parallel_b200.core.random import OffsetBasedRNGTracker
    tr = OffsetBasedRNGTracker(device="cpu", run_state_sync=False)
    tr._manual_seed(42)
    tr.distribute_region_enabled = False
    mesh = _mesh((8,), ("dp",))
    before = torch.get_rng_state()
    with tr._distribute_region(mesh, [Replicate()], (8, 4)):
        torch.rand(10)
    assert torch.equal(before, torch.get_rng_state()) and tr.get_offset() == 0
    tr.distribute_region_enabled = True
    with tr._distribute_region(device_mesh=mesh, placements=[Replicate()], global_shape=(8, 4)):
        torch.rand(10)
    assert torch.equal(before, torch.get_rng_state()) and tr.get_offset() == 32


@case
def rng_offsets_on_a_two_axis_mesh(rank):
    """Window of a shard = linear shard index x first-shard numel, rounded up to 4; afterwards the offset
    has moved by the number of distinct shards x that numel."""
    from hyper_parallel_b200 import Replicate, Shard
    from hyper_parallel_b200.core.random import OffsetBasedRNGTracker
    mesh = _mesh((2, 4), ("dp", "tp"))
    dp, tp = divmod(rank, 4)
    for placements, lin, shards, numel in (([Shard(0), Shard(1)], dp * 4 + tp, 8, 4 * 2),
                                           ([Shard(0), Replicate()], dp, 2, 4 * 8),
                                           ([Replicate(), Shard(1)], tp, 4, 8 * 2),
                                           ([Shard(1), Shard(1)], dp * 4 + tp, 8, 8 * 1)):
        tr = OffsetBasedRNGTracker(device="cpu", run_state_sync=False, seed=42)
        tr.set_offset(100)
        seen = {}
        orig = tr._set_device_state
        tr._set_device_state = lambda seed, offset: (seen.update(seed=seed, offset=offset), orig(seed, offset))
        with tr._distribute_region(mesh, placements, (8, 8)):
            pass
        assert seen == {"seed": 42, "offset": 100 + (lin * numel + 3) // 4 * 4}, (placements, seen)
        assert tr.get_offset() == 100 + (shards * numel + 3) // 4 * 4
    # uneven: the window is sized by the first (largest) shard on every rank
    tr = OffsetBasedRNGTracker(device="cpu", run_state_sync=False, seed=1)
    with tr._distribute_region(mesh, [Replicate(), Shard(0)], (10, 3)):
        pass
    assert tr.get_offset() == 4 * 3 * 3                              # 4 shards of ceil(10 / 4) = 3 rows


@case
def rng_offset_helpers_under_the_reference_names(rank):
    """Expected offsets computed with the module-level helpers equal what the tracker sets."""
    from hyper_parallel_b200 import Replicate, Shard
    from hyper_parallel_b200.core.random import (OffsetBasedRNGTracker, _PhiloxState, _calc_first_shard_size,
                                                 _calc_shard_info, _calc_shard_linear_idx)
    mesh = _mesh((2, 4), ("dp", "tp"))
    dp, tp = divmod(rank, 4)
    tr = OffsetBasedRNGTracker(device="cpu", run_state_sync=False)
    tr._manual_seed(42)
    assert tr._device_handle is torch
    for placements, lin, first in (([Shard(0), Shard(1)], dp * 4 + tp, [4, 2]), ([Shard(0), Replicate()], dp * 8, [4, 8]),
                                   ([Replicate(), Shard(1)], tp, [8, 2]), ([Shard(1), Shard(1)], (dp * 4 + tp), [8, 1])):
        idx, total = _calc_shard_info(mesh.get_coordinate(), mesh, placements)
        assert _calc_first_shard_size(mesh, placements, (8, 8)) == first
        state = _PhiloxState(tr._get_device_state())
        assert state.seed == 42 and state.offset == 0
        tr._set_pre_op_offset(state, mesh, placements, (8, 8))
        numel = first[0] * first[1]
        assert state.offset == (_calc_shard_linear_idx(idx, total) * numel + 3) // 4 * 4
        if placements[1] != Replicate():
            assert _calc_shard_linear_idx(idx, total) == lin
        tr._set_post_op_offset(state, (8, 8), 100)
        assert state.offset == 164


@case
def rng_replicated_draws_agree_whatever_the_local_seed(rank):
    import torch.distributed as dist
    from hyper_parallel_b200 import DTensor, Replicate
    from hyper_parallel_b200.core.random import OffsetBasedRNGTracker
    torch.manual_seed(rank)                                          # local generators differ
    mesh = _mesh((8,), ("dp",))
    local = torch.zeros(1, 4)
    tr = OffsetBasedRNGTracker(device="cpu")
    with tr._distribute_region(device_mesh=mesh, placements=[Replicate()], global_shape=(8, 4)):
        torch.nn.init.normal_(local)
    got = DTensor.from_local(local, mesh, [Replicate()]).to_local()
    all_ = [torch.empty_like(got) for _ in range(8)]
    dist.all_gather(all_, got)
    assert all(torch.equal(got, o) for o in all_) and got.abs().sum() > 0


@case
def random_ops_on_dtensors_use_the_tracker(rank):
    """rand_like / randn_like / dropout on a DTensor: shards differ although every rank seeded its
    generator alike, replicas agree although the ranks' generators differ, and the layout is kept."""
    import torch.distributed as dist
    import torch.nn.functional as F
    import hyper_parallel_b200.core.random as hr
    from hyper_parallel_b200 import Replicate, Shard, distribute_tensor
    mesh = _mesh((2, 4), ("dp", "tp"))
    hr._TRACKER = hr.OffsetBasedRNGTracker(device="cpu", seed=7)
    x = distribute_tensor(torch.ones(8, 16), mesh, (Replicate(), Shard(1)))
    for draw in (torch.rand_like, torch.randn_like, lambda t: F.dropout(t, 0.5, True)):
        torch.manual_seed(0 if draw is not torch.randn_like else rank)
        y = draw(x)
        assert tuple(y.placements) == tuple(x.placements) and tuple(y.shape) == (8, 16)
        loc = y.to_local().contiguous()
        all_ = [torch.empty_like(loc) for _ in range(8)]
        dist.all_gather(all_, loc)
        for r in range(8):
            same_shard = r % 4 == rank % 4
            assert torch.equal(all_[r], loc) == same_shard, (r, rank)
    off = hr.get_rng_tracker().get_offset()
    offs = [None] * 8
    dist.all_gather_object(offs, off)
    assert len(set(offs)) == 1 and off == 3 * 8 * 16                 # every rank advanced by the global numel
    hr._TRACKER = None


def _worker(rank, world, out_dir):
    results = {}
    for name, fn in CASES.items():
        try:
            fn(rank)
            results[name] = ""
        except Exception:  # noqa: BLE001  (recorded per case, reported by the parametrised test)
            results[name] = traceback.format_exc()
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump(results, f)


@pytest.fixture(scope="module")
def results(tmp_path_factory):
    out = tmp_path_factory.mktemp("dtensor_basics")
    run_distributed(_worker, WORLD, str(out), timeout=600.0)
    merged = {name: [] for name in CASES}
    for r in range(WORLD):
        with open(out / f"rank{r}.json") as f:
            for name, err in json.load(f).items():
                if err:
                    merged[name].append(f"rank {r}:\n{err}")
    return merged


@pytest.mark.parametrize("name", list(CASES))
def test_case(results, name):
    assert not results[name], "\n".join(results[name][:2])
