"""Redistribution on sub-meshes of larger meshes, one pytest id per case, all cases in ONE launch of
8 gloo ranks: sub-meshes ``mesh["tp"]`` / ``mesh["dp"]`` of a 4 x 2 and a 1 x 8 mesh (including the
size-one axis), one- and two-axis sub-meshes of a 2 x 2 x 2 mesh, Shard <-> Shard, Shard <-> Replicate
and Partial -> Shard / Replicate transitions; every local shard is compared with the slice of the
global tensor that the rank's coordinate in the sub-mesh selects.  Case list after the reference's
``tests/torch/shard/submesh.py:547-1500`` (``test_sub_mesh_redistribute_1`` .. ``_10``)."""
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


def _slice(t, placements, coords, sizes):
    """Local shard of ``t`` for a rank at ``coords`` of a mesh of ``sizes`` under ``placements``."""
    from hyper_parallel_b200 import Shard
    for p, c, n in zip(placements, coords, sizes):
        if isinstance(p, Shard):
            t = t.chunk(n, p.dim)[c]
    return t


def _coords(sub):
    import torch.distributed as dist
    ranks = list(sub.rank_list)
    idx = ranks.index(dist.get_rank())
    out = []
    for n in reversed(sub.mesh_shape):
        out.append(idx % n)
        idx //= n
    return tuple(reversed(out))


def _roundtrip(sub, t, src, dst):
    from hyper_parallel_b200 import distribute_tensor
    c, sizes = _coords(sub), sub.mesh_shape
    d = distribute_tensor(t, sub, src)
    assert torch.equal(d.to_local(), _slice(t, src, c, sizes)), ("distribute", src)
    r = d.redistribute(sub, dst)
    assert torch.equal(r.to_local(), _slice(t, dst, c, sizes)), ("redistribute", src, dst)
    assert torch.equal(r.full_tensor(), t)
    back = r.redistribute(sub, src)
    assert torch.equal(back.to_local(), d.to_local())


def _mesh(shape, names):
    import hyper_parallel_b200 as hp
    return hp.init_device_mesh("cpu", shape, mesh_dim_names=names)


@case
def mesh_4x2_tp_shard1_to_shard0(rank):
    from hyper_parallel_b200 import Shard
    _roundtrip(_mesh((4, 2), ("dp", "tp"))["tp"], torch.arange(16.0).view(4, 4), (Shard(1),), (Shard(0),))


@case
def mesh_4x2_dp_shard0_to_shard1(rank):
    from hyper_parallel_b200 import Shard
    _roundtrip(_mesh((4, 2), ("dp", "tp"))["dp"], torch.arange(64.0).view(8, 8), (Shard(0),), (Shard(1),))


@case
def mesh_4x2_dp_shard_to_replicate(rank):
    from hyper_parallel_b200 import Replicate, Shard
    _roundtrip(_mesh((4, 2), ("dp", "tp"))["dp"], torch.arange(32.0).view(8, 4), (Shard(0),), (Replicate(),))


@case
def mesh_1x8_tp_shard1_to_shard0(rank):
    from hyper_parallel_b200 import Shard
    _roundtrip(_mesh((1, 8), ("dp", "tp"))["tp"], torch.arange(64.0).view(8, 8), (Shard(1),), (Shard(0),))


@case
def mesh_1x8_size_one_axis_is_identity(rank):
    from hyper_parallel_b200 import Shard, distribute_tensor
    sub = _mesh((1, 8), ("dp", "tp"))["dp"]
    t = torch.arange(64.0).view(8, 8)
    d = distribute_tensor(t, sub, (Shard(1),))
    assert torch.equal(d.to_local(), t)
    assert torch.equal(d.redistribute(sub, (Shard(0),)).to_local(), t)


@case
def mesh_2x2x2_single_axis_submeshes(rank):
    from hyper_parallel_b200 import Replicate, Shard
    mesh = _mesh((2, 2, 2), ("dp", "cp", "tp"))
    t = torch.arange(48.0).view(4, 12)
    for name in ("dp", "cp", "tp"):
        sub = mesh[name]
        assert sub.mesh_shape == (2,) and rank in list(sub.rank_list)
        _roundtrip(sub, t, (Shard(0),), (Shard(1),))
        _roundtrip(sub, t, (Replicate(),), (Shard(1),))


@case
def mesh_2x2x2_two_axis_submesh(rank):
    from hyper_parallel_b200 import Replicate, Shard
    mesh = _mesh((2, 2, 2), ("dp", "cp", "tp"))
    sub = mesh["cp", "tp"] if hasattr(mesh, "__getitem__") else None
    assert sub.mesh_shape == (2, 2) and len(list(sub.rank_list)) == 4
    t = torch.arange(64.0).view(8, 8)
    _roundtrip(sub, t, (Shard(0), Shard(1)), (Shard(1), Shard(0)))
    _roundtrip(sub, t, (Shard(0), Replicate()), (Replicate(), Shard(1)))
    _roundtrip(sub, t, (Shard(0), Shard(0)), (Replicate(), Replicate()))


@case
def mesh_2x2x2_dp_tp_submesh_skips_middle_axis(rank):
    from hyper_parallel_b200 import Shard
    mesh = _mesh((2, 2, 2), ("dp", "cp", "tp"))
    sub = mesh["dp", "tp"]
    ranks = list(sub.rank_list)
    assert len(ranks) == 4 and rank in ranks
    cp = (rank // 2) % 2
    assert all(((r // 2) % 2) == cp for r in ranks)          # the ranks that share this rank's cp coordinate
    _roundtrip(sub, torch.arange(64.0).view(8, 8), (Shard(0), Shard(1)), (Shard(1), Shard(0)))


@case
def partial_on_submesh_reduces_within_the_submesh(rank):
    from hyper_parallel_b200 import DTensor, Partial, Replicate, Shard
    mesh = _mesh((4, 2), ("dp", "tp"))
    sub = mesh["tp"]
    local = torch.full((4, 4), float(rank + 1))
    d = DTensor.from_local(local, sub, (Partial("sum"),))
    pair = list(sub.rank_list)
    total = float(sum(r + 1 for r in pair))
    assert torch.equal(d.redistribute(sub, (Replicate(),)).to_local(), torch.full((4, 4), total))
    sh = d.redistribute(sub, (Shard(0),))
    assert torch.equal(sh.to_local(), torch.full((2, 4), total))


@case
def full_mesh_and_submesh_agree(rank):
    from hyper_parallel_b200 import Replicate, Shard, distribute_tensor
    mesh = _mesh((4, 2), ("dp", "tp"))
    t = torch.arange(64.0).view(8, 8)
    full = distribute_tensor(t, mesh, (Replicate(), Shard(1)))
    sub = distribute_tensor(t, mesh["tp"], (Shard(1),))
    assert torch.equal(full.to_local(), sub.to_local())
    assert torch.equal(full.full_tensor(), sub.full_tensor())


@case
def redistribute_to_other_submesh_raises(rank):
    from hyper_parallel_b200 import Shard, distribute_tensor
    mesh = _mesh((4, 2), ("dp", "tp"))
    a = distribute_tensor(torch.arange(16.0).view(4, 4), mesh["tp"], (Shard(0),))
    try:
        a.redistribute(mesh["dp"], (Shard(0),))
    except Exception:  # noqa: BLE001
        return
    raise AssertionError("redistribute across different sub-meshes must raise")


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
    out = tmp_path_factory.mktemp("submesh_cases")
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
