"""Pure-python unit tests of the tensor model: placements, mesh, layout conventions, planner, RNG."""
import pytest
import torch

from hyper_parallel_b200 import DTensor, Layout, Partial, Replicate, Shard
from hyper_parallel_b200.core.device_mesh import DeviceMesh, clear_mesh_cache
from hyper_parallel_b200.core.layout import _infer_slice_area_by_rank
from hyper_parallel_b200.core.tensor_redistribution import plan_redistribution


def L(shape=(2, 4), names=("dp", "mp")):
    return Layout(shape, names, init_backend=False)


def test_placements():
    assert Shard(1) == Shard(1) and Shard(1) != Shard(0) and hash(Shard(1)) == hash(Shard(1))
    assert Replicate().is_replicate() and Partial("max").is_partial("max") and not Partial().is_partial("max")
    with pytest.raises(ValueError):
        Partial("median")
    with pytest.raises(TypeError):
        Shard("0")


def test_mesh_rank_order_and_submesh():
    m = DeviceMesh("cpu", (2, 4), mesh_dim_names=("dp", "mp"), rank_list=tuple(range(8)), _init_backend=False, _rank=5)
    assert m.get_coordinate() == (1, 1)                       # row-major: last dim fastest
    assert m.get_rank_list_along_axis("mp") == [4, 5, 6, 7]
    assert m.get_rank_list_along_axis("dp") == [1, 5]
    sub = m["mp"]
    assert sub.rank_list == (4, 5, 6, 7) and sub.root_mesh is m and m["mp"] is sub
    assert m.get_local_rank("mp") == 1 and m.size() == 8 and m.size("dp") == 2
    assert m.get_global_shape((4, 8), (1, 0)) == (8, 32)
    with pytest.raises(ValueError):
        DeviceMesh("cpu", [[0, 1], [1, 2]], _init_backend=False)
    with pytest.raises(ValueError):
        DeviceMesh("cpu", (2, 2), mesh_dim_names=("interleaved_parallel", "x"), rank_list=range(4), _init_backend=False)
    with pytest.raises(KeyError):
        m["mp", "dp"]


def test_layout_tensor_map_conventions():
    lay = L()("dp", "mp")
    assert lay.tensor_map == (1, 0)                            # reversed mesh index
    assert lay.placements == (Shard(0), Shard(1))
    lay2 = L()("None", ("dp", "mp"))
    assert lay2.tensor_map == (-1, (1, 0)) and lay2.alias_tensor_map == ("None", ("dp", "mp"))
    assert lay2.get_global_shape((3, 2)) == (3, 16) and lay2.repeat_num() == 1
    assert L()("mp", "None").repeat_num() == 2
    d = lay.to_dict()
    assert set(d) == {"mesh_shape", "tensor_map", "interleaved_parallel", "alias_name", "rank_list"}
    with pytest.raises(ValueError):
        L()("dp", "dp")
    with pytest.raises(ValueError):
        L()("xx", "None")
    # placement form
    p = L()(Shard(1), Partial("sum"))
    p.placement_to_tensor_map(2)
    assert p.tensor_map == (-1, 1) and p.partial == [None, "sum"] and p.is_partial()
    with pytest.raises(ValueError):
        lay.set_partial_by_dev_axis("dp", "sum")               # shard + partial on one axis
    q = L()("dp", "None")
    q.set_partial_by_dev_axis("mp", "max")
    assert q.placements == (Shard(0), Partial("max"))
    q.reset_partial()
    assert not q.is_partial() and q == L()("dp", "None")


def test_slice_area_multi_axis_outer_first():
    # (dp, mp) shard one dim: dp is the outer split
    area = _infer_slice_area_by_rank((2, 4), ((1, 0),), 5, (16,))     # rank 5 = (dp 1, mp 1)
    assert area == [(10, 12)]
    area = _infer_slice_area_by_rank((2, 4), ((0, 1),), 5, (16,))     # mp outer, dp inner
    assert area == [(6, 8)]
    with pytest.raises(ValueError):
        _infer_slice_area_by_rank((2, 4), (0,), 0, (6,))


def test_dtensor_shapes_and_local():
    lay = L()("dp", "mp")
    t = DTensor.from_local(torch.zeros(3, 5), lay)
    assert tuple(t.shape) == (6, 20) and t.local_shape == (3, 5) and t.numel() == 120 and t.size(1) == 20
    assert t.to_local().shape == (3, 5) and t.placements == (Shard(0), Shard(1))
    t2 = DTensor.from_local(torch.zeros(3, 5), lay.mesh, (Shard(0), Replicate()))
    assert tuple(t2.shape) == (6, 5)
    assert t2.detach().layout == t2.layout and t2.float().dtype == torch.float32


def test_redistribution_plans():
    base = L()
    s = base("dp", "mp")
    r = base("None", "None")
    plan = plan_redistribution(s, r)
    assert [p[0] for p in plan] == ["all_gather", "all_gather"]
    assert plan_redistribution(r, s) == [("split", 0, 0), ("split", 1, 1)]
    a2a = plan_redistribution(base("mp", "None"), base("None", "mp"))
    assert a2a == [("all_to_all", 1, 0, 1)]
    part = base("dp", "None")
    part.set_partial_by_dev_axis("mp", "sum")
    assert plan_redistribution(part, base("dp", "mp")) == [("reduce_scatter", 1, 1, "sum")]      # Partial -> Shard
    assert plan_redistribution(part, base("dp", "None")) == [("all_reduce", 1, "sum")]
    p0 = base("None", "None")
    p0.set_partial_by_dev_axis("dp", "sum")
    assert plan_redistribution(p0, base("dp", "None")) == [("reduce_scatter", 0, 0, "sum")]      # Shard(0) too
    multi = plan_redistribution(base(("dp", "mp"), "None"), base("dp", "None"))
    assert multi == [("all_gather", 1, 0)]
    with pytest.raises(ValueError):
        plan_redistribution(s, Layout((4, 2), ("dp", "mp"), init_backend=False)("dp", "mp"))
    with pytest.raises(ValueError):
        plan_redistribution(r, part)


def test_rng_tracker_shard_consistency():
    from hyper_parallel_b200.core.random import OffsetBasedRNGTracker
    base = Layout((2, 2), ("dp", "mp"), init_backend=False)
    lay = base("None", "mp")                                     # replicated over dp, sharded over mp
    draws = {}
    for rank in range(4):
        clear_mesh_cache()
        mesh = DeviceMesh("cpu", (2, 2), mesh_dim_names=("dp", "mp"), rank_list=range(4), _init_backend=False, _rank=rank)
        l2 = Layout.from_device_mesh(mesh)("None", "mp")
        tr = OffsetBasedRNGTracker(device="cpu", run_state_sync=False, seed=123)
        with tr._distribute_region(l2, (4, 3)):
            draws[rank] = torch.rand(4, 3)
        assert tr.get_offset() == 24                              # 2 distinct shards x 12 elements
    assert torch.equal(draws[0], draws[2]) and torch.equal(draws[1], draws[3])     # replicas agree
    assert not torch.equal(draws[0], draws[1])                                      # shards differ
    clear_mesh_cache()


def test_groups_from_template_tile_the_world_like_mesh_axes():
    from hyper_parallel_b200.collectives.cc import generate_groups_from_template as groups
    assert groups([0, 1], 8) == [[0, 1], [2, 3], [4, 5], [6, 7]]
    assert groups([5, 7], 8) == [[0, 2], [1, 3], [4, 6], [5, 7]]
    assert groups([3], 4) == [[0], [1], [2], [3]]
    # every axis of a mesh: the group of any one rank generates the groups of all ranks
    shape = (2, 3, 4)
    world = 24
    for axis in range(3):
        clear_mesh_cache()
        per_rank = {}
        for rank in range(world):
            mesh = DeviceMesh("cpu", shape, mesh_dim_names=("a", "b", "c"), rank_list=range(world),
                              _init_backend=False, _rank=rank)
            per_rank[rank] = list(mesh.get_rank_list_along_axis(("a", "b", "c")[axis]))
            clear_mesh_cache()
        want = sorted({tuple(v) for v in per_rank.values()})
        for rank in (0, 7, 23):
            assert sorted(map(tuple, groups(per_rank[rank], world))) == want
    for bad, world in (([0, 1, 3], 8), ([0, 2], 6), ([0, 0], 4), ([0, 4], 4)):
        with pytest.raises(ValueError):
            groups(bad, world)


def test_device_mesh_helper_names_of_the_reference():
    clear_mesh_cache()
    m = DeviceMesh("cpu", (2, 2, 2), mesh_dim_names=("dp", "cp", "tp"), rank_list=range(8), _init_backend=False, _rank=5)
    assert (m.axis_index("dp"), m.axis_index("tp")) == (0, 2)
    assert (m.axis_id("dp"), m.axis_id("tp"), m.axis_id("None")) == (2, 0, -1)        # tensor_map numbering
    assert m.get_devices_for_axis("cp", 0) == [0, 2] and m.get_devices_for_axis(2, 6) == [6, 7]
    flat = m["dp", "cp"].flatten("dp_cp")
    assert flat.rank_list == (1, 3, 5, 7) and m["dp_cp"] is flat and m.get_flatten_mapping() == {"dp_cp": flat}
    with pytest.raises(ValueError):
        m.axis_index("xx")
    with pytest.raises(ValueError):
        m.get_devices_for_axis(3, 0)
    clear_mesh_cache()
