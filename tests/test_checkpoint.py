"""Distributed checkpoint: save/load round trips, resharding on load (save on 4 ranks, load on 2),
on-disk layout, rank-local metadata, offline ReshardHandler, layout json, single-file helpers."""
import os
import pickle

import numpy as np
import pytest
import torch

from dist_utils import run_distributed


def _full(name, shape):
    g = torch.Generator().manual_seed(sum(ord(c) for c in name))
    return torch.randn(*shape, generator=g)


SPECS = {"w_col": ((8, 12), ("None", "tp")), "w_row": ((8, 12), ("tp", "None")), "w_dp": ((8, 12), ("dp", "None")),
         "w_both": ((8, 12), ("dp", "tp")), "w_rep": ((8, 12), ("None", "None")), "w_multi": ((16, 4), (("dp", "tp"), "None"))}


def _state(mesh_shape, plain=True):
    from hyper_parallel_b200 import Layout, distribute_tensor
    layout = Layout(mesh_shape, ("dp", "tp"))
    sd = {}
    for name, (shape, spec) in SPECS.items():
        sd[name] = distribute_tensor(_full(name, shape), layout(*spec))
    if plain:
        sd["plain"] = _full("plain", (5, 3))
        sd["nested"] = {"step": 7, "lr": 0.5, "t": _full("nested.t", (4,))}
    return sd, layout


def _save_worker(rank, world, path, mesh_shape, use_collectives):
    from hyper_parallel_b200.core import checkpoint as ckpt
    sd, _ = _state(mesh_shape)
    md = ckpt.save(sd, checkpoint_id=path, use_collectives=use_collectives)
    assert set(md.state_dict_metadata) >= set(SPECS)
    if use_collectives and rank == 0:
        assert md.state_dict_metadata["w_rep"].chunks and len(md.state_dict_metadata["w_rep"].chunks) == 1
        assert len(md.state_dict_metadata["w_both"].chunks) == world


def _load_worker(rank, world, path, mesh_shape):
    from hyper_parallel_b200.core import checkpoint as ckpt
    sd, layout = _state(mesh_shape)
    expect = {k: v.to_local().clone() if hasattr(v, "to_local") else v for k, v in sd.items() if k in SPECS}
    for k in SPECS:
        sd[k].to_local().zero_()
    sd["plain"] = torch.zeros(5, 3)
    sd["nested"] = {"step": 0, "lr": 0.0, "t": torch.zeros(4)}
    ckpt.load(sd, checkpoint_id=path)
    for k in SPECS:
        assert torch.allclose(sd[k].to_local(), expect[k], atol=1e-5), k
        assert torch.allclose(sd[k].full_tensor(), _full(k, SPECS[k][0]), atol=1e-5), k
    assert torch.allclose(sd["plain"], _full("plain", (5, 3)))
    assert sd["nested"]["step"] == 7 and sd["nested"]["lr"] == 0.5
    assert torch.allclose(sd["nested"]["t"], _full("nested.t", (4,)))


def test_save_4_ranks_layout_on_disk_then_load_4_and_2(tmp_path):
    path = str(tmp_path / "ckpt")
    run_distributed(_save_worker, 4, path, (2, 2), True)
    files = sorted(os.listdir(path))
    assert ".metadata" in files
    assert all(f"_rank{r}_.safetensors" in files for r in range(4))
    assert any(f.endswith(".bytes") and "_rank" in f for f in files)
    assert not any(f.endswith(".tmp") for f in files)
    run_distributed(_load_worker, 4, path, (2, 2))
    run_distributed(_load_worker, 2, path, (1, 2))       # resharding on load
    run_distributed(_load_worker, 2, path, (2, 1))


def test_save_8_ranks_4x2_then_load_on_4_and_on_8_with_another_mesh(tmp_path):
    """The reference's resharding scenario (tests/torch/checkpoint/dcp_api.py: save on 8, load on 4)."""
    path = str(tmp_path / "ckpt8")
    run_distributed(_save_worker, 8, path, (4, 2), True)
    assert all(os.path.exists(os.path.join(path, f"_rank{r}_.safetensors")) for r in range(8))
    run_distributed(_load_worker, 4, path, (2, 2))
    run_distributed(_load_worker, 8, path, (2, 4))


def _subset_load_worker(rank, world, path):
    """Ranks 0-3 of an 8-rank job load onto a 2 x 2 mesh of their own; ranks 4-7 do not take part."""
    from hyper_parallel_b200 import Layout, distribute_tensor
    from hyper_parallel_b200.core import checkpoint as ckpt
    if rank >= 4:
        return
    lay = Layout((2, 2), ("dp", "tp"), [0, 1, 2, 3])
    sd = {k: distribute_tensor(torch.zeros(*shape), lay(*spec)) for k, (shape, spec) in SPECS.items()}
    sd["plain"] = torch.zeros(5, 3)
    sd["nested"] = {"step": 0, "lr": 0.0, "t": torch.zeros(4)}
    ckpt.load(sd, checkpoint_id=path)
    for k, (shape, _) in SPECS.items():
        assert torch.allclose(sd[k].full_tensor(), _full(k, shape), atol=1e-5), k
    assert sd["nested"]["step"] == 7


def test_a_subset_of_the_ranks_loads_what_all_ranks_saved(tmp_path):
    path = str(tmp_path / "ckpt_subset")
    run_distributed(_save_worker, 8, path, (4, 2), True)
    run_distributed(_subset_load_worker, 8, path)


def test_rank_local_metadata_without_collectives(tmp_path):
    path = str(tmp_path / "ckpt_local")
    run_distributed(_save_worker, 2, path, (1, 2), False)
    files = os.listdir(path)
    assert ".rank0_metadata" in files and ".rank1_metadata" in files and ".metadata" not in files


def test_metadata_pickle_names_reference_modules_and_reads_back(tmp_path):
    from hyper_parallel_b200.core import checkpoint as ckpt
    sd = {"a": torch.arange(6.0).reshape(2, 3), "meta": {"epoch": 3}}
    ckpt.save(sd, checkpoint_id=str(tmp_path), no_dist=True)
    raw = open(tmp_path / ".metadata", "rb").read()
    assert b"hyper_parallel.core.checkpoint.metadata" in raw       # readable by the reference
    md = ckpt.FileSystemReader(str(tmp_path)).load_metadata()
    keys = {k.fqn: k for k in md.storage_data}
    # the reference's reader looks a pickled (non-tensor) entry up without a chunk index, a tensor chunk
    # with its position in the chunk list
    assert keys["meta.epoch"].index is None and tuple(keys["meta.epoch"].offset) == ()
    assert keys["a"].index == 0 and tuple(keys["a"].offset) == (0, 0)
    out = {"a": torch.zeros(2, 3), "meta": {"epoch": 0}}
    ckpt.load(out, checkpoint_id=str(tmp_path), no_dist=True)
    assert torch.equal(out["a"], sd["a"]) and out["meta"]["epoch"] == 3
    with pytest.raises(KeyError):
        ckpt.load({"missing": torch.zeros(1)}, checkpoint_id=str(tmp_path), no_dist=True)
    ckpt.load({"missing": torch.zeros(1)}, checkpoint_id=str(tmp_path), no_dist=True,
              planner=ckpt.StandardLoadPlanner(allow_partial_load=True))


def test_reshard_handler_and_slice_area():
    from hyper_parallel_b200 import Layout
    from hyper_parallel_b200.core.checkpoint import ReshardHandler, infer_intersection, infer_slice_area_by_rank
    full = np.arange(8 * 12, dtype=np.float32).reshape(8, 12)
    src = Layout((2, 2), ("dp", "tp"), init_backend=False)("dp", "tp")
    dst = Layout((1, 4), ("dp", "tp"), init_backend=False)("tp", "None")
    shards = {}
    for r in range(4):
        a = infer_slice_area_by_rank(src.mesh_shape, src.tensor_map, r, full.shape)
        shards[r] = full[tuple(slice(b, e) for b, e in a)]
    for r in range(4):
        h = ReshardHandler("w", full.shape, src, dst, r)
        got = h.get_real_tensor(shards)
        a = infer_slice_area_by_rank(dst.mesh_shape, dst.tensor_map, r, full.shape)
        assert np.array_equal(got, full[tuple(slice(b, e) for b, e in a)])
    # the reference's contract: the caller cuts the named pieces out of the source shards itself
    h = ReshardHandler("w", full.shape, src, dst, 2)
    need = h.infer_all_tensor_offset()
    assert need == {2: ((0, 2), (0, 6)), 3: ((0, 2), (0, 6))}                 # rows 4..5 of the shards of ranks 2, 3
    pieces = {r: shards[r][tuple(slice(b, e) for b, e in a)] for r, a in need.items()}
    assert np.array_equal(h.get_real_tensor(pieces), full[4:6])
    with pytest.raises(ValueError):
        h.get_real_tensor({2: pieces[2]})                                      # a needed piece is missing
    with pytest.raises(ValueError):
        h.get_real_tensor({2: pieces[2][:1], 3: pieces[3]})                    # neither the piece nor the shard
    # None = the whole tensor on rank 0, on either side
    assert np.array_equal(ReshardHandler("w", full.shape, src, None, 0).get_real_tensor(shards), full)
    part = ReshardHandler("w", full.shape, None, dst, 3).get_real_tensor({0: full})
    assert np.array_equal(part, full[6:8])
    t = ReshardHandler("w", full.shape, None, dst, 1).get_real_tensor({0: torch.from_numpy(full)})
    assert isinstance(t, torch.Tensor) and torch.equal(t, torch.from_numpy(full[2:4]))
    with pytest.raises(ValueError):
        ReshardHandler("w", full.shape, None, None, 0)
    assert infer_intersection([(0, 4), (0, 4)], [(4, 8), (0, 4)]) is None
    with pytest.raises(ValueError):
        infer_slice_area_by_rank((2, 2), (1, 0), 0, (7, 12))


def test_layout_json_and_single_file_helpers(tmp_path):
    from hyper_parallel_b200 import Layout, distribute_tensor
    from hyper_parallel_b200.core import checkpoint as ckpt
    layout = Layout((1, 1), ("dp", "tp"), init_backend=False)
    lin = torch.nn.Linear(4, 4)
    lin.weight = torch.nn.Parameter(distribute_tensor(lin.weight.detach(), layout("None", "tp")))
    cur = ckpt.get_current_layout(lin)                      # keyed by rank id, then by parameter, as the reference's
    w = cur["0"]["weight"]
    assert w["tensor_map"] == [-1, 0] and w["alias_name"] == ["dp", "tp"]
    assert w["type"] == "torch.float32" and w["full_shape"] == [4, 4] and "bias" not in cur["0"]
    assert ckpt.get_global_layout(lin) == cur                # no process group: this rank alone
    ckpt.save_layout(cur, str(tmp_path / "rank0.layout"))
    ckpt.save_layout({"1": cur["0"]}, str(tmp_path / "rank1.layout"))
    assert ckpt.combine_layout(str(tmp_path)) == {"0": cur["0"], "1": cur["0"]}
    ckpt.save_layout(cur, str(tmp_path / "again.layout"))
    with pytest.raises(ValueError):
        ckpt.combine_layout(str(tmp_path))                   # rank 0 twice
    ckpt.save_checkpoint({"x": torch.ones(2)}, str(tmp_path / "one.pt"))
    assert torch.equal(ckpt.load_checkpoint(str(tmp_path / "one.pt"))["x"], torch.ones(2))
    # the reference's file-name rule: a stem and a suffix with a letter each; missing folders are created
    ckpt.save_checkpoint({"x": torch.zeros(1)}, tmp_path / "new_folder" / "model_1.safetensors")
    assert (tmp_path / "new_folder" / "model_1.safetensors").exists()
    for bad in ("noext", "1234.5", ".hidden", "name.123"):
        with pytest.raises(ValueError):
            ckpt.save_checkpoint({}, str(tmp_path / bad))


def _async_save_worker(rank, world, ckpt):
    from hyper_parallel_b200 import Layout, distribute_tensor
    from hyper_parallel_b200.core import checkpoint as dcp
    lay = Layout((world,), ("dp",))
    full = torch.arange(48, dtype=torch.float32).reshape(8, 6)
    sd = {"w": distribute_tensor(full.clone(), lay("dp", "None")), "b": torch.full((3,), 7.0), "step": 5}
    handle = dcp.async_save(sd, checkpoint_id=ckpt)
    sd["w"].to_local().zero_()                       # the caller may overwrite right away
    md = handle.wait()
    assert handle.done() and "w" in md.state_dict_metadata
    import torch.distributed as dist
    dist.barrier()
    # same layout
    out = {"w": distribute_tensor(torch.zeros(8, 6), lay("dp", "None")), "b": torch.zeros(3), "step": 0}
    dcp.load(out, checkpoint_id=ckpt)
    assert torch.equal(out["w"].full_tensor(), full) and torch.equal(out["b"], torch.full((3,), 7.0)) and out["step"] == 5
    # another layout: the rank-local metadata files are merged
    out2 = {"w": distribute_tensor(torch.zeros(8, 6), lay("None", "dp"))}
    dcp.load(out2, checkpoint_id=ckpt)
    assert torch.equal(out2["w"].full_tensor(), full)


def test_async_save_then_load_with_another_layout(tmp_path):
    run_distributed(_async_save_worker, 2, str(tmp_path / "async"))


class _Mlp(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.a = torch.nn.Linear(8, 16, bias=False)
        self.b = torch.nn.Linear(16, 8, bias=False)

    def forward(self, x):
        return self.b(torch.tanh(self.a(x)))


def _train_steps(net, opt, n, start=0):
    import hyper_parallel_b200 as hp
    g = torch.Generator().manual_seed(100)
    xs = torch.randn(8, 4, 8, generator=g)
    for i in range(start, start + n):
        net.zero_grads()
        net(xs[i]).pow(2).mean().backward()
        hp.hsdp_sync_stream()
        opt.step()


def _hsdp_resume_worker(rank, world, ckpt, phase):
    import hyper_parallel_b200 as hp
    from hyper_parallel_b200.core import checkpoint as dcp
    from hyper_parallel_b200.core.hsdp import get_sharded_state_dict, restore_optimizer_step
    from hyper_parallel_b200.optim import FusedAdamW
    torch.manual_seed(9)
    net = _Mlp()
    hp.hsdp(net, shard_size=world, threshold=0, optimizer_level="level3", grad_scale=1.0 / world)
    opt = FusedAdamW(net.parameters(), lr=1e-2, master_weights=False)
    if phase == "save":
        _train_steps(net, opt, 3)
        sd = get_sharded_state_dict(net, opt)
        dcp.save(sd, checkpoint_id=ckpt)
        _train_steps(net, opt, 2, start=3)            # the uninterrupted run
        full = {k: (v.full_tensor() if isinstance(v, hp.DTensor) else v) for k, v in get_sharded_state_dict(net).items()}
        if rank == 0:
            torch.save(full, ckpt + "_final.pt")
    else:
        opt.init_state()
        sd = get_sharded_state_dict(net, opt)
        dcp.load(sd, checkpoint_id=ckpt)
        restore_optimizer_step(opt, sd)
        assert opt._step_count == 3
        _train_steps(net, opt, 2, start=3)
        want = torch.load(ckpt + "_final.pt")
        for k, v in get_sharded_state_dict(net).items():
            got = v.full_tensor() if isinstance(v, hp.DTensor) else v
            assert torch.allclose(got, want[k], atol=1e-6), k


def test_hsdp_model_and_optimizer_resume_on_another_rank_count(tmp_path):
    ckpt = str(tmp_path / "hsdp_ckpt")
    run_distributed(_hsdp_resume_worker, 4, ckpt, "save")
    run_distributed(_hsdp_resume_worker, 2, ckpt, "resume")     # resumes sharded 2 ways instead of 4


def test_planner_utilities_of_the_reference(tmp_path):
    """Small helpers that planners written against the reference import: areas of chunks, narrowing, the
    chunks a rank holds, read items from chunk overlaps, folder creation, exports of the package."""
    from hyper_parallel_b200.core import checkpoint as ckpt
    from hyper_parallel_b200.core.checkpoint.standard_planner import create_read_items_for_chunk_list
    from hyper_parallel_b200.core.checkpoint.util import (check_path, chunk_to_area, create_chunk_list_for_tensor,
                                                         narrow_tensor_by_index, remove_redundant_plans)
    t = torch.arange(24).reshape(4, 6)
    assert narrow_tensor_by_index(t, (1, 2), (2, 3)).tolist() == [[8, 9, 10], [14, 15, 16]]
    assert narrow_tensor_by_index(t, (), ()) is t
    assert chunk_to_area(ckpt.ChunkStorageMetadata((1, 2), (2, 3))) == ((1, 3), (2, 5))
    assert create_chunk_list_for_tensor(t) == [ckpt.ChunkStorageMetadata((0, 0), (4, 6))]
    md = ckpt.TensorStorageMetadata(ckpt.TensorProperties("torch.int64", False, None), (4, 6),
                                    [ckpt.ChunkStorageMetadata((0, 0), (2, 6)), ckpt.ChunkStorageMetadata((2, 0), (2, 6))])
    items = create_read_items_for_chunk_list("w", md, [ckpt.ChunkStorageMetadata((1, 0), (2, 3))])
    assert [(i.dest_offsets, i.storage_index.index, i.storage_offsets, i.lengths) for i in items] == \
        [((0, 0), 0, (1, 0), (1, 3)), ((1, 0), 1, (0, 0), (1, 3))]
    assert all(i.type is ckpt.LoadItemType.TENSOR for i in items)
    check_path(tmp_path / "a" / "b.txt")
    check_path(tmp_path / "c")
    assert (tmp_path / "a").is_dir() and not (tmp_path / "a" / "b.txt").exists() and (tmp_path / "c").is_dir()
    assert remove_redundant_plans([ckpt.SavePlan(items=[]), ckpt.SavePlan(items=[])]) is not None
    for name in ("StorageReader", "StorageWriter", "WriteResult", "WriteItemType", "LoadItemType"):
        assert hasattr(ckpt, name)
