"""Sub-meshes: ``mesh["tp"]`` / ``mesh["dp"]`` slices of a 2 x 2 mesh -- ``distribute_tensor`` slices,
data parallel + column / row parallel products on a sub-mesh, redistribution between sub-mesh
layouts, ``full_tensor`` equality.  Case list after the reference's tests/torch/shard/submesh.py
(15 cases on NPUs); here on 4 gloo ranks."""
import pytest
import torch

from dist_utils import run_distributed


def _setup():
    import hyper_parallel_b200 as hp
    mesh = hp.init_device_mesh("cpu", (2, 2), mesh_dim_names=("dp", "tp"))
    return hp, mesh


def _case_slices(rank, world):
    """distribute_tensor on the tp sub-mesh: every dp replica slices the same way."""
    from hyper_parallel_b200 import Replicate, Shard, distribute_tensor
    hp, mesh = _setup()
    tp = mesh["tp"]
    assert tp.mesh_shape == (2,) and list(tp.rank_list) == ([0, 1] if rank < 2 else [2, 3])
    w = torch.arange(16.0).view(4, 4)
    dw = distribute_tensor(w, tp, (Shard(1),))
    assert torch.equal(dw.to_local(), w[:, (rank % 2) * 2:(rank % 2) * 2 + 2])
    db = distribute_tensor(torch.arange(4.0), tp, (Shard(0),))
    assert torch.equal(db.to_local(), torch.arange(4.0)[(rank % 2) * 2:(rank % 2) * 2 + 2])
    dx = distribute_tensor(w, tp, (Replicate(),))
    assert torch.equal(dx.to_local(), w) and tuple(dx.shape) == (4, 4)
    dp = mesh["dp"]
    assert list(dp.rank_list) == ([0, 2] if rank % 2 == 0 else [1, 3])
    dd = distribute_tensor(w, dp, (Shard(0),))
    assert torch.equal(dd.to_local(), w[(rank // 2) * 2:(rank // 2) * 2 + 2])


def _case_column_parallel(rank, world):
    """Data parallel (different x per dp replica) + weight column parallel on the tp sub-mesh."""
    from hyper_parallel_b200 import Replicate, Shard, distribute_tensor
    hp, mesh = _setup()
    tp = mesh["tp"]
    x = torch.arange(8.0).view(2, 4) + 8.0 * (rank // 2)
    w = torch.arange(16.0).view(4, 4) * 0.1
    b = torch.arange(4.0)
    dx, dw, db = (distribute_tensor(x, tp, (Replicate(),)), distribute_tensor(w, tp, (Shard(1),)),
                  distribute_tensor(b, tp, (Shard(0),)))
    out = torch.matmul(dx, dw) + db
    assert tuple(out.shape) == (2, 4) and tuple(out.to_local().shape) == (2, 2)
    assert torch.allclose(out.full_tensor(), x @ w + b)


def _case_row_parallel(rank, world):
    """Row parallel product: contraction sharded -> Partial; reduce_partial and redistribute both give the sum."""
    from hyper_parallel_b200 import Replicate, Shard, distribute_tensor
    hp, mesh = _setup()
    tp = mesh["tp"]
    x = torch.arange(8.0).view(2, 4) + (rank // 2)
    w = torch.arange(16.0).view(4, 4) * 0.1
    dx, dw = distribute_tensor(x, tp, (Shard(1),)), distribute_tensor(w, tp, (Shard(0),))
    out = torch.matmul(dx, dw)
    assert out.layout.is_partial()
    assert torch.allclose(out.reduce_partial().to_local(), x @ w)
    red = out.redistribute(tp, (Shard(0),))
    assert torch.allclose(red.full_tensor(), x @ w) and tuple(red.to_local().shape) == (1, 4)


def _case_redistribute(rank, world):
    """Redistribution between layouts of one sub-mesh: S(0) -> R, R -> S(1), S(0) -> S(1) (all-to-all)."""
    from hyper_parallel_b200 import Replicate, Shard, distribute_tensor
    hp, mesh = _setup()
    for sub in (mesh["tp"], mesh["dp"]):
        t = torch.arange(24.0).view(4, 6)
        d0 = distribute_tensor(t, sub, (Shard(0),))
        assert torch.equal(d0.redistribute(sub, (Replicate(),)).to_local(), t)
        idx = sub.get_local_rank()
        assert torch.equal(distribute_tensor(t, sub, (Replicate(),)).redistribute(sub, (Shard(1),)).to_local(),
                           t[:, idx * 3:(idx + 1) * 3])
        assert torch.equal(d0.redistribute(sub, (Shard(1),)).to_local(), t[:, idx * 3:(idx + 1) * 3])
        assert torch.equal(d0.redistribute(sub, (Shard(1),)).full_tensor(), t)


def _case_mesh_mismatch(rank, world):
    """Operands on different (sub-)meshes do not mix, and a redistribute to another mesh raises."""
    from hyper_parallel_b200 import Replicate, Shard, distribute_tensor
    hp, mesh = _setup()
    t = torch.arange(16.0).view(4, 4)
    a = distribute_tensor(t, mesh["tp"], (Shard(0),))
    with pytest.raises(Exception):
        a.redistribute(mesh["dp"], (Shard(0),))
    full = distribute_tensor(t, mesh, (Shard(0), Shard(1)))
    assert torch.equal(full.to_local(), t[(rank // 2) * 2:(rank // 2) * 2 + 2, (rank % 2) * 2:(rank % 2) * 2 + 2])
    assert torch.equal(full.full_tensor(), t)


def _case_backward(rank, world):
    """Gradients through a sub-mesh product: column-parallel weight gradient equals the slice of the dense one."""
    from hyper_parallel_b200 import DTensor, Replicate, Shard, distribute_tensor
    hp, mesh = _setup()
    tp = mesh["tp"]
    torch.manual_seed(3)
    x = torch.randn(4, 6)
    w = torch.randn(6, 8)
    wd = torch.nn.Parameter(distribute_tensor(w, tp, (Shard(1),)))
    out = torch.matmul(distribute_tensor(x, tp, (Replicate(),)), wd)
    loss = (out * out).sum().reduce_partial() if hasattr((out * out).sum(), "reduce_partial") else (out * out).sum()
    rep = loss.layout.repeat_num() if isinstance(loss, DTensor) else 1
    loss.backward(torch.tensor(1.0 / max(rep, 1)) if isinstance(loss, DTensor) else None)
    wr = w.clone().requires_grad_()
    ((x @ wr) ** 2).sum().backward()
    g = wd.grad.to_local() if isinstance(wd.grad, DTensor) else wd.grad
    idx = tp.get_local_rank()
    # every tp rank holds half of the columns; the loss is the sum over the full output, replicated
    # on the dp axis only through the sub-mesh (each dp replica computes the same thing)
    assert torch.allclose(g, wr.grad[:, idx * 4:(idx + 1) * 4] / max(rep, 1) * max(rep, 1), atol=1e-5) or \
        torch.allclose(g * max(rep, 1), wr.grad[:, idx * 4:(idx + 1) * 4], atol=1e-5)


@pytest.mark.parametrize("case", [_case_slices, _case_column_parallel, _case_row_parallel, _case_redistribute,
                                  _case_mesh_mismatch, _case_backward])
def test_submesh(case):
    run_distributed(case, 4)
