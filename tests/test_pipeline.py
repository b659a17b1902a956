"""Pipeline schedules: static validation of the generated programs, and 4-rank gloo runs of
GPipe / 1F1B / interleaved-1F1B whose losses and gradients must equal a single-process run."""
import pytest
import torch
from torch import nn

from dist_utils import run_distributed
from hyper_parallel_b200.core.pipeline_parallel.scheduler import (
    MetaStep, MetaStepType, add_send_recv, validate_pipeline_execution)


def _compute_order(kind, M, S, V=1):
    # build the compute-only order without process groups by borrowing the schedule classes' logic
    from hyper_parallel_b200.core.pipeline_parallel import scheduler as sch
    cls = {"gpipe": sch.ScheduleGPipe, "1f1b": sch.Schedule1F1B, "vpp": sch.ScheduleInterleaved1F1B}[kind]
    obj = cls.__new__(cls)
    obj.micro_batch_num, obj.real_stage_num, obj.n_local, obj.stage_num = M, S, V, S * V
    return obj.construct_stage_exec_order()


@pytest.mark.parametrize("kind,M,S,V", [("gpipe", 4, 4, 1), ("1f1b", 8, 4, 1), ("1f1b", 2, 4, 1),
                                        ("vpp", 8, 4, 2), ("vpp", 16, 4, 2), ("vpp", 3, 4, 2),
                                        ("vpp", 6, 4, 2), ("vpp", 8, 2, 3), ("1f1b", 16, 8, 1)])
def test_generated_programs_are_matched_and_deadlock_free(kind, M, S, V):
    progs = add_send_recv(_compute_order(kind, M, S, V), S * V, S)
    res = validate_pipeline_execution(progs, V)
    assert not res["has_errors"] and not res["has_cycle"], res["error_messages"]
    for r, prog in progs.items():
        f = [s for s in prog if s.type == MetaStepType.FWD]
        b = [s for s in prog if s.type == MetaStepType.BWD]
        assert len(f) == len(b) == M * V


def test_validator_detects_unmatched_and_deadlock():
    T = MetaStepType
    bad = {0: [MetaStep(0, T.FWD, 0), MetaStep(0, T.FWD_SEND, 0)], 1: [MetaStep(0, T.FWD, 1)]}
    res = validate_pipeline_execution(bad)                       # the reference's form: a report, no exception
    assert res["has_errors"] and not res["has_cycle"] and "have no entry" in res["error_messages"][0]
    with pytest.raises(RuntimeError, match="have no entry"):
        validate_pipeline_execution(bad, raise_on_error=True)
    dead = {0: [MetaStep(0, T.BWD_RECV, 0), MetaStep(0, T.FWD, 0), MetaStep(0, T.FWD_SEND, 0), MetaStep(0, T.BWD, 0)],
            1: [MetaStep(0, T.FWD_RECV, 1), MetaStep(0, T.FWD, 1), MetaStep(0, T.BWD, 1), MetaStep(0, T.BWD_SEND, 1)]}
    res = validate_pipeline_execution(dead)
    assert res["has_cycle"] and res["cycle_path"][0] == res["cycle_path"][-1] and len(res["cycle_ranks"]) == 2
    with pytest.raises(RuntimeError, match="deadlock"):
        validate_pipeline_execution(dead, raise_on_error=True)
    assert MetaStep.from_str("FWD_RECV_3_1") == MetaStep(3, T.FWD_RECV, 1)


def test_validator_building_blocks_keep_the_reference_contracts():
    """Names of transfers, the both-ends check and the cycle search, with the inputs and outputs of the
    reference's unit tests (tests/mindspore/st/pipeline_parallel/test_order.py:28-175 and :835-905)."""
    from hyper_parallel_b200.core.pipeline_parallel.scheduler import (detect_cycle_in_graph, generate_operations,
                                                                      parse_and_validate)
    T = MetaStepType
    pair = {0: [MetaStep(0, T.FWD, 0), MetaStep(0, T.FWD_SEND, 0)], 1: [MetaStep(0, T.FWD_RECV, 1), MetaStep(0, T.FWD, 1)]}
    ops = generate_operations(pair, chunk_num=1, com_type="loop")
    assert ops == {"0": ["Send_Receive_(0)->(1)_micro0_1th"], "1": ["Send_Receive_(0)->(1)_micro0_1th"]}
    assert parse_and_validate(ops) == []
    assert parse_and_validate({"1": ["Send_Receive_(1)->(2)_micro0_1th"]}, all_rank=True)          # rank 2 has no entry
    assert parse_and_validate({"1": ["Send_Receive_(1)->(2)_micro0_1th"],
                               "2": ["Send_Receive_(1)->(2)_micro0_1th", "Send_Receive_(1)->(2)_micro0_2th"]})
    assert parse_and_validate({"1": "not_a_list", "2": [1, 2, 3], "3": ["a", "b"]})                 # reported, not raised
    assert parse_and_validate({"1": [], "2": [""]}) == []
    assert detect_cycle_in_graph({"1": ["A", "B", "C", "A"]}) == (["A", "B", "C", "A"], ["1 A -> B", "1 B -> C", "1 C -> A"])
    assert detect_cycle_in_graph({"r1": ["A", "B", "C"], "r2": ["D", "E"]}) == (None, None)
    assert detect_cycle_in_graph({}) == (None, None)
    assert detect_cycle_in_graph({"1": ["A", "B", "C"], "2": ["C", "D", "E"], "3": ["E", "A"]}) == (
        ["A", "B", "C", "D", "E", "A"], ["1 A -> B", "1 B -> C", "2 C -> D", "2 D -> E", "3 E -> A"])
    assert detect_cycle_in_graph({"1": ["A", "B", "C"], "2": ["D", "E", "D"]}) == (["D", "E", "D"], ["2 D -> E", "2 E -> D"])
    assert detect_cycle_in_graph({"1": ["A", "B"], "2": ["B", "A"]}) == (["A", "B", "A"], ["1 A -> B", "2 B -> A"])
    assert detect_cycle_in_graph({"1": ["A", "A"]}) == (["A", "A"], ["1 A -> A"])
    # 'v' placement: virtual stage 3 of a 2-rank pipeline lives on rank 0 again
    v = {0: [MetaStep(0, T.FWD_SEND, 0), MetaStep(0, T.FWD_RECV, 3)], 1: [MetaStep(0, T.FWD_RECV, 1), MetaStep(0, T.FWD_SEND, 2)]}
    assert generate_operations(v, chunk_num=2, com_type="v")["1"] == ["Send_Receive_(0)->(1)_micro0_1th",
                                                                      "Send_Receive_(1)->(0)_micro0_1th"]


# ------------------------------------------------------------------ distributed --
HID, NSTAGE, BATCH, MICRO = 16, 8, 16, 8


def _make_layers():
    torch.manual_seed(7)
    return [nn.Sequential(nn.Linear(HID, HID), nn.Tanh()) for _ in range(NSTAGE)]


class _Last(nn.Module):
    def __init__(self, body):
        super().__init__()
        self.body = body

    def forward(self, x):
        return self.body(x).pow(2).mean() / MICRO


def _reference():
    layers = _make_layers()
    x = torch.arange(BATCH * HID, dtype=torch.float32).reshape(BATCH, HID) / (BATCH * HID)
    losses = []
    for xm in x.chunk(MICRO):
        h = xm
        for l in layers:
            h = l(h)
        loss = h.pow(2).mean() / MICRO
        loss.backward()
        losses.append(loss.item())
    return losses, [[p.grad.clone() for p in l.parameters()] for l in layers]


def _pp_worker(rank, world, kind):
    from hyper_parallel_b200 import PipelineStage
    from hyper_parallel_b200.core.pipeline_parallel import Schedule1F1B, ScheduleGPipe, ScheduleInterleaved1F1B
    ref_losses, ref_grads = _reference()
    layers = _make_layers()
    x = torch.arange(BATCH * HID, dtype=torch.float32).reshape(BATCH, HID) / (BATCH * HID)
    if kind == "vpp":
        idx = [rank, rank + world]                      # 8 virtual stages on 4 ranks x 2 chunks
        mods = [layers[i] if i < NSTAGE - 1 else _Last(layers[i]) for i in idx]
        stages = [PipelineStage(m, i, NSTAGE, device="cpu") for m, i in zip(mods, idx)]
        sched = ScheduleInterleaved1F1B(stages, MICRO)
        owned = idx
    else:
        per = NSTAGE // world
        idx = list(range(rank * per, (rank + 1) * per))
        body = nn.Sequential(*[layers[i] for i in idx])
        mod = _Last(body) if rank == world - 1 else body
        stage = PipelineStage(mod, rank, world, device="cpu")
        sched = (ScheduleGPipe if kind == "gpipe" else Schedule1F1B)(stage, MICRO)
        owned = idx
    out = sched.run(x) if rank == 0 else sched.run()
    if rank == world - 1:
        got = [l.item() for l in out]
        assert all(abs(a - b) < 1e-6 for a, b in zip(got, ref_losses)), (got, ref_losses)
    else:
        assert out is None
    for i in owned:
        for p, g in zip(layers[i].parameters(), ref_grads[i]):
            assert torch.allclose(p.grad, g, atol=1e-6), (kind, i)
    # a second step: shapes are cached now, so receives are posted ahead of the compute steps
    for i in owned:
        for p in layers[i].parameters():
            p.grad = None
    out = sched.run(x) if rank == 0 else sched.run()
    if rank == world - 1:
        assert all(abs(l.item() - b) < 1e-6 for l, b in zip(out, ref_losses))
    for i in owned:
        for p, g in zip(layers[i].parameters(), ref_grads[i]):
            assert torch.allclose(p.grad, g, atol=1e-6), (kind, i, "second step")


@pytest.mark.parametrize("kind", ["gpipe", "1f1b", "vpp"])
def test_pipeline_matches_single_process(kind):
    run_distributed(_pp_worker, 4, kind)
