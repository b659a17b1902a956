"""Discrete-event simulator of pipeline schedules (1F1B, interleaved / VPP, GPipe).

Role of hyper_parallel/auto_parallel/fast-tuner/fast_tuner/pipeline_conductor/pp_simulator.py:
given per-(stage, chunk) forward / backward times and a p2p latency it replays the schedule's
compute order with data dependencies and reports the makespan, per-stage busy time, bubble
ratio and the peak number of live micro-batch activations per stage.  The compute orders come
from the same generators the runtime uses, so what is simulated is what runs.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Sequence

from ...core.pipeline_parallel.scheduler import (MetaStep, MetaStepType, Schedule1F1B, ScheduleGPipe,
                                                ScheduleInterleaved1F1B)


@dataclass
class SimResult:
    makespan: float
    busy: List[float]
    bubble_ratio: float
    peak_live: List[int]
    timeline: Dict[int, list]


def compute_order(kind: str, micro: int, stages: int, chunks: int = 1) -> Dict[int, List[MetaStep]]:
    cls = {"gpipe": ScheduleGPipe, "1f1b": Schedule1F1B, "vpp": ScheduleInterleaved1F1B}[kind]
    obj = cls.__new__(cls)
    obj.micro_batch_num, obj.real_stage_num, obj.n_local, obj.stage_num = micro, stages, chunks, stages * chunks
    return obj.construct_stage_exec_order()


def simulate(order: Dict[int, List[MetaStep]], fwd: Sequence[float], bwd: Sequence[float], stages: int,
             p2p: float = 0.0) -> SimResult:
    """``fwd[v]`` / ``bwd[v]``: time of one micro-batch on virtual stage ``v``."""
    n_virtual = len(fwd)
    F, B = MetaStepType.FWD, MetaStepType.BWD
    finish: Dict[tuple, float] = {}
    clock = [0.0] * stages
    ptr = [0] * stages
    busy = [0.0] * stages
    live = [0] * stages
    peak = [0] * stages
    timeline = {s: [] for s in range(stages)}
    remaining = sum(len(v) for v in order.values())
    while remaining:
        progressed = False
        for s in range(stages):
            while ptr[s] < len(order[s]):
                st = order[s][ptr[s]]
                v, m = st.stage_index, st.micro_index
                if st.type == F:
                    dep = None if v == 0 else (F, m, v - 1)
                    deps = [dep] if dep else []
                else:
                    deps = [(F, m, v)] + ([] if v == n_virtual - 1 else [(B, m, v + 1)])
                if any(d not in finish for d in deps):
                    break
                ready = 0.0
                for d in deps:
                    same_rank = (d[2] % stages) == s
                    ready = max(ready, finish[d] + (0.0 if same_rank else p2p))
                start = max(clock[s], ready)
                dur = fwd[v] if st.type == F else bwd[v]
                clock[s] = start + dur
                finish[(st.type, m, v)] = clock[s]
                busy[s] += dur
                live[s] += 1 if st.type == F else -1
                peak[s] = max(peak[s], live[s])
                timeline[s].append((start, clock[s], st.type.name, m, v))
                ptr[s] += 1
                remaining -= 1
                progressed = True
        if not progressed:
            raise RuntimeError("simulated schedule deadlocks")
    makespan = max(clock)
    bubble = 1.0 - sum(busy) / (makespan * stages) if makespan > 0 else 0.0
    return SimResult(makespan, busy, bubble, peak, timeline)
