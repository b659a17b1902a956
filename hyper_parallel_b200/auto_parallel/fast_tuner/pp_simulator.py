"""Discrete-event simulator of pipeline schedules (1F1B, interleaved / VPP, GPipe).

Role of hyper_parallel/auto_parallel/fast-tuner/fast_tuner/pipeline_conductor/pp_simulator.py:
given per-(stage, chunk) forward / backward times and a p2p latency it replays the schedule's
compute order with data dependencies and reports the makespan, per-stage busy time, bubble
ratio and the peak number of live micro-batch activations per stage.  The compute orders come
from the same generators the runtime uses, so what is simulated is what runs.

Communication is modelled as blocks of its own (reference pp_simulator.py:820-1397 draws them as
separate lanes): an activation or gradient that crosses ranks occupies the sender's p2p lane for
``p2p`` time units, transfers of one sender are serialised in issue order, and the consumer can start
when the block ends.  Memory is tracked per stage as a timeline: ``static_bytes[s]`` plus
``act_bytes[v]`` for every micro-batch whose forward on virtual stage ``v`` has started and whose
backward has not finished.  ``render_text`` draws the lanes as text, ``timeline_rows`` gives them as
rows for a CSV file.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

from ...core.pipeline_parallel.scheduler import (MetaStep, MetaStepType, Schedule1F1B, ScheduleGPipe,
                                                ScheduleInterleaved1F1B)


@dataclass
class SimResult:
    makespan: float
    busy: List[float]
    bubble_ratio: float
    peak_live: List[int]
    timeline: Dict[int, list]
    comm: Dict[int, list] = None            # per sending stage: (start, end, "F"|"B", micro, from_v, to_stage)
    mem_timeline: Dict[int, list] = None    # per stage: (time, bytes) after every change
    peak_bytes: List[float] = None


def compute_order(kind: str, micro: int, stages: int, chunks: int = 1) -> Dict[int, List[MetaStep]]:
    cls = {"gpipe": ScheduleGPipe, "1f1b": Schedule1F1B, "vpp": ScheduleInterleaved1F1B}[kind]
    obj = cls.__new__(cls)
    obj.micro_batch_num, obj.real_stage_num, obj.n_local, obj.stage_num = micro, stages, chunks, stages * chunks
    return obj.construct_stage_exec_order()


def simulate(order: Dict[int, List[MetaStep]], fwd: Sequence[float], bwd: Sequence[float], stages: int,
             p2p: float = 0.0, act_bytes: Sequence[float] = None, static_bytes: Sequence[float] = None) -> SimResult:
    """``fwd[v]`` / ``bwd[v]``: time of one micro-batch on virtual stage ``v``; ``p2p``: duration of one
    stage-boundary transfer; ``act_bytes[v]``: activation bytes one micro-batch keeps on virtual stage
    ``v`` between its forward and its backward; ``static_bytes[s]``: weights + optimizer state of stage ``s``."""
    n_virtual = len(fwd)
    act = list(act_bytes) if act_bytes is not None else [0.0] * n_virtual
    static = list(static_bytes) if static_bytes is not None else [0.0] * stages
    lane_free = [0.0] * stages                       # when the p2p lane of a stage is free again
    arrive: Dict[tuple, float] = {}                  # (kind, micro, v) -> time its output reached the next rank
    comm = {s: [] for s in range(stages)}
    mem = list(static)
    mem_tl = {s: [(0.0, static[s])] for s in range(stages)}
    peak_b = list(static)
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
                    ready = max(ready, arrive.get(d, finish[d]))
                start = max(clock[s], ready)
                dur = fwd[v] if st.type == F else bwd[v]
                clock[s] = start + dur
                finish[(st.type, m, v)] = clock[s]
                # the transfer of the result is a block on this stage's p2p lane, issued the moment
                # the data exists (steps of a stage finish in time order, so the lane stays ordered)
                nxt = v + 1 if st.type == F else v - 1
                if p2p > 0.0 and 0 <= nxt < n_virtual and nxt % stages != s:
                    t0 = max(clock[s], lane_free[s])
                    lane_free[s] = t0 + p2p
                    arrive[(st.type, m, v)] = t0 + p2p
                    comm[s].append((t0, t0 + p2p, st.type.name[0], m, v, nxt % stages))
                if st.type == F:
                    mem[s] += act[v]
                    mem_tl[s].append((start, mem[s]))
                    peak_b[s] = max(peak_b[s], mem[s])
                else:
                    mem[s] -= act[v]
                    mem_tl[s].append((clock[s], mem[s]))
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
    return SimResult(makespan, busy, bubble, peak, timeline, comm, mem_tl, peak_b)


class CompiledOrder:
    """A compute order prepared for many evaluations with different step times (a balancer's inner
    loop): steps and their dependencies as integer ids, worked out once.  ``makespan`` replays the
    same rules as :func:`simulate` (same order, same p2p lane model) and returns the end time only --
    no timelines, no memory -- at a fraction of the cost."""

    def __init__(self, order: Dict[int, List[MetaStep]], n_virtual: int, stages: int):
        self.stages, self.n_virtual = stages, n_virtual
        micro = 1 + max((st.micro_index for seq in order.values() for st in seq), default=0)
        F = MetaStepType.FWD

        def key(is_f, m, v):
            return (m * n_virtual + v) * 2 + (1 if is_f else 0)

        self.n_keys = micro * n_virtual * 2
        self.steps = []                                      # per stage: (own id, is forward, v, deps, sends)
        for s in range(stages):
            seq = []
            for st in order[s]:
                v, m, is_f = st.stage_index, st.micro_index, st.type == F
                if is_f:
                    deps = () if v == 0 else (key(True, m, v - 1),)
                else:
                    deps = (key(True, m, v),) + (() if v == n_virtual - 1 else (key(False, m, v + 1),))
                nxt = v + 1 if is_f else v - 1
                sends = 0 <= nxt < n_virtual and nxt % stages != s
                seq.append((key(is_f, m, v), is_f, v, deps, sends))
            self.steps.append(seq)
        self.total = sum(len(q) for q in self.steps)

    def makespan(self, fwd: Sequence[float], bwd: Sequence[float], p2p: float = 0.0) -> float:
        stages = self.stages
        avail = [-1.0] * self.n_keys                         # when a step's result can be consumed; -1 = not run
        clock, lane, ptr = [0.0] * stages, [0.0] * stages, [0] * stages
        remaining = self.total
        while remaining:
            progressed = False
            for s in range(stages):
                seq, i, t = self.steps[s], ptr[s], clock[s]
                n = len(seq)
                while i < n:
                    k, is_f, v, deps, sends = seq[i]
                    ready = 0.0
                    for d in deps:
                        a = avail[d]
                        if a < 0.0:
                            ready = -1.0
                            break
                        if a > ready:
                            ready = a
                    if ready < 0.0:
                        break
                    t = (t if t > ready else ready) + (fwd[v] if is_f else bwd[v])
                    if sends and p2p > 0.0:
                        t0 = t if t > lane[s] else lane[s]
                        lane[s] = avail[k] = t0 + p2p
                    else:
                        avail[k] = t
                    i += 1
                if i != ptr[s]:
                    remaining -= i - ptr[s]
                    ptr[s], clock[s], progressed = i, t, True
            if not progressed:
                raise RuntimeError("simulated schedule deadlocks")
        return max(clock)


def timeline_rows(res: SimResult) -> List[list]:
    """``[lane, stage, start, end, kind, micro, virtual stage]`` rows (compute and p2p lanes) for a CSV."""
    rows = []
    for s, items in res.timeline.items():
        rows += [["compute", s, round(a, 6), round(b, 6), k, m, v] for a, b, k, m, v in items]
    for s, items in (res.comm or {}).items():
        rows += [["p2p", s, round(a, 6), round(b, 6), k, m, v] for a, b, k, m, v, _dst in items]
    return sorted(rows, key=lambda r: (r[1], r[0], r[2]))


def render_text(res: SimResult, width: int = 100) -> str:
    """The schedule as text: one compute lane per stage (forward = micro-batch digit, backward = letter),
    one p2p lane per stage ('>' forward activation, '<' gradient), and the peak memory per stage."""
    if res.makespan <= 0:
        return ""
    scale = width / res.makespan
    out = []
    for s in sorted(res.timeline):
        lane = [" "] * width
        for a, b, k, m, _v in res.timeline[s]:
            ch = str(m % 10) if k == "FWD" else chr(ord("a") + m % 26)
            for x in range(int(a * scale), max(int(b * scale), int(a * scale) + 1)):
                if x < width:
                    lane[x] = ch
        out.append(f"stage {s} |" + "".join(lane) + "|")
        if res.comm and res.comm.get(s):
            lane = [" "] * width
            for a, b, k, _m, _v, _d in res.comm[s]:
                for x in range(int(a * scale), max(int(b * scale), int(a * scale) + 1)):
                    if x < width:
                        lane[x] = ">" if k == "F" else "<"
            out.append(f"  p2p {s} |" + "".join(lane) + "|")
    if res.peak_bytes and any(res.peak_bytes):
        out.append("peak bytes per stage: " + ", ".join(f"{b:.3g}" for b in res.peak_bytes))
    out.append(f"makespan {res.makespan:.4g}, bubble {res.bubble_ratio:.3f}")
    return "\n".join(out)


def render_svg(res: SimResult, path: Optional[str] = None, width: int = 1200, lane_h: int = 22) -> str:
    """The schedule as a self-contained SVG drawing (no plotting library needed): per stage one compute
    lane (forward blocks light, backward blocks dark, labelled with the micro-batch), one p2p lane, and
    below them the live-activation memory of every stage as a step line.  Returns the SVG text and
    writes it to ``path`` when given.  Counterpart of the matplotlib timelines of the reference's
    simulator (fast_tuner/pipeline_conductor/pp_simulator.py:820-1397)."""
    if res.makespan <= 0:
        return ""
    stages = sorted(res.timeline)
    has_comm = bool(res.comm) and any(res.comm.get(s) for s in stages)
    rows_per_stage = 2 if has_comm else 1
    left, top = 70, 24
    sx = (width - left - 10) / res.makespan
    lanes_h = len(stages) * rows_per_stage * (lane_h + 4)
    mem_h = 90 if res.mem_timeline and any(res.mem_timeline.get(s) for s in stages) else 0
    height = top + lanes_h + mem_h + 40
    palette = ["#4e79a7", "#f28e2b", "#59a14f", "#e15759", "#76b7b2", "#edc948", "#b07aa1", "#9c755f"]
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" font-family="monospace" '
           f'font-size="10">',
           f'<text x="{left}" y="14">makespan {res.makespan:.4g}, bubble {res.bubble_ratio:.3f}</text>']
    y = top
    for s in stages:
        out.append(f'<text x="4" y="{y + lane_h - 7}">stage {s}</text>')
        for a, b, k, m, v in res.timeline[s]:
            x, w = left + a * sx, max((b - a) * sx, 0.5)
            fill = "#cfe2f3" if k == "FWD" else "#3d6b99"
            ink = "#000" if k == "FWD" else "#fff"
            out.append(f'<rect x="{x:.1f}" y="{y}" width="{w:.1f}" height="{lane_h}" fill="{fill}" stroke="#222" '
                       f'stroke-width="0.4"><title>{k} micro {m} virtual stage {v}: {a:.4g} - {b:.4g}</title></rect>')
            if w > 12:
                out.append(f'<text x="{x + 2:.1f}" y="{y + lane_h - 7}" fill="{ink}">{m}</text>')
        y += lane_h + 4
        if has_comm:
            out.append(f'<text x="4" y="{y + lane_h - 7}">p2p {s}</text>')
            for a, b, k, m, v, dst in res.comm.get(s, []):
                x, w = left + a * sx, max((b - a) * sx, 0.5)
                fill = "#a8d08d" if k == "F" else "#c27ba0"
                out.append(f'<rect x="{x:.1f}" y="{y + 4}" width="{w:.1f}" height="{lane_h - 8}" fill="{fill}">'
                           f'<title>{"activation" if k == "F" else "gradient"} micro {m} of virtual stage {v} -> stage '
                           f'{dst}</title></rect>')
            y += lane_h + 4
    if mem_h:
        peak = max(max((b for _t, b in res.mem_timeline.get(s, [])), default=0.0) for s in stages) or 1.0
        base = y + mem_h - 6
        out.append(f'<text x="4" y="{y + 12}">live activations</text>')
        for i, s in enumerate(stages):
            pts, last = [], 0.0
            for t, b in res.mem_timeline.get(s, []):
                pts.append(f"{left + t * sx:.1f},{base - last / peak * (mem_h - 20):.1f}")
                pts.append(f"{left + t * sx:.1f},{base - b / peak * (mem_h - 20):.1f}")
                last = b
            if pts:
                out.append(f'<polyline fill="none" stroke="{palette[i % len(palette)]}" stroke-width="1.2" '
                           f'points="{" ".join(pts)}"><title>stage {s}</title></polyline>')
    out.append("</svg>")
    text = "\n".join(out)
    if path:
        with open(path, "w") as f:
            f.write(text)
    return text
