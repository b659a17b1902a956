"""Pipeline schedules: GPipe, 1F1B and interleaved 1F1B (VPP), with a static validator.

Capabilities of hyper_parallel/core/pipeline_parallel/scheduler.py:29-848 of the reference
(``MetaStep`` programs interpreted per rank; ``run(*args)`` returns the list of last-stage
outputs per micro-batch).  ``ScheduleGPipe`` works here, and ``overlap_p2p`` is a real
constructor argument of every schedule.

How a program is built:

1. each schedule emits a *compute-only* order per real stage (``FWD`` / ``BWD`` steps);
2. ``add_send_recv`` replays all ranks in lock-step, respecting data dependencies, and each
   time a step produces data for another rank it appends the ``*_SEND`` to the producer's
   program and, at the same moment, the matching ``*_RECV`` to the consumer's program.
   Sends and receives of any pair of ranks therefore appear in the same relative order on
   both sides -- the property NCCL p2p needs (no tags) -- and receives are posted as early
   as the data can exist, which is what lets them overlap with compute.

``validate_pipeline_execution`` replays programs with blocking semantics and reports
unmatched pairs or a deadlock.
"""
from __future__ import annotations

import logging
import os
from enum import Enum, auto
from typing import Dict, List, Optional, Tuple

import torch

from .stage import PipelineStage
from .utils import MicroBatch

logger = logging.getLogger(__name__)
_LOG = logger


class MetaStepType(Enum):
    FWD = auto()
    BWD = auto()
    FWD_RECV = auto()
    FWD_SEND = auto()
    BWD_RECV = auto()
    BWD_SEND = auto()


class MetaStep:
    """One instruction of a pipeline program: (micro-batch, type, virtual stage)."""

    __slots__ = ("_micro_index", "_type", "_stage_index")

    def __init__(self, micro_index: int, meta_type: MetaStepType, stage_index: int):
        self._micro_index = micro_index
        self._type = meta_type
        self._stage_index = stage_index

    micro_index = property(lambda self: self._micro_index)
    type = property(lambda self: self._type)
    stage_index = property(lambda self: self._stage_index)

    def __eq__(self, other):
        if not isinstance(other, MetaStep):
            return NotImplemented
        return (self._type, self._micro_index, self._stage_index) == \
            (other._type, other._micro_index, other._stage_index)

    def __hash__(self):
        return hash((self._type, self._micro_index, self._stage_index))

    def __repr__(self):
        return f"MetaStep(type={self._type}, micro_index={self._micro_index}, stage_index={self._stage_index})"

    @staticmethod
    def from_str(text: str) -> "MetaStep":
        """Parse ``"FWD_3_1"`` style text: type, micro index, stage index."""
        *kind, micro, stage = text.strip().split("_")
        return MetaStep(int(micro), MetaStepType["_".join(kind)], int(stage))


# ----------------------------------------------------------------- comm insertion --
def add_send_recv(compute_order: Dict[int, List[MetaStep]], stage_num: int, real_stage_num: int,
                  style: str = "loop") -> Dict[int, List[MetaStep]]:
    """Insert matched SEND/RECV steps into per-real-stage compute orders (see module docstring).

    ``style``: ``"loop"`` places virtual stage ``s`` on real stage ``s % real_stage_num``;
    ``"v"`` folds back (``s`` and ``2*real-1-s`` share a rank).
    """
    def owner(s: int) -> int:
        if style == "v":
            r = s % (2 * real_stage_num)
            return r if r < real_stage_num else 2 * real_stage_num - 1 - r
        return s % real_stage_num

    F, B = MetaStepType.FWD, MetaStepType.BWD
    progs: Dict[int, List[MetaStep]] = {r: [] for r in compute_order}
    ptr = {r: 0 for r in compute_order}
    done = set()
    total = sum(len(v) for v in compute_order.values())
    executed = 0
    while executed < total:
        ready = []
        for r, order in compute_order.items():
            if ptr[r] >= len(order):
                continue
            st = order[ptr[r]]
            if st is None:          # explicit bubble
                ready.append((r, None))
                continue
            s, m = st.stage_index, st.micro_index
            if st.type == F:
                ok = s == 0 or (F, m, s - 1) in done
            else:
                ok = (F, m, s) in done and (s == stage_num - 1 or (B, m, s + 1) in done)
            if ok:
                ready.append((r, st))
        if not ready:
            raise RuntimeError("pipeline compute order deadlocks: no stage can make progress")
        newly = []
        for r, st in ready:
            ptr[r] += 1
            executed += 1
            if st is None:
                continue
            s, m = st.stage_index, st.micro_index
            progs[r].append(st)
            newly.append((st.type, m, s))
            if st.type == F and s < stage_num - 1:
                dst = owner(s + 1)
                if dst != r:
                    progs[r].append(MetaStep(m, MetaStepType.FWD_SEND, s))
                    progs[dst].append(MetaStep(m, MetaStepType.FWD_RECV, s + 1))
            elif st.type == B and s > 0:
                dst = owner(s - 1)
                if dst != r:
                    progs[r].append(MetaStep(m, MetaStepType.BWD_SEND, s))
                    progs[dst].append(MetaStep(m, MetaStepType.BWD_RECV, s - 1))
        done.update(newly)
    return progs


# --------------------------------------------------------------------- validator --
# Function names, arguments and return values follow the reference's static checker
# (core/pipeline_parallel/scheduler.py:571-848 there), so tools written against it keep working:
# ``generate_operations`` names every transfer of every rank, ``parse_and_validate`` checks that each
# named transfer appears on both of its ranks, ``detect_cycle_in_graph`` looks for a cycle in the
# "happens before on one rank" graph of those names (a cycle = ranks waiting for one another), and
# ``validate_pipeline_execution`` runs all three.  On top of that the programs are replayed with
# blocking receives, which also catches a receive whose send never comes.
def _stage_owner(stage_index: int, com_type: str, total_stages: int, real_stage_num: int) -> int:
    if com_type == "loop":
        return stage_index % real_stage_num
    if com_type == "v":
        r = stage_index % (2 * real_stage_num)
        return r if r < real_stage_num else 2 * real_stage_num - 1 - r
    raise ValueError(f"com_type must be 'loop' or 'v', got {com_type!r}")


def generate_operations(order_list: Dict[int, List[MetaStep]], chunk_num: int = 1,
                        com_type: str = "loop") -> Dict[str, List[str]]:
    """``{str(rank): ["Send_Receive_(src)->(dst)_micro<m>_<k>th", ...]}``: the transfers of every rank in
    program order.  Both ends of a transfer get the same name; ``k`` counts the transfers of one
    (src, dst, micro-batch) triple on that rank, so matching sends and receives pair up by name."""
    real = len(order_list)
    total = real * chunk_num
    out: Dict[str, List[str]] = {}
    for rank, steps in order_list.items():
        counter: Dict[tuple, int] = {}
        ops = []
        for st in steps:
            t, s = st.type, st.stage_index
            if t in (MetaStepType.FWD_SEND, MetaStepType.BWD_SEND):
                peer_stage = s + 1 if t == MetaStepType.FWD_SEND else s - 1
                if not 0 <= peer_stage < total:
                    continue
                pair = (rank, _stage_owner(peer_stage, com_type, total, real), st.micro_index)
            elif t in (MetaStepType.FWD_RECV, MetaStepType.BWD_RECV):
                peer_stage = s - 1 if t == MetaStepType.FWD_RECV else s + 1
                if not 0 <= peer_stage < total:
                    continue
                pair = (_stage_owner(peer_stage, com_type, total, real), rank, st.micro_index)
            else:
                continue
            counter[pair] = counter.get(pair, 0) + 1
            ops.append(f"Send_Receive_({pair[0]})->({pair[1]})_micro{pair[2]}_{counter[pair]}th")
        if ops:
            out[str(rank)] = ops
    return out


def parse_and_validate(data, all_rank: bool = True) -> List[str]:
    """Check a ``{rank: [transfer names]}`` table: every name must be listed by both ranks it mentions
    (with ``all_rank`` a mentioned rank that has no entry at all is an error too).  Problems are logged
    and returned as a list of messages; malformed input is reported, never raised."""
    import re
    errors: List[str] = []
    if not isinstance(data, dict):
        errors.append("input must be a dict of rank -> list of transfer names")
    else:
        good = {k: set(v) for k, v in data.items() if isinstance(v, list) and all(isinstance(i, str) for i in v)}
        for key, values in data.items():
            if key not in good:
                errors.append(f"values for key {key!r} must be a list of strings")
                continue
            for value in values:
                ranks = set(re.findall(r"\((\d+)\)", value)[:2])
                if all_rank:
                    missing = ranks - good.keys()
                    if missing:
                        errors.append(f"ranks {sorted(missing)} named by {value!r} have no entry")
                        continue
                for r in (ranks if all_rank else ranks & good.keys()):
                    if value not in good[r]:
                        errors.append(f"rank {r} lacks the transfer {value!r}")
    for e in errors:
        _LOG.error("pipeline schedule: %s", e)
    return errors


def detect_cycle_in_graph(ranks_map: Dict[str, List[str]]):
    """``(cycle_path, cycle_ranks)`` of the first cycle in the graph whose edges join consecutive entries
    of each rank's list -- ``cycle_path`` the nodes (first = last), ``cycle_ranks`` one
    ``"<rank> <u> -> <v>"`` per edge -- or ``(None, None)``."""
    graph: Dict[str, List[str]] = {}
    edge_rank: Dict[tuple, str] = {}
    for rank, nodes in (ranks_map or {}).items():
        for u, v in zip(nodes, nodes[1:]):
            graph.setdefault(u, []).append(v)
            graph.setdefault(v, [])
            edge_rank[(u, v)] = rank
    done = set()
    for root in graph:
        if root in done:
            continue
        path, on_path, iters = [root], {root}, [iter(graph[root])]
        while iters:
            nxt = next(iters[-1], None)
            if nxt is None:                         # every edge of the last node followed: leave it
                node = path.pop()
                on_path.discard(node)
                done.add(node)
                iters.pop()
            elif nxt in on_path:
                cyc = path[path.index(nxt):] + [nxt]
                return cyc, [f"{edge_rank[(u, v)]} {u} -> {v}" for u, v in zip(cyc, cyc[1:])]
            elif nxt not in done:
                path.append(nxt)
                on_path.add(nxt)
                iters.append(iter(graph[nxt]))
    return None, None


def output_cycle_results(cycle_path, cycle_ranks) -> None:
    if cycle_path:
        _LOG.error("pipeline schedule: ranks wait for one another: %s (%s)", " -> ".join(cycle_path),
                   "; ".join(cycle_ranks))


def _replay_blocking(order_list: Dict[int, List[MetaStep]]) -> Optional[str]:
    """Replay with blocking receives; returns a message when some rank can never proceed."""
    ptr = {r: 0 for r in order_list}
    sent: Dict[Tuple[str, int, int], bool] = {}
    progress = True
    while progress:
        progress = False
        for r, prog in order_list.items():
            while ptr[r] < len(prog):
                st = prog[ptr[r]]
                t, m, s = st.type, st.micro_index, st.stage_index
                if t == MetaStepType.FWD_SEND:
                    sent[("f", m, s + 1)] = True
                elif t == MetaStepType.BWD_SEND:
                    sent[("b", m, s - 1)] = True
                elif t == MetaStepType.FWD_RECV:
                    if not sent.get(("f", m, s)):
                        break
                elif t == MetaStepType.BWD_RECV:
                    if not sent.get(("b", m, s)):
                        break
                ptr[r] += 1
                progress = True
    stuck = {r: order_list[r][p] for r, p in ptr.items() if p < len(order_list[r])}
    if stuck:
        return "deadlock: " + ", ".join(f"rank {r} waits at {st}" for r, st in stuck.items())
    return None


def validate_pipeline_execution(order_list: Dict[int, List[MetaStep]], chunk_num: int = 1,
                                com_type: str = "loop", raise_on_error: bool = False) -> dict:
    """Static check of per-rank programs.  Returns ``{"formatted_operations", "cycle_path",
    "cycle_ranks", "has_cycle"}`` as the reference does, plus ``"error_messages"`` (unmatched transfers,
    the cycle, a replay that gets stuck) and ``"has_errors"``.  With ``raise_on_error`` any error raises
    ``RuntimeError`` instead -- the form the schedules use on themselves."""
    ops = generate_operations(order_list, chunk_num, com_type)
    messages = list(parse_and_validate(ops, True))
    cycle_path, cycle_ranks = detect_cycle_in_graph(ops)
    output_cycle_results(cycle_path, cycle_ranks)
    if cycle_path:
        messages.append("ranks wait for one another: " + " -> ".join(cycle_path))
    stuck = _replay_blocking(order_list)
    if stuck:
        messages.append(stuck)
    result = {"formatted_operations": ops, "cycle_path": cycle_path, "cycle_ranks": cycle_ranks,
              "has_cycle": bool(cycle_path), "error_messages": messages, "has_errors": bool(messages)}
    if raise_on_error and messages:
        raise RuntimeError("invalid pipeline programs: " + "; ".join(messages))
    return result


# ----------------------------------------------------------------------- runtime --
class PipelineScheduleRuntime:
    """Interprets a per-rank MetaStep program over one or several local (virtual) stages."""

    def __init__(self, stages, micro_batch_num: int, args_batch_dim=None, kwargs_batch_dim=None,
                 output_concat_dim=None, overlap_p2p: bool = True):
        self.stages: List[PipelineStage] = list(stages) if isinstance(stages, (list, tuple)) else [stages]
        self.micro_batch_num = micro_batch_num
        self.n_local = len(self.stages)
        self.splitter = MicroBatch(micro_batch_num, args_batch_dim, kwargs_batch_dim)
        self.output_concat_dim = output_concat_dim
        self.overlap_p2p = overlap_p2p
        for st in self.stages:
            st.init(self.n_local)
        s0 = self.stages[0]
        self.stage_num = s0.stage_num
        self.real_stage_num = s0.real_stage_num
        self.real_stage_index = s0.real_stage_index
        self.stage_by_index = {st.stage_index: st for st in self.stages}
        self.exec_order: Dict[int, List[MetaStep]] = {}
        # Receives are posted ahead of the compute steps, so an NCCL receive kernel sits on a few SMs
        # and spins until its peer sends -- for most of a backward step in 1F1B.  The persistent GEMMs
        # stride their tiles over one CTA per SM and cannot share an SM with it: the CTAs meant for
        # those SMs start when others finish and the GEMM takes far longer (measured on the last
        # stage of PP=2: backward 88 ms with a receive pending, 73 ms without).  Leaving 16 SMs out of
        # the persistent grids (8 were not enough) removes that and costs next to nothing under the
        # power cap; HPB_PP_RESERVE_SMS overrides the number (0 = off).
        if overlap_p2p and torch.cuda.is_available():
            from ...ops import native as _native
            want = int(os.environ.get("HPB_PP_RESERVE_SMS", "16"))
            if want > _native._sm_reserve:
                _native.reserve_sms(want)
        # HPB_PP_TRACE=1: CUDA-event timers on the compute stream around every compute step, split
        # into the wait for its received operand and the compute itself (``trace_report()``)
        self.tracer = None
        self.timeline = None              # HPB_PP_TRACE=2: (label, micro, start event, end event) of the last run
        if os.environ.get("HPB_PP_TRACE", "0") == "1":
            from ...utils.tracing import CudaTimer
            self.tracer = CudaTimer()
        elif os.environ.get("HPB_PP_TRACE", "0") == "2" and torch.cuda.is_available():
            self.timeline = []
        self.build_exec_order()

    # subclasses fill self.exec_order = {real_stage: [MetaStep]}
    def construct_stage_exec_order(self) -> Dict[int, List[MetaStep]]:
        raise NotImplementedError

    def build_exec_order(self) -> None:
        compute = self.construct_stage_exec_order()
        self.exec_order = add_send_recv(compute, self.stage_num, self.real_stage_num)

    def run(self, *args, **kwargs):
        micro_args, micro_kwargs = self.splitter(args, kwargs) if (args or kwargs) else \
            ([()] * self.micro_batch_num, [{}] * self.micro_batch_num)
        return self.run_microbatches(micro_args, micro_kwargs)

    def trace_report(self) -> Dict[str, tuple]:
        """``{key: (mean ms, count)}`` of the traced steps so far (synchronises); empty without HPB_PP_TRACE=1."""
        if self.tracer is None:
            return {}
        means = self.tracer.resolve()
        return {k: (means[k], self.tracer.counts[k]) for k in means}

    def trace_timeline(self) -> List[tuple]:
        """``[(label, micro, start ms, end ms)]`` of the compute steps of the last run on this rank's
        compute stream, relative to its first step (synchronises); empty without HPB_PP_TRACE=2."""
        if not self.timeline:
            return []
        torch.cuda.synchronize()
        t0 = self.timeline[0][2]
        return [(lab, m, t0.elapsed_time(s), t0.elapsed_time(e)) for lab, m, s, e in self.timeline if e is not None]

    def run_microbatches(self, micro_args, micro_kwargs):
        prog = self.exec_order[self.real_stage_index]
        T = MetaStepType
        recv_f: Dict[Tuple[int, int], object] = {}
        recv_b: Dict[Tuple[int, int], object] = {}
        losses = [None] * self.micro_batch_num
        bwd_seen: Dict[int, int] = {}
        for st in self.stages:
            st.fwd_cache.clear()
            st.input_grads.clear()
        if self.timeline is not None:
            self.timeline = []

        def mark(label, micro):
            if self.timeline is None:
                return None
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.timeline.append([label, micro, ev, None])
            return self.timeline[-1]

        def done(rec):
            if rec is not None:
                rec[3] = torch.cuda.Event(enable_timing=True)
                rec[3].record()

        for step in prog:
            stage = self.stage_by_index[step.stage_index]
            m = step.micro_index
            if step.type == T.FWD_RECV:
                p = stage.post_forward_recv()
                if not self.overlap_p2p:
                    p.wait()
                recv_f[(step.stage_index, m)] = p
            elif step.type == T.FWD:
                if stage.is_first:
                    a, k = micro_args[m], micro_kwargs[m]
                else:
                    tok = self.tracer.start("fwd_recv_wait") if self.tracer else None
                    a, k = stage.finish_forward_recv(recv_f.pop((step.stage_index, m))), {}
                    if tok:
                        self.tracer.stop(tok)
                tok = self.tracer.start("fwd") if self.tracer else None
                rec = mark("F", m)
                out = stage.forward_one_chunk(m, a, k)
                done(rec)
                if tok:
                    self.tracer.stop(tok)
                if stage.is_last:
                    losses[m] = out
            elif step.type == T.FWD_SEND:
                stage.send_forward(m)
                if not self.overlap_p2p:
                    stage.wait_sends()
            elif step.type == T.BWD_RECV:
                p = stage.post_backward_recv()
                if not self.overlap_p2p:
                    p.wait()
                recv_b[(step.stage_index, m)] = p
            elif step.type == T.BWD:
                grads = None
                if not stage.is_last:
                    tok = self.tracer.start("bwd_recv_wait") if self.tracer else None
                    p = recv_b.pop((step.stage_index, m))
                    p.wait()
                    if tok:
                        self.tracer.stop(tok)
                    grads = [stage._rebuild(b, meta) for b, meta in zip(p.buffers, p.metas)]
                n = bwd_seen.get(step.stage_index, 0) + 1
                bwd_seen[step.stage_index] = n
                tok = self.tracer.start("bwd") if self.tracer else None
                rec = mark("B", m)
                stage.backward_one_chunk(m, grads, last_micro=(n == self.micro_batch_num))
                done(rec)
                if tok:
                    self.tracer.stop(tok)
            elif step.type == T.BWD_SEND:
                stage.send_backward(m)
                if not self.overlap_p2p:
                    stage.wait_sends()
        for st in self.stages:
            st.wait_sends()
            st.sync_shared_parameters_grad()
        if not any(st.is_last for st in self.stages):
            return None
        if self.output_concat_dim is not None and all(isinstance(l, torch.Tensor) for l in losses):
            return torch.cat([l if l.dim() > 0 else l.reshape(1) for l in losses], dim=self.output_concat_dim)
        return losses


class ScheduleGPipe(PipelineScheduleRuntime):
    """All forwards of every micro-batch, then all backwards (in reverse micro-batch order)."""

    def construct_stage_exec_order(self):
        M, S = self.micro_batch_num, self.real_stage_num
        if self.n_local != 1:
            raise ValueError("ScheduleGPipe takes exactly one stage per rank")
        order = {}
        for s in range(S):
            order[s] = [MetaStep(m, MetaStepType.FWD, s) for m in range(M)] + \
                       [MetaStep(m, MetaStepType.BWD, s) for m in range(M)]
        return order


class Schedule1F1B(PipelineScheduleRuntime):
    """Warm-up of ``min(S - s, M)`` forwards, then one-forward-one-backward, then drain."""

    def construct_stage_exec_order(self):
        M, S = self.micro_batch_num, self.real_stage_num
        if self.n_local != 1:
            raise ValueError("Schedule1F1B takes exactly one stage per rank")
        order = {}
        for s in range(S):
            warm = min(S - s, M)
            steps = [MetaStep(m, MetaStepType.FWD, s) for m in range(warm)]
            f, b = warm, 0
            while b < M:
                steps.append(MetaStep(b, MetaStepType.BWD, s))
                b += 1
                if f < M:
                    steps.append(MetaStep(f, MetaStepType.FWD, s))
                    f += 1
            order[s] = steps
        return order


class ScheduleInterleaved1F1B(PipelineScheduleRuntime):
    """Interleaved 1F1B (virtual pipeline): ``v`` chunks per rank, loop placement.

    Micro-batches advance in rounds of ``S`` (the first round takes the remainder when
    ``M % S != 0``; ``M < S`` is one short round).  Within a round a rank runs the round's
    micro-batches through chunk 0, then chunk 1, ...; backwards run the chunks in reverse.
    Warm-up on real stage ``s`` is ``(v - 1) * round0 + 2 * (S - s - 1)`` forwards (capped).
    """

    def construct_stage_exec_order(self):
        M, S, V = self.micro_batch_num, self.real_stage_num, self.n_local
        if self.stage_num != S * V:
            raise ValueError("every rank must hold the same number of virtual stages")
        rounds = []
        if M <= S:
            rounds = [list(range(M))]
        else:
            first = M % S or S
            rounds.append(list(range(first)))
            start = first
            while start < M:
                rounds.append(list(range(start, start + S)))
                start += S
        fwd_seq, bwd_seq = [], []
        for rd in rounds:
            for c in range(V):
                fwd_seq += [(m, c) for m in rd]
            for c in reversed(range(V)):
                bwd_seq += [(m, c) for m in rd]
        total = len(fwd_seq)
        if M % S == 0:
            return self._classic_order(fwd_seq, bwd_seq, S, V, total)
        caps = {s: min((V - 1) * len(rounds[0]) + 2 * (S - s - 1) + 1, total) for s in range(S)}
        return self._greedy_order(fwd_seq, bwd_seq, S, caps)

    def _classic_order(self, fwd_seq, bwd_seq, S, V, total):
        """The interleaved 1F1B program for ``M % S == 0``: on real stage ``s`` a warm-up of
        ``2 (S - s - 1) + (V - 1) S`` forwards, then strictly one forward, one backward, then the
        remaining backwards -- forwards and backwards each in the round order above.  A backward is
        never run early, which is what keeps the other ranks' steps aligned: the list scheduler
        below produces runs of ``S`` backwards followed by runs of ``S`` forwards, whose bubbles add
        up to more than the plain 1F1B bubble (simulated, 4 stages x 2 chunks, 16 micro-batches:
        60.0 against 57.0 time units; this order: 52.5)."""
        F, B = MetaStepType.FWD, MetaStepType.BWD
        order = {}
        for s in range(S):
            warm = min(2 * (S - s - 1) + (V - 1) * S, total)
            steps = [MetaStep(m, F, c * S + s) for m, c in fwd_seq[:warm]]
            for k in range(total - warm):
                m, c = fwd_seq[warm + k]
                steps.append(MetaStep(m, F, c * S + s))
                m, c = bwd_seq[k]
                steps.append(MetaStep(m, B, c * S + s))
            for m, c in bwd_seq[total - warm:]:
                steps.append(MetaStep(m, B, c * S + s))
            order[s] = steps
        return order

    def _greedy_order(self, fwd_seq, bwd_seq, S, caps):
        """Lock-step list scheduling: a rank runs its next backward as soon as it is ready,
        otherwise its next forward while fewer than ``caps[s]`` forwards are in flight.  If no
        rank can move, the cap of a rank with a ready forward is lifted for one step, so the
        result is always deadlock-free; for the regular cases it is the classic interleaved order."""
        F, B = MetaStepType.FWD, MetaStepType.BWD
        last = self.stage_num - 1
        order = {s: [] for s in range(S)}
        fi = {s: 0 for s in range(S)}
        bi = {s: 0 for s in range(S)}
        done = set()
        total = len(fwd_seq)
        while any(bi[s] < total for s in range(S)):
            picks = {}
            fwd_ready = {}
            for s in range(S):
                if bi[s] < total:
                    m, c = bwd_seq[bi[s]]
                    vs = c * S + s
                    if (F, m, vs) in done and (vs == last or (B, m, vs + 1) in done):
                        picks[s] = (B, m, vs)
                        continue
                if fi[s] < total:
                    m, c = fwd_seq[fi[s]]
                    vs = c * S + s
                    if vs == 0 or (F, m, vs - 1) in done:
                        fwd_ready[s] = (F, m, vs)
                        if fi[s] - bi[s] < caps[s]:
                            picks[s] = (F, m, vs)
            if not picks:
                if not fwd_ready:
                    raise RuntimeError("interleaved schedule cannot make progress")
                s = min(fwd_ready)
                picks[s] = fwd_ready[s]
            for s, (t, m, vs) in picks.items():
                order[s].append(MetaStep(m, t, vs))
                if t == F:
                    fi[s] += 1
                else:
                    bi[s] += 1
            done.update(picks.values())
        return order
