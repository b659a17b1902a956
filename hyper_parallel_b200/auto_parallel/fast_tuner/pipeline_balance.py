"""Layer-to-stage balancing for pipeline parallelism with two layer types and recomputation.

The reference formulates this as a MILP (OR-Tools -> MPS -> HiGHS,
hyper_parallel/auto_parallel/fast-tuner/fast_tuner/pipeline_conductor/math_model.py:30-486): integer
layer counts per (stage, virtual chunk) for dense ("type 1") and MoE ("type 2") layers, dense
layers occupying a prefix of the (chunk, stage) sequence, a number of fully recomputed layers per
slot, per-stage memory limits, objective = end of the last backward under a fixed 1F1B / VPP
order.  Neither solver is installed here, so the same model is solved natively: a bounded
depth-first search over the layer distribution with the discrete-event simulator as the exact
objective, pruned by the load lower bound, followed by a greedy choice of the recompute counts
that makes each stage fit its memory limit at the least extra time.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

from .pp_simulator import CompiledOrder, compute_order, simulate


@dataclass
class LayerProfile:
    """Per-layer times (any unit) and memory (MB) of the two layer types."""
    dense_fw: float = 1.0
    dense_bw: float = 2.0
    moe_fw: float = 1.0
    moe_bw: float = 2.0
    head_fw: float = 0.0          # output head + loss on the last virtual stage
    head_bw: float = 0.0
    embed_fw: float = 0.0         # embedding on the first virtual stage
    embed_bw: float = 0.0
    recompute_extra: float = 1.0  # extra backward time of a fully recomputed layer, in units of its forward
    select_extra: float = 0.3     # the same for a selectively recomputed layer (attention core / activations only)
    act_mem: float = 1.0          # activation MB per layer per live micro-batch
    recomp_mem: float = 0.1       # the same for a fully recomputed layer
    select_mem: Optional[float] = None    # the same for a selectively recomputed layer; None: no selective recompute
    layer_mem: float = 1.0        # static MB per layer (weights + optimizer)
    static_mem: float = 0.0       # static MB per stage
    lm_head_mem: float = 0.0
    # MoE layers where they differ from dense ones, and the first stage (embedding) where it differs
    # from the others (the reference's memory table keeps both apart, pipeline_conductor/memory.py:28-60)
    moe_act_mem: Optional[float] = None
    moe_recomp_mem: Optional[float] = None
    moe_select_mem: Optional[float] = None
    moe_layer_mem: Optional[float] = None
    static_mem0: Optional[float] = None

    def mem_of(self, moe: bool):
        """``(act, recomp, select, layer)`` MB of a dense or a MoE layer."""
        pick = (lambda m, d: d if m is None else m) if moe else (lambda m, d: d)
        return (pick(self.moe_act_mem, self.act_mem), pick(self.moe_recomp_mem, self.recomp_mem),
                pick(self.moe_select_mem, self.select_mem), pick(self.moe_layer_mem, self.layer_mem))


@dataclass
class BalanceResult:
    layers: List[List[int]]                # [chunk][stage] total layers
    dense: List[List[int]]                 # [chunk][stage] dense layers
    recompute: List[List[int]]             # [chunk][stage] fully recomputed layers
    makespan: float
    bubble_ratio: float
    peak_mem: List[float]
    offset: List[List[int]] = field(default_factory=list)   # deviation from the even split
    select_recompute: List[List[int]] = field(default_factory=list)   # [chunk][stage] selectively recomputed layers


def _slot_times(dense, moe, rec, prof: LayerProfile, S: int, V: int, sel=None):
    fwd, bwd = [], []
    for v in range(S * V):
        c, s = divmod(v, S)
        d, m, r = dense[c][s], moe[c][s], rec[c][s]
        f = d * prof.dense_fw + m * prof.moe_fw
        b = d * prof.dense_bw + m * prof.moe_bw
        total = d + m
        if total and r:
            avg_fw = f / total
            b += r * avg_fw * prof.recompute_extra
        if total and sel is not None and sel[c][s]:
            b += sel[c][s] * (f / total) * prof.select_extra
        if v == 0:
            f += prof.embed_fw
            b += prof.embed_bw
        if v == S * V - 1:
            f += prof.head_fw
            b += prof.head_bw
        fwd.append(f)
        bwd.append(b)
    return fwd, bwd


def _split_types(layers, n_dense: int):
    """Dense layers fill the (chunk, stage) sequence from the front; the rest is MoE."""
    dense = [[0] * len(layers[0]) for _ in layers]
    moe = [[0] * len(layers[0]) for _ in layers]
    left = n_dense
    for c in range(len(layers)):
        for s in range(len(layers[0])):
            d = min(left, layers[c][s])
            dense[c][s] = d
            moe[c][s] = layers[c][s] - d
            left -= d
    return dense, moe


def balance_pipeline(num_layers: int, num_dense: int, stages: int, chunks: int, micro: int,
                     prof: LayerProfile, mem_limit_mb: Optional[float] = None, p2p: float = 0.0,
                     max_offset: int = 2, max_nodes: int = 4000) -> BalanceResult:
    S, V = stages, chunks
    slots = S * V
    kind = "vpp" if V > 1 else "1f1b"
    order = compute_order(kind, micro, S, V)
    base, rem = divmod(num_layers, slots)
    even = [base + (1 if i < rem else 0) for i in range(slots)]
    best = {"t": float("inf"), "x": None}
    nodes = [0]
    fast = CompiledOrder(order, slots, S)        # the search only needs the makespan
    zero = [[0] * S for _ in range(V)]

    def objective(flat: Sequence[int]) -> float:
        layers = [[flat[c * S + s] for s in range(S)] for c in range(V)]
        dense, moe = _split_types(layers, num_dense)
        fwd, bwd = _slot_times(dense, moe, zero, prof, S, V)
        return fast.makespan(fwd, bwd, p2p)

    def evaluate(flat: Sequence[int]):
        layers = [[flat[c * S + s] for s in range(S)] for c in range(V)]
        dense, moe = _split_types(layers, num_dense)
        zero = [[0] * S for _ in range(V)]
        fwd, bwd = _slot_times(dense, moe, zero, prof, S, V)
        return simulate(order, fwd, bwd, S, p2p), layers, dense, moe

    avg_layer = ((prof.dense_fw + prof.dense_bw) * num_dense +
                 (prof.moe_fw + prof.moe_bw) * (num_layers - num_dense)) / max(num_layers, 1)

    def dfs(i: int, flat: List[int], left: int):
        if nodes[0] >= max_nodes:
            return
        if i == slots - 1:
            if left < 0 or abs(left - even[i]) > max_offset + 1:
                return
            cand = flat + [left]
            nodes[0] += 1
            t = objective(cand)
            if t < best["t"]:
                best["t"], best["x"] = t, cand
            return
        for delta in sorted(range(-max_offset, max_offset + 1), key=abs):
            n = even[i] + delta
            if n < 0 or n > left:
                continue
            # lower bound: the most loaded stage cannot finish before its own work
            stage_load = sum(flat[j] for j in range(len(flat)) if j % S == i % S) + n
            if stage_load * avg_layer * micro >= best["t"]:
                continue
            dfs(i + 1, flat + [n], left - n)

    res0, *_ = evaluate(even)
    best["t"], best["x"] = res0.makespan, list(even)
    dfs(0, [], num_layers)
    res, layers, dense, moe = evaluate(best["x"])
    rec = [[0] * S for _ in range(V)]
    sel = [[0] * S for _ in range(V)]
    peak_mem = _stage_memory(layers, rec, res.peak_live, prof, S, V, dense, sel)
    if mem_limit_mb is not None:
        limits = list(mem_limit_mb) if isinstance(mem_limit_mb, (list, tuple)) else [float(mem_limit_mb)] * S
        if len(limits) != S:
            raise ValueError(f"mem_limit_mb needs one value or one per stage ({S}), got {len(limits)}")
        # greedy: on the stage that exceeds its limit the most, take the move (selectively recompute one
        # more layer / fully recompute one more layer, per chunk) that frees the most memory per unit
        # of extra backward time
        for _ in range(4 * num_layers):
            over = [(peak_mem[s] - limits[s], s) for s in range(S) if peak_mem[s] > limits[s] + 1e-9]
            if not over:
                break
            _, s = max(over)
            best_move, best_score = None, 0.0
            for c in range(V):
                n = layers[c][s]
                if not n:
                    continue
                avg_fw = (dense[c][s] * prof.dense_fw + moe[c][s] * prof.moe_fw) / n
                moves = []
                if rec[c][s] + sel[c][s] < n:
                    moves.append(("rec", 0, prof.recompute_extra))
                    if prof.select_mem is not None or prof.moe_select_mem is not None:
                        moves.append(("sel", 0, prof.select_extra))
                if sel[c][s] > 0:
                    moves.append(("rec", -1, prof.recompute_extra - prof.select_extra))   # upgrade a selected layer
                for kind, dsel, extra in moves:
                    rec[c][s] += kind == "rec"
                    sel[c][s] += (kind == "sel") + dsel
                    saved = peak_mem[s] - _stage_memory(layers, rec, res.peak_live, prof, S, V, dense, sel)[s]
                    rec[c][s] -= kind == "rec"
                    sel[c][s] -= (kind == "sel") + dsel
                    score = saved / max(extra * avg_fw, 1e-9)
                    if saved > 1e-9 and score > best_score:
                        best_move, best_score = (c, kind, dsel), score
            if best_move is None:
                break
            c, kind, dsel = best_move
            rec[c][s] += kind == "rec"
            sel[c][s] += (kind == "sel") + dsel
            peak_mem = _stage_memory(layers, rec, res.peak_live, prof, S, V, dense, sel)
        fwd, bwd = _slot_times(dense, moe, rec, prof, S, V, sel)
        res = simulate(order, fwd, bwd, S, p2p)
    offset = [[layers[c][s] - even[c * S + s] for s in range(S)] for c in range(V)]
    return BalanceResult(layers, dense, rec, res.makespan, res.bubble_ratio, peak_mem, offset, sel)


def _stage_memory(layers, rec, peak_live, prof: LayerProfile, S: int, V: int, dense=None, sel=None) -> List[float]:
    """Peak MB of every stage: static part (per stage, per layer by type, the head on the last stage)
    plus the activations of the live micro-batches.  ``dense[c][s]`` of the ``layers[c][s]`` layers
    are dense (all of them when not given); ``rec`` / ``sel`` of them are fully / selectively
    recomputed -- MoE layers first, their activations being the larger ones."""
    out = []
    act_d, rec_d, sel_d, lay_d = prof.mem_of(False)
    act_m, rec_m, sel_m, lay_m = prof.mem_of(True)
    sel_d = act_d if sel_d is None else sel_d
    sel_m = act_m if sel_m is None else sel_m
    for s in range(S):
        live = max(peak_live[s], 1) / max(V, 1)
        static = prof.static_mem0 if (s == 0 and prof.static_mem0 is not None) else prof.static_mem
        if s == S - 1:
            static += prof.lm_head_mem
        act = 0.0
        for c in range(V):
            n = layers[c][s]
            d = n if dense is None else dense[c][s]
            m = n - d
            r = rec[c][s]
            q = sel[c][s] if sel is not None else 0
            r_m = min(r, m)
            r_d = r - r_m
            q_m = min(q, m - r_m)
            q_d = q - q_m
            static += d * lay_d + m * lay_m
            act += ((d - r_d - q_d) * act_d + r_d * rec_d + q_d * sel_d +
                    (m - r_m - q_m) * act_m + r_m * rec_m + q_m * sel_m)
        out.append(static + act * live)
    return out


def layer_ranges(layers: Sequence[Sequence[int]]) -> List[tuple]:
    """``[chunk][stage]`` layer counts -> ``(first, end)`` layer range of every virtual stage, in model
    order (virtual stage ``v = chunk * stages + stage``): what a pipeline runtime needs to build
    the module of each virtual stage from a :class:`BalanceResult`."""
    out, lo = [], 0
    for row in layers:
        for n in row:
            out.append((lo, lo + int(n)))
            lo += int(n)
    return out


def dense_transformer_profile(hidden: int, ffn: int, heads: int, kv_heads: int, head_dim: int, vocab: int,
                              seq_len: int) -> LayerProfile:
    """Analytic :class:`LayerProfile` of a dense decoder (times in GFLOP per token, backward = 2 x
    forward): enough to place the output head, which costs ``2 * hidden * vocab`` per token -- more
    than two layers of an 8B model with a 128k vocabulary -- on a stage with fewer layers."""
    mm = (heads + 2 * kv_heads) * head_dim * hidden + heads * head_dim * hidden + 3 * hidden * ffn
    layer = (2.0 * mm + 4.0 * heads * head_dim * seq_len / 2) / 1e9
    head = 2.0 * hidden * vocab / 1e9
    return LayerProfile(dense_fw=layer, dense_bw=2 * layer, moe_fw=layer, moe_bw=2 * layer,
                        head_fw=head, head_bw=2 * head)
