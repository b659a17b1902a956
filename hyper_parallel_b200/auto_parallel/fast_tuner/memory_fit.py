"""Correction of the balancer's memory model from measured peaks.

Role of hyper_parallel/auto_parallel/fast-tuner/fast_tuner/pipeline_conductor/fitting.py:28-360 of
the reference (``FitMem``): the balancer places layers and recompute counts under a per-stage memory
limit using a linear model of the peak,

    peak[s] = static + layers[s] * layer + head * [s is last]
              + ((layers[s] - recomputed[s]) * act + recomputed[s] * recomp) * live[s] / chunks

whose five coefficients first come from an estimate.  After a dry run (or a short real run) has
reported the true peak of every stage, the coefficients are re-fitted by non-negative least squares
over all observations so far and the balance is repeated; the loop ends when the measured peaks fit
the limit, or after a few rounds with the limit tightened by the remaining overshoot, as the
reference does (``reduce_mem_lim_for_fitting``).
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Callable, List, Optional, Sequence

import numpy as np

from .pipeline_balance import BalanceResult, LayerProfile, balance_pipeline

_FIELDS = ("static_mem", "layer_mem", "lm_head_mem", "act_mem", "recomp_mem")


@dataclass
class MemoryObservation:
    """One stage of one run: what was placed there and the peak (MB) that was measured."""
    layers: int
    recomputed: int
    live: float            # peak number of live micro-batch activations on the stage / chunks
    is_last: bool
    peak_mb: float

    def row(self) -> List[float]:
        return [1.0, float(self.layers), 1.0 if self.is_last else 0.0,
                (self.layers - self.recomputed) * self.live, self.recomputed * self.live]


def observations_of(result: BalanceResult, measured_mb: Sequence[float], peak_live: Sequence[int]) -> List[MemoryObservation]:
    """Observations of one balanced pipeline: ``measured_mb[s]`` is the peak of stage ``s``,
    ``peak_live[s]`` the simulator's peak count of live micro-batches there."""
    V, S = len(result.layers), len(result.layers[0])
    out = []
    for s in range(S):
        n = sum(result.layers[c][s] for c in range(V))
        r = sum(result.recompute[c][s] for c in range(V))
        out.append(MemoryObservation(n, r, max(peak_live[s], 1) / max(V, 1), s == S - 1, float(measured_mb[s])))
    return out


def predict(prof: LayerProfile, obs: MemoryObservation) -> float:
    return float(np.dot(obs.row(), [getattr(prof, f) for f in _FIELDS]))


def fit_memory(observations: Sequence[MemoryObservation], prior: LayerProfile) -> LayerProfile:
    """Non-negative least-squares fit of the five memory coefficients.  Coefficients that the
    observations cannot tell apart (a column that is zero or a copy of another, e.g. no stage ever
    recomputed a layer) keep the prior's value: the fit runs on the residual against those."""
    from scipy.optimize import nnls
    if not observations:
        return prior
    A = np.array([o.row() for o in observations], dtype=np.float64)
    y = np.array([o.peak_mb for o in observations], dtype=np.float64)
    x0 = np.array([getattr(prior, f) for f in _FIELDS], dtype=np.float64)
    free = []
    for j in range(A.shape[1]):
        col = A[:, j]
        if not np.any(col):
            continue
        # identifiable only if adding the column raises the rank of what is already free
        if np.linalg.matrix_rank(A[:, free + [j]]) > len(free):
            free.append(j)
    fixed = [j for j in range(A.shape[1]) if j not in free]
    resid = y - A[:, fixed] @ x0[fixed] if fixed else y
    x = x0.copy()
    if free:
        scale = np.maximum(np.abs(A[:, free]).max(axis=0), 1e-12)      # condition the columns
        sol, _ = nnls(A[:, free] / scale, resid)
        x[free] = sol / scale
    return replace(prior, **{f: float(v) for f, v in zip(_FIELDS, x)})


@dataclass
class FitRound:
    result: BalanceResult
    measured_mb: List[float]
    profile: LayerProfile
    limit_used: float
    over_mb: float


def balance_with_memory_feedback(num_layers: int, num_dense: int, stages: int, chunks: int, micro: int,
                                 prof: LayerProfile, mem_limit_mb: float,
                                 measure: Callable[[BalanceResult], Sequence[float]],
                                 p2p: float = 0.0, max_rounds: int = 4, peak_live: Optional[Sequence[int]] = None,
                                 **balance_kw) -> List[FitRound]:
    """Balance -> measure -> re-fit -> balance again, until every measured stage peak is within
    ``mem_limit_mb`` or ``max_rounds`` is reached.  ``measure(result)`` returns the true per-stage peaks
    (MB) of a balanced pipeline -- a dry run, or a few steps of the real job.  Returns the rounds in
    order; the last one is the answer (its ``over_mb`` is 0 when it fits)."""
    from .pp_simulator import compute_order, simulate
    rounds: List[FitRound] = []
    seen: List[MemoryObservation] = []
    limit = mem_limit_mb
    kind = "vpp" if chunks > 1 else "1f1b"
    for _ in range(max_rounds):
        res = balance_pipeline(num_layers, num_dense, stages, chunks, micro, prof, mem_limit_mb=limit, p2p=p2p,
                               **balance_kw)
        measured = [float(m) for m in measure(res)]
        live = peak_live
        if live is None:
            unit = [1.0] * (stages * chunks)
            live = simulate(compute_order(kind, micro, stages, chunks), unit, [2.0 * u for u in unit], stages).peak_live
        over = max(max(measured) - mem_limit_mb, 0.0)
        rounds.append(FitRound(res, measured, prof, limit, over))
        if over <= 0.0:
            break
        seen += observations_of(res, measured, live)
        new_prof = fit_memory(seen, prof)
        same_model = all(abs(getattr(new_prof, f) - getattr(prof, f)) <= 1e-6 * max(abs(getattr(prof, f)), 1.0)
                         for f in _FIELDS)
        prof = new_prof
        # the corrected model explains the overshoot -> balance against the true limit again; if the
        # model did not move (nothing left to learn) tighten the limit by what is still over
        limit = mem_limit_mb if not same_model else limit - over
    return rounds
