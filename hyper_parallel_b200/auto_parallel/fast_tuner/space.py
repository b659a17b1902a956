"""N-D search space and rule-based ("expert") pruning.

Item format (hyper_parallel/auto_parallel/fast-tuner/fast_tuner/ndsearch/build_initial_spaces.py:44-116):
``[[(dp, tp, cp, pp), (ep, op, vp, mbs)], sp]`` -- every factorisation of the world size into
(dp, tp, cp, pp); ``ep`` in {1, even numbers <= expert_num}; ``op`` (optimizer / FSDP shard degree)
a divisor of dp, or ``-1`` = "takes what is left" when FSDP is not searched; ``vp`` in
``[1, ceil(L / pp))``; ``mbs`` in {1, 2, 4}; ``sp`` False, plus True when tp > 1.

Rules (expert_filter_configs.py:101-200): cp == 1, tp <= 64, ep <= 64, sp forced on at >= 1000
ranks, pp <= min(L, gbs / dp / mbs), gbs % dp == 0, the TorchTitan EP constraints
``ep % (cp*tp) == 0`` and ``(op*cp*tp) % ep == 0``, pp <= 32, tp % 3 != 0.
"""
from __future__ import annotations

import itertools
import math
from typing import Callable, List

from .config import ModelSpec, Strategy

Config = list  # [[(dp,tp,cp,pp),(ep,op,vp,mbs)], sp]


def divisors(n: int) -> List[int]:
    return [d for d in range(1, n + 1) if n % d == 0]


def factorizations4(world: int):
    """All ordered (dp, tp, cp, pp) with product ``world``."""
    out = []
    for dp in divisors(world):
        r1 = world // dp
        for tp in divisors(r1):
            r2 = r1 // tp
            for cp in divisors(r2):
                out.append((dp, tp, cp, r2 // cp))
    return out


def build_initial_spaces(spec: ModelSpec, strategy: Strategy = Strategy(DP=True, TP=True, PP=True, EP=True,
                                                                       CP=True, FSDP=True)) -> List[Config]:
    part1 = factorizations4(spec.world_size)
    if not strategy.DP:
        part1 = [c for c in part1 if c[0] == 1]
    if not strategy.TP:
        part1 = [c for c in part1 if c[1] == 1]
    if not strategy.CP:
        part1 = [c for c in part1 if c[2] == 1]
    if not strategy.PP:
        part1 = [c for c in part1 if c[3] == 1]
    ep_options = [1] if not spec.expert_num else [i for i in range(1, spec.expert_num + 1) if i == 1 or i % 2 == 0]
    if not strategy.EP:
        ep_options = [1]
    out: List[Config] = []
    for dp, tp, cp, pp in part1:
        # interleave depths: 1 without a pipeline, else every depth below ceil(layers / pp)
        vp_options = [1] if pp == 1 else list(range(1, math.ceil(spec.num_layers / pp)))
        for ep, op, vp, mbs in itertools.product(ep_options, divisors(dp), vp_options, (1, 2, 4)):
            if not strategy.FSDP and op != dp:
                op = -1
            item = [(dp, tp, cp, pp), (ep, op, vp, mbs)]
            out.append([item, False])
            if tp != 1:
                out.append([item, True])
    return out


# accessors ---------------------------------------------------------------------------
def dp_of(c): return c[0][0][0]
def tp_of(c): return c[0][0][1]
def cp_of(c): return c[0][0][2]
def pp_of(c): return c[0][0][3]
def ep_of(c): return c[0][1][0]
def op_of(c): return c[0][1][1]
def vp_of(c): return c[0][1][2]
def mbs_of(c): return c[0][1][3]
def sp_of(c): return c[1]
def world_of(c): return dp_of(c) * tp_of(c) * cp_of(c) * pp_of(c)


class ExpertFilterManager:
    """Ordered list of pruning rules; each rule maps a candidate list to a shorter one."""

    def __init__(self, spec: ModelSpec, gbs: int):
        self.spec, self.gbs = spec, gbs
        self.expert_filters: List[Callable[[List[Config]], List[Config]]] = []

    def add_experience(self, fn) -> None:
        if fn not in self.expert_filters:
            self.expert_filters.append(fn)

    def remove_experience(self, fn) -> None:
        if fn in self.expert_filters:
            self.expert_filters.remove(fn)

    def sequential_combination(self, filters, space: List[Config]) -> List[Config]:
        for f in filters:
            if not space:
                break
            space = f(space)
        return space

    # rules -------------------------------------------------------------------------
    def cp_for_deepseek_expert(self, s): return [c for c in s if cp_of(c) == 1]
    def tp_for_large_scale_expert(self, s): return [c for c in s if tp_of(c) <= 64]
    def tp_for_node_expert(self, s, per_node=8): return [c for c in s if tp_of(c) <= per_node]
    def ep_for_large_scale_expert(self, s): return [c for c in s if ep_of(c) <= 64]
    def pp_for_768die(self, s): return [c for c in s if pp_of(c) <= 32]
    def tp_for_large_scale_768die(self, s): return [c for c in s if tp_of(c) % 3 != 0]
    def pp_for_deepseek(self, s): return [c for c in s if pp_of(c) > 1]
    def gbs_for_dp_expert(self, s): return [c for c in s if self.gbs % dp_of(c) == 0]
    def dp_cp_ep_for_megatron_expert(self, s): return [c for c in s if dp_of(c) * cp_of(c) % ep_of(c) == 0]

    def sp_for_lm_expert(self, s):
        if not s:
            return s
        w = world_of(s[0])
        return [c for c in s if w < 1000 or tp_of(c) == 1 or sp_of(c)]

    def pp_for_mbs_expert(self, s):
        L = self.spec.num_layers
        return [c for c in s if pp_of(c) <= min(L, self.gbs // dp_of(c) // mbs_of(c))]

    def ep_for_torchtitan(self, s):
        out = []
        for c in s:
            ep, cp, tp, op = ep_of(c), cp_of(c), tp_of(c), op_of(c)
            if ep % (cp * tp) == 0 and (op * cp * tp) % ep == 0:
                out.append(c)
        return out

    def ep_for_mindspore(self, s):
        return [c for c in s if op_of(c) % ((dp_of(c) * tp_of(c)) / ep_of(c)) == 0]


def expert_filter_configs(space: List[Config], spec: ModelSpec, gbs: int) -> List[Config]:
    m = ExpertFilterManager(spec, gbs)
    for rule in (m.cp_for_deepseek_expert, m.tp_for_large_scale_expert, m.ep_for_large_scale_expert,
                 m.sp_for_lm_expert, m.pp_for_mbs_expert, m.gbs_for_dp_expert, m.ep_for_torchtitan,
                 m.pp_for_768die, m.tp_for_large_scale_768die):
        m.add_experience(rule)
    return m.sequential_combination(m.expert_filters, space)
