"""Profile preparation, launch and parsing.

Roles of hyper_parallel/auto_parallel/fast-tuner/fast_tuner/utils/profiling/profile_prepare.py,
profile_launch.py and profile_parser.py of the reference, adapted to this framework's own
records: a candidate is shrunk to the ranks that are available, the trainer is launched in its own
process group, and per-layer times are read from the JSON lines that ``hyper_parallel_b200.utils.
tracing.LayerTimer`` writes (CUDA-event durations per module and phase) instead of vendor kernel CSVs.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
from dataclasses import dataclass
from typing import Dict, List, Optional

from .config import ModelSpec
from .pipeline_balance import LayerProfile
from .space import Config, cp_of, ep_of, tp_of


@dataclass
class ProfileInfo:
    dense_fw: float = 0.0
    dense_bw: float = 0.0
    moe_fw: float = 0.0
    moe_bw: float = 0.0
    recompute_bw: float = 0.0
    head: float = 0.0
    embed: float = 0.0

    @property
    def layer_ratio(self) -> float:
        d = self.moe_fw + self.moe_bw
        return (self.dense_fw + self.dense_bw) / d if d else 1.0

    @property
    def backward_ratio(self) -> float:
        return self.moe_bw / self.moe_fw if self.moe_fw else (self.dense_bw / self.dense_fw if self.dense_fw else 2.0)

    def to_layer_profile(self) -> LayerProfile:
        return LayerProfile(dense_fw=self.dense_fw or 1.0, dense_bw=self.dense_bw or 2.0,
                            moe_fw=self.moe_fw or self.dense_fw or 1.0, moe_bw=self.moe_bw or self.dense_bw or 2.0,
                            head_fw=self.head / 3.0, head_bw=self.head * 2.0 / 3.0,
                            embed_fw=self.embed / 3.0, embed_bw=self.embed * 2.0 / 3.0,
                            recompute_extra=(self.recompute_bw / self.dense_fw) if (self.recompute_bw and self.dense_fw) else 1.0)


def shrink_candidate(c: Config, rank_num: int) -> Optional[Config]:
    """Scale a candidate down to ``rank_num`` ranks for profiling: pp -> 1, then divide dp (and the
    FSDP degree) by the overshoot; candidates whose FSDP degree would reach 0 are dropped."""
    dp, tp, cp, pp = c[0][0]
    ep, op, vp, mbs = c[0][1]
    world = dp * tp * cp
    if tp * cp > rank_num:
        return None
    factor = max(world // rank_num, 1)
    if world % rank_num and world > rank_num:
        return None
    new_dp = max(dp // factor, 1)
    new_op = op if op == -1 else op // factor
    if new_op == 0:
        return None
    new_ep = min(ep, new_dp * tp)
    return [[(new_dp, tp, cp, 1), (new_ep, new_op, 1, mbs)], c[1]]


def select_profile_candidates(space: List[Config], rank_num: int, limit: int = 10) -> List[Config]:
    """At most ``limit`` distinct shrunk candidates, preferring small tp, small cp, large ep."""
    seen, out = set(), []
    for c in sorted(space, key=lambda c: (tp_of(c), cp_of(c), -ep_of(c))):
        s = shrink_candidate(c, rank_num)
        if s is None:
            continue
        key = (s[0][0], s[0][1][0], s[0][1][1], s[0][1][3], s[1])
        if key in seen:
            continue
        seen.add(key)
        out.append(s)
        if len(out) >= limit:
            break
    return out


def write_profile_config(c: Config, spec: ModelSpec, out_dir: str, idx: int) -> str:
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, f"profile_{idx:03d}.json")
    (dp, tp, cp, pp), (ep, op, vp, mbs) = c[0]
    with open(path, "w") as f:
        json.dump({"dp": dp, "tp": tp, "cp": cp, "pp": pp, "ep": ep, "op": op, "vp": vp, "mbs": mbs, "sp": c[1],
                   "model": {k: getattr(spec, k) for k in spec.__dataclass_fields__}}, f, indent=1)
    return path


BUILTIN_TRAINER = "hyper_parallel_b200.auto_parallel.fast_tuner.profile_trainer"


def launch_profile(config_path: str, trainer: Optional[str], nproc: int, timeout: int = 1800, env=None,
                   port: int = 29591) -> int:
    """Run the trainer (``python -m torch.distributed.run ... trainer --profile-config path``) in its own
    process group so that a timeout can end exactly the processes that were started.  ``trainer`` is a
    script path, a module name, or ``None`` for this package's own :mod:`profile_trainer`."""
    trainer = trainer or BUILTIN_TRAINER
    target = [trainer] if trainer.endswith(".py") else ["-m", trainer]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), *target, "--profile-config", config_path]
    proc = subprocess.Popen(cmd, env={**os.environ, **(env or {})}, start_new_session=True)
    try:
        return proc.wait(timeout=timeout)
    except subprocess.TimeoutExpired:
        os.killpg(proc.pid, 15)
        return -1


def parse_layer_records(path: str) -> ProfileInfo:
    """Aggregate ``{"module": kind, "phase": "fwd"|"bwd"|"recompute", "ms": t}`` JSON lines into per-layer means."""
    sums: Dict[tuple, List[float]] = {}
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            r = json.loads(line)
            sums.setdefault((r["module"], r["phase"]), []).append(float(r["ms"]))
    mean = lambda k: (sum(sums[k]) / len(sums[k])) if k in sums else 0.0  # noqa: E731
    return ProfileInfo(dense_fw=mean(("dense", "fwd")), dense_bw=mean(("dense", "bwd")),
                       moe_fw=mean(("moe", "fwd")), moe_bw=mean(("moe", "bwd")),
                       recompute_bw=mean(("dense", "recompute")),
                       head=mean(("head", "fwd")) + mean(("head", "bwd")),
                       embed=mean(("embed", "fwd")) + mean(("embed", "bwd")))
