"""``fast-tuner-pipeline``: rank the candidates of an earlier search by pipeline cost.

Stand-alone second phase, the role of hyper_parallel/auto_parallel/fast-tuner/fast_tuner/pipeline_tool.py:26-70
of the reference: the first phase (``parallel_tool --alg_phase 1``) leaves ``nd_candidate_config.csv``
(dp, tp, pp, ep, cp, op and the estimated memory); this tool reads it, expands every row over the
interleave depths up to ``--max_vpp`` and the micro-batch sizes, takes per-layer times either from a
profile (``--parser_result``: the records file a profiling run wrote) or from the ratios below,
balances every pipelined candidate, replays the best in the schedule simulator and writes
``pipeline_output/ranked_configs.csv`` with one text and one SVG drawing per candidate.

Ratios (names of the reference's ``args_for_pipeline_parallel.json``), used when no profile is given:
``--backward_ratio`` backward / forward time of a layer, ``--layer_ratio`` MoE / dense forward time,
``--head_loss`` output head + loss in units of one dense layer, ``--recompute_ratio`` extra backward
time of a recomputed layer in units of its forward.
"""
from __future__ import annotations

import argparse
import csv
import sys
from typing import List, Optional

from .config import ModelSpec, TunerConfig, load_model_spec
from .parallel_tool import rank_candidates
from .pipeline_balance import LayerProfile
from .profiling import parse_layer_records
from .space import Config


def read_candidates(path: str, spec: ModelSpec, gbs: int, max_vpp: int = 2,
                    mbs_choices: Optional[List[int]] = None) -> List[Config]:
    """Rows of ``nd_candidate_config.csv`` -> search-space entries ``[[(dp, tp, cp, pp), (ep, op, vp, mbs)], sp]``.

    The file has no interleave depth, micro-batch size or sequence-parallel flag: every row is
    expanded over ``vp`` in 1..``max_vpp`` (only depths that leave at least one layer per virtual
    stage; 1 when there is no pipeline), over the micro-batch sizes that divide the per-replica batch,
    and sequence parallelism is on wherever ``tp > 1``.  Duplicated rows collapse."""
    out, seen = [], set()
    with open(path, newline="") as f:
        for row in csv.DictReader(f):
            dp, tp, pp, ep = (int(row[k]) for k in ("dp", "tp", "pp", "ep"))
            cp, op = int(row.get("cp") or 1), int(row.get("op") or 1)
            per_replica = max(gbs // max(dp, 1), 1)
            sizes = [m for m in (mbs_choices or [1, 2, 4]) if per_replica % m == 0] or [1]
            depths = [v for v in range(1, max_vpp + 1) if pp * v <= spec.num_layers] if pp > 1 else [1]
            for vp in depths:
                for mbs in sizes:
                    key = (dp, tp, cp, pp, ep, op, vp, mbs)
                    if key in seen:
                        continue
                    seen.add(key)
                    out.append([[(dp, tp, cp, pp), (ep, op, vp, mbs)], tp > 1])
    return out


def profile_from_ratios(backward_ratio: float = 2.0, layer_ratio: float = 1.0, head_loss: float = 0.0,
                        recompute_ratio: float = 1.0) -> LayerProfile:
    return LayerProfile(dense_fw=1.0, dense_bw=backward_ratio, moe_fw=layer_ratio, moe_bw=layer_ratio * backward_ratio,
                        head_fw=head_loss, head_bw=head_loss * backward_ratio, recompute_extra=recompute_ratio)


def pipeline_search_tool(cfg: TunerConfig, nd_path: str, spec: Optional[ModelSpec] = None,
                         lp: Optional[LayerProfile] = None, max_vpp: int = 2, top_k: int = 20,
                         mbs_choices: Optional[List[int]] = None) -> List[dict]:
    spec = spec or load_model_spec(cfg)
    space = read_candidates(nd_path, spec, cfg.gbs, max_vpp, mbs_choices)
    if not space:
        raise ValueError(f"{nd_path} lists no candidate")
    return rank_candidates(space, spec, cfg, None, lp, top_k)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="fast-tuner-pipeline", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config", help="json file with the keys of the parallel tool (model, cluster, output_path)")
    ap.add_argument("--nd_path", required=True, help="nd_candidate_config.csv of an earlier search")
    ap.add_argument("--toml_path"); ap.add_argument("--yaml_path"); ap.add_argument("--shell_path")
    ap.add_argument("--model_json")
    ap.add_argument("--rank_num", type=int); ap.add_argument("--gbs", type=int)
    ap.add_argument("--npus_per_node", "--gpus_per_node", dest="gpus_per_node", type=int)
    ap.add_argument("--output_path")
    ap.add_argument("--parser_result", help="records file (.jsonl) of a profiling run: measured per-layer times")
    ap.add_argument("--backward_ratio", type=float, default=2.0)
    ap.add_argument("--layer_ratio", type=float, default=1.0)
    ap.add_argument("--head_loss", type=float, default=0.0)
    ap.add_argument("--recompute_ratio", type=float, default=1.0)
    ap.add_argument("--max_vpp", type=int, default=2)
    ap.add_argument("--mbs", type=int, nargs="*", help="micro-batch sizes to try (default 1 2 4)")
    ap.add_argument("--topn", type=int, default=20)
    ap.add_argument("--select_recompute", action="store_true")
    ap.add_argument("--profile_data_dir", help="folder of a profiling run; its first *.records.jsonl is the profile "
                                               "when --parser_result is not given")
    # accepted for command lines written for the reference's tool; they have no effect here (no external
    # trainer is driven, the balancer is the built-in one, the re-check is the schedule simulator)
    for flag in ("--files_dir", "--mindformers_dir", "--mindspeed_path", "--solver_name", "--env_json",
                 "--register_path", "--parallel_num", "--dryrun", "--check"):
        ap.add_argument(flag, help=argparse.SUPPRESS)
    ns = ap.parse_args(argv)
    if not ns.parser_result and ns.profile_data_dir:
        import glob
        import os
        found = sorted(glob.glob(os.path.join(ns.profile_data_dir, "*.records.jsonl")))
        ns.parser_result = found[0] if found else None
    cfg = TunerConfig.from_json(ns.config) if ns.config else TunerConfig()
    for k in ("toml_path", "yaml_path", "shell_path", "model_json", "rank_num", "gbs", "gpus_per_node", "output_path"):
        if getattr(ns, k) is not None:
            setattr(cfg, k, getattr(ns, k))
    if ns.select_recompute:
        cfg.select_recompute = True
    if ns.parser_result:
        lp = parse_layer_records(ns.parser_result).to_layer_profile()
    else:
        lp = profile_from_ratios(ns.backward_ratio, ns.layer_ratio, ns.head_loss, ns.recompute_ratio)
    ranked = pipeline_search_tool(cfg, ns.nd_path, lp=lp, max_vpp=ns.max_vpp, top_k=ns.topn, mbs_choices=ns.mbs)
    for i, e in enumerate(ranked[:10]):
        print(i, e)
    return 0


if __name__ == "__main__":
    sys.exit(main())
