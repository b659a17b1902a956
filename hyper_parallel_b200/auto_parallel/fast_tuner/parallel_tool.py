"""``fast-tuner-parallel``: search (dp, tp, cp, pp, ep, fsdp, vpp, mbs, sp) for a model on a cluster.

Pipeline of hyper_parallel/auto_parallel/fast-tuner/fast_tuner/parallel_tool.py:42-158 of the
reference: read the trainer/model config -> build the N-D space -> rule pruning -> memory pruning
(-> stop here with ``--alg_phase 1``) -> profile a handful of shrunk candidates (or, with
``--dryrun``, use the analytic cost model) -> balance the pipeline of every surviving candidate ->
write the ranked CSV.
"""
from __future__ import annotations

import argparse
import csv
import json
import os
import sys
from typing import List, Optional

from .config import ModelSpec, Strategy, TunerConfig, load_model_spec
from .cost_model import Hardware, estimate_step_time
from .memory_model import (GIB, activation_memory, compute_weight_and_optimizer_memory, filter_oom,
                           write_candidate_csv)
from .pipeline_balance import LayerProfile, balance_pipeline
from .profiling import (launch_profile, parse_layer_records, select_profile_candidates,
                        write_profile_config)
from .pp_simulator import compute_order, render_svg, render_text, simulate
from .space import (Config, build_initial_spaces, dp_of, ep_of, expert_filter_configs, mbs_of, op_of, pp_of,
                    sp_of, tp_of, vp_of)


def taylor_search_tool(cfg: TunerConfig, spec: Optional[ModelSpec] = None, hw: Optional[Hardware] = None,
                       top_k: int = 20) -> List[dict]:
    spec = spec or load_model_spec(cfg)
    hw = hw or Hardware(gpus_per_node=cfg.gpus_per_node)
    os.makedirs(cfg.output_path, exist_ok=True)
    space = build_initial_spaces(spec, cfg.strategy)
    n0 = len(space)
    space = expert_filter_configs(space, spec, cfg.gbs)
    space = [c for c in space if ep_of(c) <= cfg.max_expert_parallel]
    n1 = len(space)
    space, rows = filter_oom(space, spec, cfg.max_mem_gib, recompute=cfg.select_recompute)
    write_candidate_csv(rows, cfg.output_path)
    summary = {"initial": n0, "after_expert_rules": n1, "after_memory": len(space)}
    with open(os.path.join(cfg.output_path, "search_summary.json"), "w") as f:
        json.dump(summary, f)
    if cfg.alg_phase == 1 or not space:
        return [{"summary": summary}]
    # profile (or estimate) ------------------------------------------------------------
    # Without --dryrun the candidates are PROFILED: the search launches a trainer (an external one given
    # by trainer_path, else this package's own profile_trainer) on the ranks at hand and reads the
    # per-layer device times it records; the first candidate that runs supplies the layer profile.
    profile = None
    if not cfg.dryrun:
        for i, cand in enumerate(select_profile_candidates(space, cfg.rank_num)):
            path = write_profile_config(cand, spec, os.path.join(cfg.output_path, "profile"), i)
            rc = launch_profile(path, cfg.trainer_path, min(cfg.rank_num, cand[0][0][0] * cand[0][0][1]),
                                timeout=cfg.profile_timeout, port=cfg.profile_port + i)
            rec = path.replace(".json", ".records.jsonl")
            if rc == 0 and os.path.exists(rec):
                profile = parse_layer_records(rec)
                summary["profiled"] = os.path.basename(path)
                break
        with open(os.path.join(cfg.output_path, "search_summary.json"), "w") as f:
            json.dump(summary, f)
    return rank_candidates(space, spec, cfg, hw, profile.to_layer_profile() if profile is not None else None, top_k)


def rank_candidates(space: List[Config], spec: ModelSpec, cfg: TunerConfig, hw: Optional[Hardware] = None,
                    lp: Optional[LayerProfile] = None, top_k: int = 20) -> List[dict]:
    """Second half of the search, also the body of the stand-alone pipeline tool: score every
    candidate with the cost model, balance the pipeline of the pipelined ones with the layer profile
    ``lp`` (measured, or the analytic stand-in: a backward costs two forwards, a MoE layer as much as
    a dense one), re-check the best ``top_k`` in the schedule simulator and write
    ``pipeline_output/ranked_configs.csv``."""
    hw = hw or Hardware(gpus_per_node=cfg.gpus_per_node)
    lp = lp or LayerProfile(dense_fw=1.0, dense_bw=2.0, moe_fw=1.0, moe_bw=2.0)
    ranked = []
    scored = sorted(space, key=lambda c: estimate_step_time(spec, c, hw))[: max(top_k * 5, 50)]
    memo = {}                                   # many candidates share (stages, chunks, micro-batches)

    def balanced(pp, vp, micro, max_offset=None):
        key = (pp, vp, micro, max_offset)
        if key not in memo:
            kw = {} if max_offset is None else {"max_offset": max_offset}
            memo[key] = balance_pipeline(spec.num_layers, spec.dense_layers, pp, vp, micro, lp, **kw)
        return memo[key]

    for c in scored:
        t = estimate_step_time(spec, c, hw)
        pp, vp = pp_of(c), vp_of(c)
        entry = {"dp": dp_of(c), "tp": tp_of(c), "pp": pp, "ep": ep_of(c), "op": op_of(c), "vp": vp,
                 "mbs": mbs_of(c), "sp": sp_of(c), "step_time_us": t * 1e6}
        if pp > 1:
            micro = max(cfg.gbs // (dp_of(c) * mbs_of(c)), 1)
            bal = balanced(pp, vp, min(micro, 4 * pp))
            entry.update({"layers": bal.layers, "offset": bal.offset, "recompute": bal.recompute,
                          "select_recompute": bal.select_recompute, "bubble": round(bal.bubble_ratio, 4)})
            even = balanced(pp, vp, min(micro, 4 * pp), 0)
            entry["step_time_us"] = t * 1e6 * bal.makespan / max(even.makespan, 1e-9)
        ranked.append(entry)
    ranked.sort(key=lambda e: e["step_time_us"])
    ranked = ranked[:top_k]
    # Re-check of the survivors (the reference's dry-run double check, pipeline_parallel.py:34-64): the
    # balanced layer split of every pipelined candidate is replayed in the schedule simulator with p2p
    # blocks and per-stage memory; a candidate whose simulated peak exceeds the budget is flagged.
    by_key = {(dp_of(c), tp_of(c), pp_of(c), ep_of(c), op_of(c), vp_of(c), mbs_of(c), sp_of(c)): c for c in scored}
    for e in ranked:
        c = by_key.get((e["dp"], e["tp"], e["pp"], e["ep"], e["op"], e["vp"], e["mbs"], e["sp"]))
        if c is None or e["pp"] <= 1 or "layers" not in e:
            e["check"] = "n/a"
            continue
        e.update(_recheck(spec, c, e, lp, cfg, os.path.join(cfg.output_path, "pipeline_output")))
    out_csv = os.path.join(cfg.output_path, "pipeline_output")
    os.makedirs(out_csv, exist_ok=True)
    with open(os.path.join(out_csv, "ranked_configs.csv"), "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["rank", "dp", "tp", "pp", "ep", "op", "vp", "mbs", "sp", "step_time(us)", "layers", "offset",
                    "recompute", "select_recompute", "bubble", "sim_bubble", "sim_peak_gib", "check"])
        for i, e in enumerate(ranked):
            w.writerow([i, e["dp"], e["tp"], e["pp"], e["ep"], e["op"], e["vp"], e["mbs"], e["sp"],
                        round(e["step_time_us"]), e.get("layers", ""), e.get("offset", ""), e.get("recompute", ""),
                        e.get("select_recompute", ""), e.get("bubble", ""), e.get("sim_bubble", ""), e.get("sim_peak_gib", ""), e.get("check", "")])
    return ranked


def _recheck(spec: ModelSpec, c: Config, e: dict, lp: LayerProfile, cfg: TunerConfig, out_dir: str) -> dict:
    """Replay one ranked candidate in the schedule simulator: virtual-stage times from its balanced layer
    split, one p2p block per stage boundary, static + activation bytes per stage."""
    pp, vp = e["pp"], max(e["vp"], 1)
    layers = e["layers"]                                   # [chunk][stage]
    micro = max(cfg.gbs // (e["dp"] * e["mbs"]), 1)
    micro = min(micro, 4 * pp)
    n_virtual = pp * vp
    fwd, bwd = [], []
    dense_left = spec.dense_layers
    for v in range(n_virtual):
        n = layers[v // pp][v % pp]
        nd = min(dense_left, n)
        dense_left -= nd
        f = nd * lp.dense_fw + (n - nd) * lp.moe_fw
        b = nd * lp.dense_bw + (n - nd) * lp.moe_bw
        if v == 0:
            f, b = f + lp.embed_fw, b + lp.embed_bw
        if v == n_virtual - 1:
            f, b = f + lp.head_fw, b + lp.head_bw
        fwd.append(f)
        bwd.append(b)
    per_layer_act = activation_memory(spec, c, cfg.select_recompute) / max(-(-spec.num_layers // pp) * pp, 1)
    act = [layers[v // pp][v % pp] * per_layer_act for v in range(n_virtual)]
    static = [compute_weight_and_optimizer_memory(spec, c)] * pp
    unit = (lp.dense_fw + lp.dense_bw) / 3.0 or 1.0
    kind = "vpp" if vp > 1 else "1f1b"
    res = simulate(compute_order(kind, micro, pp, vp), fwd, bwd, pp, p2p=0.02 * unit, act_bytes=act,
                   static_bytes=static)
    peak = max(res.peak_bytes) / GIB
    os.makedirs(out_dir, exist_ok=True)
    name = f"sim_dp{e['dp']}_tp{e['tp']}_pp{pp}_vp{vp}_mbs{e['mbs']}.txt"
    with open(os.path.join(out_dir, name), "w") as f:
        f.write(render_text(res) + "\n")
    render_svg(res, os.path.join(out_dir, name[:-4] + ".svg"))
    return {"sim_bubble": round(res.bubble_ratio, 4), "sim_peak_gib": round(peak, 1),
            "check": "ok" if peak <= cfg.max_mem_gib else "over budget"}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="fast-tuner-parallel", description=__doc__)
    ap.add_argument("--config", help="json file with the keys below")
    ap.add_argument("--toml_path"); ap.add_argument("--yaml_path"); ap.add_argument("--shell_path")
    ap.add_argument("--model_json")
    ap.add_argument("--torchtitan_path", "--mindformers_dir", "--mindspeed_path", dest="trainer_path")
    ap.add_argument("--rank_num", type=int); ap.add_argument("--gbs", type=int)
    ap.add_argument("--nnodes", type=int); ap.add_argument("--npus_per_node", "--gpus_per_node", dest="gpus_per_node", type=int)
    ap.add_argument("--output_path")
    ap.add_argument("--strategy", nargs="*", choices=["DP", "TP", "PP", "EP", "CP", "FSDP"])
    ap.add_argument("--alg_phase", type=int, choices=[0, 1, 2])
    ap.add_argument("--max_expert_parallel", type=int)
    ap.add_argument("--select_recompute", action="store_true")
    ap.add_argument("--solver_name", default=None)
    ap.add_argument("--dryrun", action="store_true"); ap.add_argument("--check", action="store_true")
    ns = ap.parse_args(argv)
    cfg = TunerConfig.from_json(ns.config) if ns.config else TunerConfig()
    for k, v in vars(ns).items():
        if k in ("config", "strategy") or v in (None, False):
            continue
        setattr(cfg, k, v)
    if ns.strategy is not None:
        cfg.strategy = Strategy(**{k: (k in ns.strategy) for k in ("DP", "TP", "PP", "EP", "CP", "FSDP")})
    result = taylor_search_tool(cfg)
    for i, e in enumerate(result[:10]):
        print(i, e)
    return 0


if __name__ == "__main__":
    sys.exit(main())
