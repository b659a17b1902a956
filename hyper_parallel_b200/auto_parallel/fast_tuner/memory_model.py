"""Analytic per-device memory model and OOM pruning.

Follows the structure of hyper_parallel/auto_parallel/fast-tuner/fast_tuner/ndsearch/
memory_model.py:107-173 (``filter_oom``) and :292-417 (weights + optimizer bytes): 18 bytes per
parameter for bf16 weights + fp32 gradients-in-optimizer + fp32 master/moments without a
distributed optimizer, ``6 + 12 / op`` with one; MoE expert parameters are divided by ``ep``;
MLA projections are counted when the model has ``kv_lora_rank``.  The device budget defaults to
90 % of a B200's 180 GB instead of the reference's 58 GiB (Ascend 910B).  Activations are
estimated per micro-batch and multiplied by the number of micro-batches in flight under 1F1B.
"""
from __future__ import annotations

import csv
import os
from typing import List

from .config import ModelSpec
from .space import Config, cp_of, dp_of, ep_of, mbs_of, op_of, pp_of, sp_of, tp_of, vp_of

GIB = 1024 ** 3


def attention_params(m: ModelSpec) -> int:
    h = m.hidden_size
    if m.kv_lora_rank:   # MLA
        qk = m.qk_nope_head_dim + m.qk_rope_head_dim
        q = (h * m.q_lora_rank + m.q_lora_rank * m.num_attention_heads * qk) if m.q_lora_rank \
            else h * m.num_attention_heads * qk
        kv = h * (m.kv_lora_rank + m.qk_rope_head_dim) + \
            m.kv_lora_rank * m.num_attention_heads * (m.qk_nope_head_dim + m.v_head_dim)
        o = m.num_attention_heads * m.v_head_dim * h
        return q + kv + o
    hd = m.head_dim
    return h * (m.num_attention_heads + 2 * m.kv_heads) * hd + m.num_attention_heads * hd * h


def dense_layer_params(m: ModelSpec) -> int:
    return attention_params(m) + 3 * m.hidden_size * m.ffn_hidden_size + 2 * m.hidden_size


def moe_layer_params(m: ModelSpec):
    """(non-expert params, routed-expert params) of one MoE layer."""
    f = m.moe_ffn_hidden_size or m.ffn_hidden_size
    shared = attention_params(m) + 2 * m.hidden_size + m.hidden_size * (m.expert_num or 0) \
        + m.shared_expert_num * 3 * m.hidden_size * f
    routed = (m.expert_num or 0) * 3 * m.hidden_size * f
    return shared, routed


def embedding_params(m: ModelSpec) -> int:
    return m.vocab_size * m.hidden_size


def compute_weight_and_optimizer_memory(m: ModelSpec, c: Config) -> float:
    """Bytes of weights + gradients + optimizer state on the most loaded pipeline stage."""
    dp, tp, pp, ep, op = dp_of(c), tp_of(c), pp_of(c), ep_of(c), op_of(c)
    shard = dp if op == -1 else max(op, 1)
    bytes_per = 18.0 if shard == 1 else 6.0 + 12.0 / shard
    layers_per_stage = -(-m.num_layers // pp)
    moe_frac = m.moe_layers / m.num_layers if m.num_layers else 0.0
    n_moe = layers_per_stage * moe_frac
    n_dense = layers_per_stage - n_moe
    shared, routed = moe_layer_params(m)
    params = n_dense * dense_layer_params(m) / tp + n_moe * (shared / tp + routed / max(ep, 1) / 1)
    first_stage_extra = embedding_params(m) / tp
    last_stage_extra = embedding_params(m) / tp if pp > 1 else 0
    params += max(first_stage_extra + (last_stage_extra if pp == 1 else 0), last_stage_extra)
    if pp == 1:
        params += embedding_params(m) / tp
    return params * bytes_per


def activation_memory(m: ModelSpec, c: Config, recompute: bool = False) -> float:
    tp, cp, pp, mbs, sp, vp = tp_of(c), cp_of(c), pp_of(c), mbs_of(c), sp_of(c), vp_of(c)
    s, h = m.seq_length / cp, m.hidden_size
    tokens = s * mbs
    sp_div = tp if sp else 1
    f = m.ffn_hidden_size
    # bf16 activations kept per layer: norms / residuals (sequence-parallel part) + qkv/attn + MLP (tp part)
    per_layer = 2 * tokens * (6 * h / sp_div + (3 * h + 3 * f) / tp)
    if recompute:
        per_layer = 2 * tokens * h / sp_div
    layers_per_stage = -(-m.num_layers // pp)
    in_flight = pp if pp > 1 else 1
    if vp > 1:
        in_flight = pp * (1 + (pp - 1) / (pp * vp))
    logits = 2 * tokens * m.vocab_size / tp * 2
    return per_layer * layers_per_stage * in_flight + logits


def estimate_peak_memory(m: ModelSpec, c: Config, recompute: bool = False) -> float:
    return compute_weight_and_optimizer_memory(m, c) + activation_memory(m, c, recompute)


def filter_oom(space: List[Config], m: ModelSpec, max_mem_gib: float = 162.0, recompute: bool = False):
    """Keep candidates whose estimated peak fits; returns ``[dp, tp, pp, ep, cp, op, mem_mib]`` rows too."""
    kept, rows = [], []
    for c in space:
        mem = estimate_peak_memory(m, c, recompute)
        if mem <= max_mem_gib * GIB:
            kept.append(c)
            rows.append([dp_of(c), tp_of(c), pp_of(c), ep_of(c), cp_of(c), op_of(c), round(mem / 2 ** 20)])
    return kept, rows


def grey_box_memory_prune(m: ModelSpec, dryrun_info: List[list], test_ep: List[int], max_expert_parallel: int,
                          max_mem_mib: float = 162.0 * 1024):
    """Fit ``mem(ep) = static + expert / ep`` from dry-runs of the same (dp, tp, pp) at two ``ep``
    values (rows ``[dp, tp, pp, ep, peak_mem]``) and extrapolate to every even ``ep`` up to the limit
    (reference: grey_box_memory_prune, memory_model.py:58-97)."""
    by_key = {}
    for dp, tp, pp, ep, mem in dryrun_info:
        by_key.setdefault((dp, tp, pp), {})[ep] = mem
    out = []
    e0, e1 = test_ep[0], test_ep[1]
    for (dp, tp, pp), d in by_key.items():
        if e0 not in d or e1 not in d:
            continue
        expert = (d[e0] - d[e1]) / (1.0 / e0 - 1.0 / e1)
        static = d[e0] - expert / e0
        ep = 1
        while ep <= max_expert_parallel:
            if (m.expert_num or ep) % ep == 0 and (dp * tp) % ep == 0:
                mem = static + expert / ep
                if mem <= max_mem_mib:
                    out.append([dp, tp, pp, ep, round(mem)])
            ep = 2 if ep == 1 else ep + 2
    return out


def write_candidate_csv(rows: List[list], out_dir: str, name: str = "nd_candidate_config.csv") -> str:
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, name)
    with open(path, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["dp", "tp", "pp", "ep", "cp", "op", "evaluate_mem_MiB"])
        w.writerows(rows)
    return path
