"""Analytic step-time model for a B200 node (used for ranking when profiling is skipped, and to
order the candidates that are worth profiling).

Compute time = FLOPs / (sustained bf16 GEMM throughput x an efficiency that drops with small TP
shards); communication = bytes / NVLink bandwidth with all-gather / reduce-scatter volumes of the
TP (per layer, activations) and FSDP (per step, parameters) groups; pipeline bubble from the
1F1B / VPP formula.  The constants default to the numbers measured on this pool.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass

from .config import ModelSpec
from .memory_model import dense_layer_params, embedding_params, moe_layer_params
from .space import Config, cp_of, dp_of, ep_of, mbs_of, op_of, pp_of, sp_of, tp_of, vp_of


@dataclass
class Hardware:
    bf16_tflops: float = 1418.6          # sustained cuBLAS bf16 on B200 (measured)
    hbm_gbs: float = 6547.5
    nvlink_gbs: float = 770.0            # measured peer copy per direction
    allreduce_busbw_gbs: float = 725.0   # measured 8-rank all-reduce bus bandwidth
    internode_gbs: float = 50.0          # per GPU across nodes (400 Gb/s NIC)
    gpus_per_node: int = 8
    launch_us: float = 5.0

    @staticmethod
    def from_measured(path: str) -> "Hardware":
        hw = Hardware()
        try:
            with open(path) as f:
                m = json.load(f)
            hw.bf16_tflops = float(m.get("bf16_tflops_sustained", hw.bf16_tflops))
            hw.hbm_gbs = float(m.get("hbm_gbs", hw.hbm_gbs))
        except (OSError, ValueError):
            pass
        return hw


def estimate_step_time(m: ModelSpec, c: Config, hw: Hardware = Hardware()) -> float:
    """Estimated seconds per optimizer step for candidate ``c``."""
    dp, tp, cp, pp = dp_of(c), tp_of(c), cp_of(c), pp_of(c)
    ep, op, vp, mbs, sp = ep_of(c), op_of(c), vp_of(c), mbs_of(c), sp_of(c)
    gbs = m.global_batch_size
    micro = max(gbs // (dp * mbs), 1)
    tokens_mb = mbs * m.seq_length / cp
    shared, routed = moe_layer_params(m)
    active_moe = shared + routed * (m.num_experts_per_tok / max(m.expert_num or 1, 1))
    layer_flops_dense = 6 * dense_layer_params(m) * tokens_mb
    layer_flops_moe = 6 * active_moe * tokens_mb
    attn = 12 * m.num_attention_heads * m.head_dim * m.seq_length / 2 * tokens_mb
    eff = 0.72 * min(1.0, (m.hidden_size / tp) / 1024) ** 0.25
    per_layer = lambda fl: (fl + attn) / tp / (hw.bf16_tflops * 1e12 * eff)  # noqa: E731
    n_dense, n_moe = m.dense_layers, m.moe_layers
    layers_per_stage = (n_dense + n_moe) / pp
    t_layer = (n_dense * per_layer(layer_flops_dense) + n_moe * per_layer(layer_flops_moe)) / max(n_dense + n_moe, 1)
    # TP collectives: 4 per layer (2 fwd + 2 bwd) x 2 directions of activation volume
    tp_bw = hw.nvlink_gbs if tp <= hw.gpus_per_node else hw.internode_gbs
    act_bytes = 2 * tokens_mb * m.hidden_size
    t_tp = 0.0 if tp == 1 else 8 * act_bytes * (tp - 1) / tp / (tp_bw * 1e9) * (0.6 if sp else 1.0)
    # EP all-to-all: dispatch + combine, fwd + bwd
    t_ep = 0.0
    if ep > 1 and n_moe:
        a2a = 2 * tokens_mb * m.num_experts_per_tok * m.hidden_size * (ep - 1) / ep
        ep_bw = hw.nvlink_gbs if ep * tp <= hw.gpus_per_node else hw.internode_gbs
        t_ep = 4 * a2a / (ep_bw * 1e9) * (n_moe / max(n_dense + n_moe, 1))
    t_stage_mb = layers_per_stage * (t_layer + t_tp + t_ep)
    head = 6 * embedding_params(m) * tokens_mb / tp / (hw.bf16_tflops * 1e12 * eff)
    # pipeline: micro + bubble
    bubble = (pp - 1) / vp
    t_pipe = (micro + bubble) * t_stage_mb + micro * head / max(pp, 1)
    # FSDP / DP parameter traffic per step (all-gather x2 + reduce-scatter), overlappable to ~70 %
    shard = dp if op == -1 else max(op, 1)
    stage_params = layers_per_stage * (n_dense * dense_layer_params(m) + n_moe * (shared + routed / max(ep, 1))) \
        / max(n_dense + n_moe, 1) / tp
    dp_bw = hw.nvlink_gbs if dp * tp * pp <= hw.gpus_per_node else hw.internode_gbs
    t_dp = 0.0 if dp == 1 else 3 * 2 * stage_params * (shard - 1) / max(shard, 1) / (dp_bw * 1e9) * 0.3
    return t_pipe + t_dp
