"""Inputs of the strategy search: the model description and the tuning job.

Ingests the same sources as hyper_parallel/auto_parallel/fast-tuner/fast_tuner/ndsearch/
para_for_nd_search.py:10-317 of the reference: a TorchTitan TOML (+ model args), a MindFormers
YAML, a Megatron / MindSpeed launch script (regex over ``--flag value``), or a plain JSON / dict.
"""
from __future__ import annotations

import json
import os
import re
from dataclasses import dataclass, field
from typing import Any, Dict, Optional

import yaml


@dataclass
class ModelSpec:
    num_layers: int = 32
    hidden_size: int = 4096
    ffn_hidden_size: int = 14336
    num_attention_heads: int = 32
    num_kv_heads: Optional[int] = None
    vocab_size: int = 128256
    seq_length: int = 4096
    # MoE
    expert_num: Optional[int] = None
    moe_ffn_hidden_size: Optional[int] = None
    num_experts_per_tok: int = 1
    shared_expert_num: int = 0
    first_k_dense: int = 0
    # MLA
    kv_lora_rank: Optional[int] = None
    q_lora_rank: Optional[int] = None
    qk_nope_head_dim: int = 128
    qk_rope_head_dim: int = 64
    v_head_dim: int = 128
    # job
    world_size: int = 8
    global_batch_size: int = 16
    bytes_per_param: int = 2

    @property
    def kv_heads(self) -> int:
        return self.num_kv_heads or self.num_attention_heads

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @property
    def moe_layers(self) -> int:
        return 0 if not self.expert_num else self.num_layers - self.first_k_dense

    @property
    def dense_layers(self) -> int:
        return self.num_layers - self.moe_layers


@dataclass
class Strategy:
    DP: bool = True
    TP: bool = True
    PP: bool = True
    EP: bool = False
    CP: bool = False
    FSDP: bool = True


@dataclass
class TunerConfig:
    rank_num: int = 8                    # ranks available for profiling
    gbs: int = 16
    gpus_per_node: int = 8
    nnodes: int = 1
    output_path: str = "./output/"
    strategy: Strategy = field(default_factory=Strategy)
    alg_phase: int = 0                   # 0 = all, 1 = stop after pruning, 2 = pipeline balance only
    max_expert_parallel: int = 64
    select_recompute: bool = False
    solver_name: str = "native"
    dryrun: bool = False
    check: bool = False
    max_mem_gib: float = 162.0           # 90 % of a B200's 180 GB
    toml_path: Optional[str] = None
    yaml_path: Optional[str] = None
    shell_path: Optional[str] = None
    model_json: Optional[str] = None
    trainer_path: Optional[str] = None   # torchtitan_path / mindformers_dir / mindspeed_path; None = built-in trainer
    profile_timeout: int = 1800          # seconds per profiled candidate
    profile_port: int = 29591            # rendezvous port of the first profile run

    @staticmethod
    def from_json(path: str) -> "TunerConfig":
        with open(path, "r", encoding="utf-8") as f:
            raw = json.load(f)
        cfg = TunerConfig.from_dict(raw)
        # a model file named relative to the setup file (not to the working directory) is found too
        base = os.path.dirname(os.path.abspath(path))
        for k in ("model_json", "toml_path", "yaml_path", "shell_path"):
            v = getattr(cfg, k)
            if v and not os.path.isabs(v) and not os.path.exists(v) and os.path.exists(os.path.join(base, v)):
                setattr(cfg, k, os.path.join(base, v))
        return cfg

    @staticmethod
    def from_dict(raw: Dict[str, Any]) -> "TunerConfig":
        cfg = TunerConfig()
        alias = {"npus_per_node": "gpus_per_node", "torchtitan_path": "trainer_path",
                 "mindformers_dir": "trainer_path", "mindspeed_path": "trainer_path"}
        for k, v in raw.items():
            k = alias.get(k, k)
            if k == "strategy":
                cfg.strategy = Strategy(**{kk: bool(vv) for kk, vv in v.items() if hasattr(Strategy, kk)})
            elif hasattr(cfg, k):
                setattr(cfg, k, v)
        return cfg


# ------------------------------------------------------------------ ingestion --
def _apply(spec: ModelSpec, mapping: Dict[str, Any], table: Dict[str, str]) -> None:
    for src, dst in table.items():
        if src in mapping and mapping[src] is not None:
            cur = getattr(spec, dst)
            val = mapping[src]
            setattr(spec, dst, type(cur)(val) if isinstance(cur, (int, float)) and cur is not None else val)


_TITAN = {"n_layers": "num_layers", "dim": "hidden_size", "n_heads": "num_attention_heads",
          "n_kv_heads": "num_kv_heads", "vocab_size": "vocab_size", "ffn_dim": "ffn_hidden_size",
          "num_experts": "expert_num", "moe_inter_dim": "moe_ffn_hidden_size", "top_k": "num_experts_per_tok",
          "n_dense_layers": "first_k_dense", "kv_lora_rank": "kv_lora_rank", "q_lora_rank": "q_lora_rank"}

_MINDFORMERS = {"num_layers": "num_layers", "hidden_size": "hidden_size", "num_heads": "num_attention_heads",
                "n_kv_heads": "num_kv_heads", "vocab_size": "vocab_size", "intermediate_size": "ffn_hidden_size",
                "seq_length": "seq_length", "expert_num": "expert_num", "moe_intermediate_size": "moe_ffn_hidden_size",
                "num_experts_chosen": "num_experts_per_tok", "shared_expert_num": "shared_expert_num",
                "first_k_dense_replace": "first_k_dense", "kv_lora_rank": "kv_lora_rank", "q_lora_rank": "q_lora_rank",
                "qk_nope_head_dim": "qk_nope_head_dim", "qk_rope_head_dim": "qk_rope_head_dim", "v_head_dim": "v_head_dim"}

_MEGATRON = {"num-layers": "num_layers", "hidden-size": "hidden_size", "ffn-hidden-size": "ffn_hidden_size",
             "num-attention-heads": "num_attention_heads", "num-query-groups": "num_kv_heads",
             "padded-vocab-size": "vocab_size", "vocab-size": "vocab_size", "seq-length": "seq_length",
             "num-experts": "expert_num", "moe-ffn-hidden-size": "moe_ffn_hidden_size",
             "moe-router-topk": "num_experts_per_tok", "n-shared-experts": "shared_expert_num",
             "first-k-dense-replace": "first_k_dense", "kv-lora-rank": "kv_lora_rank", "q-lora-rank": "q_lora_rank",
             "global-batch-size": "global_batch_size"}


def model_from_toml(path: str, model_args: Optional[Dict[str, Any]] = None) -> ModelSpec:
    import tomllib
    with open(path, "rb") as f:
        raw = tomllib.load(f)
    spec = ModelSpec()
    flat: Dict[str, Any] = {}
    for section in ("model", "training", "parallelism"):
        flat.update(raw.get(section, {}))
    flat.update(model_args or {})
    _apply(spec, flat, _TITAN)
    if "seq_len" in flat:
        spec.seq_length = int(flat["seq_len"])
    if "global_batch_size" in flat and int(flat["global_batch_size"]) > 0:
        spec.global_batch_size = int(flat["global_batch_size"])
    return spec


def model_from_yaml(path: str) -> ModelSpec:
    with open(path, "r", encoding="utf-8") as f:
        raw = yaml.safe_load(f)
    spec = ModelSpec()
    mc = (raw.get("model") or {}).get("model_config") or raw.get("model_config") or {}
    _apply(spec, mc, _MINDFORMERS)
    moe = raw.get("moe_config") or {}
    _apply(spec, moe, _MINDFORMERS)
    par = raw.get("parallel_config") or {}
    rc = raw.get("runner_config") or {}
    if all(k in par for k in ("data_parallel", "model_parallel", "pipeline_stage")):
        spec.world_size = int(par["data_parallel"]) * int(par["model_parallel"]) * int(par["pipeline_stage"])
        if "batch_size" in rc:
            spec.global_batch_size = int(rc["batch_size"]) * int(par["data_parallel"]) * int(par.get("micro_batch_num", 1))
    return spec


_FLAG = re.compile(r"--([a-zA-Z0-9\-]+)[ =]+\$?\{?([A-Za-z0-9_\.\-/]+)\}?")
_VAR = re.compile(r"^\s*([A-Z_][A-Z0-9_]*)=([^\s#]+)", re.M)


def model_from_shell(path: str) -> ModelSpec:
    with open(path, "r", encoding="utf-8") as f:
        text = f.read()
    variables = {k: v.strip("\"'") for k, v in _VAR.findall(text)}
    flags: Dict[str, Any] = {}
    for name, val in _FLAG.findall(text.replace("\\\n", " ")):
        val = variables.get(val, val)
        try:
            flags[name] = int(val)
        except ValueError:
            try:
                flags[name] = float(val)
            except ValueError:
                flags[name] = val
    spec = ModelSpec()
    _apply(spec, flags, _MEGATRON)
    return spec


def model_from_json(path_or_dict) -> ModelSpec:
    raw = path_or_dict
    if isinstance(raw, str):
        with open(raw, "r", encoding="utf-8") as f:
            raw = json.load(f)
    spec = ModelSpec()
    for k, v in raw.items():
        if hasattr(spec, k):
            setattr(spec, k, v)
    return spec


def load_model_spec(cfg: TunerConfig) -> ModelSpec:
    if cfg.model_json:
        spec = model_from_json(cfg.model_json)
    elif cfg.toml_path:
        spec = model_from_toml(cfg.toml_path)
    elif cfg.yaml_path:
        spec = model_from_yaml(cfg.yaml_path)
    elif cfg.shell_path:
        spec = model_from_shell(cfg.shell_path)
    else:
        raise ValueError("one of model_json / toml_path / yaml_path / shell_path is required")
    spec.world_size = cfg.gpus_per_node * cfg.nnodes if cfg.nnodes * cfg.gpus_per_node > 0 else spec.world_size
    if cfg.gbs:
        spec.global_batch_size = cfg.gbs
    return spec
