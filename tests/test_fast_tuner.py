"""Fast-Tuner: space sizes, rule pruning, memory model, simulator, balancer, CLI dry-run."""
import csv
import json
import os

import pytest

from hyper_parallel_b200.auto_parallel.fast_tuner import ModelSpec, Strategy, TunerConfig, taylor_search_tool
from hyper_parallel_b200.auto_parallel.fast_tuner import config as ftc
from hyper_parallel_b200.auto_parallel.fast_tuner.memory_model import (dense_layer_params, estimate_peak_memory,
                                                                       filter_oom, grey_box_memory_prune)
from hyper_parallel_b200.auto_parallel.fast_tuner.pipeline_balance import LayerProfile, balance_pipeline
from hyper_parallel_b200.auto_parallel.fast_tuner.pp_simulator import compute_order, simulate
from hyper_parallel_b200.auto_parallel.fast_tuner.space import (build_initial_spaces, expert_filter_configs,
                                                                factorizations4, pp_of, tp_of)

LLAMA8B = ModelSpec(num_layers=32, hidden_size=4096, ffn_hidden_size=14336, num_attention_heads=32, num_kv_heads=8,
                    vocab_size=128256, seq_length=4096, world_size=8, global_batch_size=16)


def test_space_sizes_and_rules():
    assert len(factorizations4(8)) == 20            # ordered 4-factorisations of 2^3: C(6,3)
    space = build_initial_spaces(LLAMA8B)
    assert len(space) == len({json.dumps(c) for c in space})
    assert all(c[0][0][0] * c[0][0][1] * c[0][0][2] * c[0][0][3] == 8 for c in space)
    assert any(c[1] for c in space) and all(tp_of(c) > 1 for c in space if c[1])      # sp only with tp > 1
    pruned = expert_filter_configs(space, LLAMA8B, 16)
    assert 0 < len(pruned) < len(space)
    assert all(c[0][0][2] == 1 for c in pruned)                                         # cp == 1 rule
    assert all(pp_of(c) <= 16 // c[0][0][0] // c[0][1][3] for c in pruned)              # pp <= gbs/dp/mbs
    no_pp = build_initial_spaces(LLAMA8B, Strategy(PP=False, CP=False, EP=False))
    assert all(pp_of(c) == 1 for c in no_pp)
    assert all(c[0][1][2] == 1 for c in space if pp_of(c) == 1)                         # no pipeline: depth 1 only
    # the size of the space follows from the rules: per (dp, tp, cp, pp): divisors(dp) FSDP degrees x
    # depths below ceil(L / pp) (1 without a pipeline) x 3 micro-batch sizes x (1 + E / 2) expert
    # degrees, doubled by the sequence-parallel switch where tp > 1
    moe = ModelSpec(num_layers=12, expert_num=8, world_size=16)
    want = 0
    for dp, tp, cp, pp in factorizations4(16):
        depths = 1 if pp == 1 else max(-(-12 // pp) - 1, 0)
        want += sum(1 for d in range(1, dp + 1) if dp % d == 0) * depths * 3 * (1 + 8 // 2) * (2 if tp > 1 else 1)
    assert len(build_initial_spaces(moe)) == want


def test_memory_model_orders_and_prunes():
    assert abs(dense_layer_params(LLAMA8B) * 32 / 1e9 - 6.98) < 0.1
    base = [[(8, 1, 1, 1), (1, 1, 1, 1)], False]          # pure DP: 18 B/param -> ~145 GB > 80
    fsdp = [[(8, 1, 1, 1), (1, 8, 1, 1)], False]
    assert estimate_peak_memory(LLAMA8B, base) > estimate_peak_memory(LLAMA8B, fsdp)
    kept, rows = filter_oom([base, fsdp], LLAMA8B, max_mem_gib=80.0)
    assert kept == [fsdp] and len(rows) == 1 and len(rows[0]) == 7
    moe = ModelSpec(expert_num=64, world_size=64)
    out = grey_box_memory_prune(moe, [[8, 1, 8, 4, 90000], [8, 1, 8, 8, 60000]], [4, 8], 16, max_mem_mib=70000)
    assert out and all(r[3] <= 16 and r[4] <= 70000 for r in out)


def test_simulator_matches_closed_forms():
    S, M = 4, 8
    res = simulate(compute_order("1f1b", M, S), [1.0] * S, [2.0] * S, S)
    assert abs(res.makespan - (M + S - 1) * 3.0) < 1e-9            # classic 1F1B makespan
    assert res.peak_live[0] == S and res.peak_live[-1] == 1         # in-flight activations
    g = simulate(compute_order("gpipe", M, S), [1.0] * S, [2.0] * S, S)
    assert abs(g.makespan - res.makespan) < 1e-9 and g.peak_live[0] == M
    v = simulate(compute_order("vpp", M, S, 2), [0.5] * (2 * S), [1.0] * (2 * S), S)
    assert v.makespan < res.makespan                                 # interleaving shrinks the bubble
    assert 0 < v.bubble_ratio < res.bubble_ratio


def test_balancer_moves_layers_off_the_loaded_last_stage():
    prof = LayerProfile(dense_fw=1.0, dense_bw=2.0, moe_fw=1.0, moe_bw=2.0, head_fw=2.0, head_bw=4.0)
    even = balance_pipeline(32, 32, 4, 1, 8, prof, max_offset=0)
    bal = balance_pipeline(32, 32, 4, 1, 8, prof, max_offset=2)
    assert sum(sum(r) for r in bal.layers) == 32
    assert bal.makespan < even.makespan and bal.layers[0][-1] < 8
    tight = balance_pipeline(32, 32, 4, 1, 8, LayerProfile(act_mem=10.0, recomp_mem=1.0, layer_mem=1.0),
                             mem_limit_mb=200.0)
    assert any(any(r) for r in tight.recompute) and max(tight.peak_mem) <= 200.0 + 1e-6


def test_config_ingestion(tmp_path):
    toml = tmp_path / "m.toml"
    toml.write_text('[model]\nn_layers = 8\ndim = 256\nn_heads = 16\nvocab_size = 2048\n[training]\nseq_len = 2048\n')
    s = ftc.model_from_toml(str(toml))
    assert (s.num_layers, s.hidden_size, s.seq_length) == (8, 256, 2048)
    sh = tmp_path / "run.sh"
    sh.write_text('NL=12\npython pretrain.py --num-layers ${NL} --hidden-size 1024 \\\n  --num-attention-heads 8 --seq-length 4096\n')
    s = ftc.model_from_shell(str(sh))
    assert (s.num_layers, s.hidden_size, s.num_attention_heads) == (12, 1024, 8)
    ya = tmp_path / "m.yaml"
    ya.write_text("model:\n  model_config:\n    num_layers: 6\n    hidden_size: 512\n    num_heads: 8\n"
                  "parallel_config:\n  data_parallel: 2\n  model_parallel: 2\n  pipeline_stage: 2\n")
    s = ftc.model_from_yaml(str(ya))
    assert s.num_layers == 6 and s.world_size == 8


def test_cli_dryrun_ranks_candidates(tmp_path):
    mj = tmp_path / "model.json"
    mj.write_text(json.dumps({k: getattr(LLAMA8B, k) for k in LLAMA8B.__dataclass_fields__}))
    cfg = TunerConfig(rank_num=8, gbs=16, gpus_per_node=8, nnodes=1, output_path=str(tmp_path / "out"),
                      dryrun=True, model_json=str(mj), strategy=Strategy(EP=False, CP=False))
    ranked = taylor_search_tool(cfg, top_k=5)
    assert 1 <= len(ranked) <= 5 and ranked == sorted(ranked, key=lambda e: e["step_time_us"])
    assert os.path.exists(tmp_path / "out" / "nd_candidate_config.csv")
    assert os.path.exists(tmp_path / "out" / "pipeline_output" / "ranked_configs.csv")
    cfg.alg_phase = 1
    assert "summary" in taylor_search_tool(cfg)[0]


def test_search_profile_balance_csv_end_to_end(tmp_path):
    """The whole loop without --dryrun on two CPU ranks: search -> the built-in trainer profiles a
    shrunk candidate (gloo, tiny model, LayerTimer records) -> the balancer uses those times -> the
    survivors are replayed in the simulator -> ranked CSV with the re-check columns."""
    tiny = ModelSpec(num_layers=8, hidden_size=64, ffn_hidden_size=128, num_attention_heads=4, num_kv_heads=2,
                     vocab_size=256, seq_length=32, world_size=2, global_batch_size=8)
    mj = tmp_path / "model.json"
    mj.write_text(json.dumps({k: getattr(tiny, k) for k in tiny.__dataclass_fields__}))
    cfg = TunerConfig(rank_num=2, gbs=8, gpus_per_node=2, nnodes=1, output_path=str(tmp_path / "out"), dryrun=False,
                      model_json=str(mj), strategy=Strategy(EP=False, CP=False, TP=False), profile_timeout=300,
                      profile_port=29711)
    ranked = taylor_search_tool(cfg, top_k=60)
    out = tmp_path / "out"
    summary = json.loads((out / "search_summary.json").read_text())
    assert summary.get("profiled", "").startswith("profile_")
    recs = [json.loads(l) for l in (out / "profile" / "profile_000.records.jsonl").read_text().splitlines()]
    assert {r["module"] for r in recs} >= {"dense", "head", "embed"} and all(r["ms"] >= 0 for r in recs)
    assert any(r["module"] == "dense" and r["ms"] > 0 for r in recs)
    rows = list(csv.reader(open(out / "pipeline_output" / "ranked_configs.csv")))
    assert rows[0][-3:] == ["sim_bubble", "sim_peak_gib", "check"] and len(rows) == len(ranked) + 1
    piped = [e for e in ranked if e["pp"] > 1]
    assert piped and all(e["check"] == "ok" and 0.0 <= e["sim_bubble"] < 1.0 for e in piped)
    assert any(f.name.startswith("sim_") for f in (out / "pipeline_output").iterdir())


def test_simulator_svg_rendering(tmp_path):
    """The SVG drawing holds one block per compute step and per transfer, and the memory lines."""
    from hyper_parallel_b200.auto_parallel.fast_tuner import pp_simulator as sim
    order = sim.compute_order("vpp", 8, 4, 2)
    res = sim.simulate(order, [1.0] * 8, [2.0] * 8, 4, p2p=0.1, act_bytes=[1e9] * 8, static_bytes=[2e9] * 4)
    path = tmp_path / "schedule.svg"
    text = sim.render_svg(res, str(path))
    assert path.read_text() == text and text.startswith("<svg") and text.rstrip().endswith("</svg>")
    n_compute = sum(len(v) for v in res.timeline.values())
    n_comm = sum(len(v) for v in res.comm.values())
    assert n_compute == 2 * 8 * 8 and n_comm > 0
    assert text.count("<rect") == n_compute + n_comm
    assert text.count("<polyline") == 4 and "bubble" in text
    import xml.dom.minidom
    xml.dom.minidom.parseString(text)                  # well-formed


def test_balanced_layer_ranges_put_fewer_layers_beside_the_head():
    from hyper_parallel_b200.auto_parallel.fast_tuner.pipeline_balance import (
        dense_transformer_profile, layer_ranges)
    prof = dense_transformer_profile(4096, 14336, 32, 8, 128, 128256, 4096)
    assert prof.head_fw > 2 * prof.dense_fw            # Llama-3-8B: the head is worth more than two layers
    for stages, chunks in ((2, 1), (4, 1), (2, 2), (4, 2)):
        even = balance_pipeline(32, 32, stages, chunks, 8, prof, max_offset=0)
        bal = balance_pipeline(32, 32, stages, chunks, 8, prof, max_offset=3)
        assert bal.makespan < even.makespan
        rng = layer_ranges(bal.layers)
        assert len(rng) == stages * chunks and rng[0][0] == 0 and rng[-1][1] == 32
        assert all(a[1] == b[0] for a, b in zip(rng, rng[1:]))           # contiguous, in model order
        sizes = [hi - lo for lo, hi in rng]
        assert sizes[-1] < 32 // (stages * chunks)                       # the head's stage is lighter


def test_compiled_order_matches_full_simulation():
    import random
    from hyper_parallel_b200.auto_parallel.fast_tuner.pp_simulator import CompiledOrder, compute_order, simulate
    rnd = random.Random(0)
    for kind, S, V, M in (("1f1b", 4, 1, 8), ("vpp", 4, 2, 8), ("vpp", 2, 3, 6), ("gpipe", 3, 1, 5), ("vpp", 4, 2, 6)):
        order = compute_order(kind, M, S, V)
        fast = CompiledOrder(order, S * V, S)
        for p2p in (0.0, 0.3, 2.0):
            f = [rnd.uniform(0.5, 2) for _ in range(S * V)]
            b = [rnd.uniform(1, 4) for _ in range(S * V)]
            assert abs(simulate(order, f, b, S, p2p).makespan - fast.makespan(f, b, p2p)) < 1e-9


def test_pipeline_tool_ranks_the_candidates_of_an_earlier_search(tmp_path):
    """Phase 1 leaves the candidate CSV; the stand-alone pipeline tool expands it over interleave depths
    and micro-batch sizes, balances with the given ratios and writes the ranked CSV and drawings."""
    import csv
    from hyper_parallel_b200.auto_parallel.fast_tuner import pipeline_tool
    mj = tmp_path / "model.json"
    mj.write_text(json.dumps({k: getattr(LLAMA8B, k) for k in LLAMA8B.__dataclass_fields__}))
    cfg = TunerConfig(rank_num=8, gbs=16, gpus_per_node=8, nnodes=1, output_path=str(tmp_path / "out"),
                      dryrun=True, model_json=str(mj), strategy=Strategy(EP=False, CP=False), alg_phase=1)
    assert "summary" in taylor_search_tool(cfg)[0]
    nd = tmp_path / "out" / "nd_candidate_config.csv"
    space = pipeline_tool.read_candidates(str(nd), LLAMA8B, 16, max_vpp=2)
    assert space and all(c[0][1][2] == 1 for c in space if c[0][0][3] == 1)        # no pipeline: no interleaving
    assert any(c[0][1][2] == 2 for c in space) and len({repr(c) for c in space}) == len(space)
    rc = pipeline_tool.main(["--nd_path", str(nd), "--model_json", str(mj), "--gbs", "16", "--rank_num", "8",
                             "--output_path", str(tmp_path / "out2"), "--head_loss", "2.2", "--topn", "6"])
    assert rc == 0
    rows = list(csv.DictReader(open(tmp_path / "out2" / "pipeline_output" / "ranked_configs.csv")))
    assert 1 <= len(rows) <= 6
    times = [float(r["step_time(us)"]) for r in rows]
    assert times == sorted(times)
    piped = [r for r in rows if int(r["pp"]) > 1]
    for r in piped:                                                               # the head's stage is lighter
        layers = json.loads(r["layers"])
        assert sum(map(sum, layers)) == LLAMA8B.num_layers and layers[-1][-1] <= layers[0][0]
        assert r["check"] in ("ok", "over budget")
    lp = pipeline_tool.profile_from_ratios(backward_ratio=2.5, layer_ratio=0.33, head_loss=1.5, recompute_ratio=1.0)
    assert (lp.dense_bw, lp.moe_fw, lp.head_bw) == (2.5, 0.33, 3.75) and abs(lp.moe_bw - 0.825) < 1e-9


def test_shipped_examples_parse_and_search(tmp_path):
    """Every example model file is read by its ingester, and the two setup files drive a dry-run search."""
    from hyper_parallel_b200.auto_parallel.fast_tuner import config as tcfg
    ex = os.path.join(os.path.dirname(tcfg.__file__), "examples")
    titan = tcfg.model_from_toml(os.path.join(ex, "moe_16b_titan.toml"))
    assert (titan.num_layers, titan.expert_num, titan.num_experts_per_tok, titan.first_k_dense) == (28, 64, 6, 1)
    assert titan.moe_layers == 27 and titan.seq_length == 4096 and titan.global_batch_size == 64
    mf = tcfg.model_from_yaml(os.path.join(ex, "dense_13b_mindformers.yaml"))
    assert (mf.num_layers, mf.hidden_size, mf.ffn_hidden_size, mf.world_size, mf.global_batch_size) == (40, 5120, 13824, 8, 8)
    mg = tcfg.model_from_shell(os.path.join(ex, "moe_megatron.sh"))
    assert (mg.num_layers, mg.hidden_size, mg.expert_num, mg.num_kv_heads, mg.first_k_dense) == (24, 4096, 32, 8, 2)
    cfg = TunerConfig.from_json(os.path.join(ex, "args_for_parallel_tool.json"))
    cfg.output_path = str(tmp_path / "dense")
    ranked = taylor_search_tool(cfg, top_k=5)
    assert ranked and "step_time_us" in ranked[0]
    assert os.path.exists(os.path.join(cfg.output_path, "pipeline_output", "ranked_configs.csv"))
    moe = TunerConfig.from_json(os.path.join(ex, "args_for_moe_search.json"))
    moe.output_path, moe.alg_phase = str(tmp_path / "moe"), 1            # the pruning phases only: 32 ranks, EP on
    summary = taylor_search_tool(moe)[0]["summary"]
    assert summary["initial"] > summary["after_expert_rules"] >= summary["after_memory"] > 0
    assert os.path.exists(os.path.join(moe.output_path, "nd_candidate_config.csv"))


def test_memory_model_is_refitted_from_measured_peaks():
    """The balancer's estimate of activation memory is 40 % low: the first balance overshoots the limit
    when 'measured', the re-fit learns the true coefficients from the measured stage peaks and the next
    balance recomputes more layers and fits."""
    from hyper_parallel_b200.auto_parallel.fast_tuner import memory_fit
    from hyper_parallel_b200.auto_parallel.fast_tuner.pipeline_balance import _stage_memory
    from hyper_parallel_b200.auto_parallel.fast_tuner.pp_simulator import compute_order, simulate
    S, V, M, L = 4, 1, 8, 32
    truth = LayerProfile(act_mem=10.0, recomp_mem=1.0, layer_mem=3.0, static_mem=20.0, lm_head_mem=15.0)
    guess = LayerProfile(act_mem=6.0, recomp_mem=1.0, layer_mem=3.0, static_mem=20.0, lm_head_mem=15.0)
    live = simulate(compute_order("1f1b", M, S, V), [1.0] * S, [2.0] * S, S).peak_live

    def measure(res):
        return _stage_memory(res.layers, res.recompute, live, truth, S, V)

    limit = 260.0
    rounds = memory_fit.balance_with_memory_feedback(L, L, S, V, M, guess, limit, measure)
    assert len(rounds) >= 2 and rounds[0].over_mb > 0          # the low estimate overshoots when measured
    last = rounds[-1]
    assert last.over_mb == 0 and max(last.measured_mb) <= limit
    assert sum(map(sum, last.result.recompute)) > sum(map(sum, rounds[0].result.recompute))
    assert abs(last.profile.act_mem - truth.act_mem) < 0.5     # learnt from the measured peaks
    # a coefficient the observations cannot identify keeps its prior value
    obs = [memory_fit.MemoryObservation(8, 0, 4.0, False, 20.0 + 8 * 3.0 + 8 * 4.0 * 10.0),
           memory_fit.MemoryObservation(6, 0, 2.0, False, 20.0 + 6 * 3.0 + 6 * 2.0 * 10.0),
           memory_fit.MemoryObservation(9, 0, 3.0, False, 20.0 + 9 * 3.0 + 9 * 3.0 * 10.0)]
    fit = memory_fit.fit_memory(obs, guess)
    assert fit.recomp_mem == guess.recomp_mem and fit.lm_head_mem == guess.lm_head_mem
    assert abs(fit.act_mem - 10.0) < 1e-6 and abs(memory_fit.predict(fit, obs[0]) - obs[0].peak_mb) < 1e-6


def test_grey_box_prune_reproduces_the_reference_unit_test_count():
    """Golden vector of the reference's ``unit_tests/nd_search_test.py:28-84``: forty dry-run peaks
    (20 (dp, tp, pp) groups at ep 4 and 8) of DeepSeek-V3 on 1024 ranks, a 55 GB limit and ep <= 64
    leave exactly 10 candidates of 5 fields each."""
    info = [[32, 2, 16, 8, 142786], [128, 2, 4, 8, 188944], [16, 2, 32, 4, 153480], [16, 8, 8, 8, 96950],
            [64, 8, 2, 8, 825586], [64, 2, 8, 4, 221281], [8, 4, 32, 8, 81943], [64, 4, 4, 4, 283005],
            [64, 1, 16, 8, 241679], [32, 8, 4, 4, 270048], [8, 4, 32, 4, 98967], [256, 2, 2, 4, 1656206],
            [64, 4, 4, 8, 162045], [8, 8, 16, 8, 68632], [4, 8, 32, 8, 54686], [128, 1, 8, 4, 299846],
            [8, 8, 16, 4, 101784], [32, 8, 4, 8, 148595], [256, 1, 4, 4, 363705], [32, 4, 8, 8, 116591],
            [4, 8, 32, 4, 71710], [32, 4, 8, 4, 181999], [32, 2, 16, 4, 175938], [16, 2, 32, 8, 136456],
            [64, 8, 2, 4, 1635569], [64, 2, 8, 8, 155874], [128, 1, 8, 8, 234458], [16, 4, 16, 8, 93350],
            [256, 2, 2, 8, 847944], [128, 4, 2, 8, 832465], [16, 8, 8, 4, 162358], [32, 1, 32, 8, 245502],
            [512, 1, 2, 8, 927251], [64, 1, 16, 4, 274811], [16, 4, 16, 4, 126502], [128, 2, 4, 4, 309904],
            [32, 1, 32, 4, 262506], [256, 1, 4, 8, 242746], [128, 4, 2, 4, 1642448], [512, 1, 2, 4, 1687161]]
    out = grey_box_memory_prune(ModelSpec(expert_num=256, world_size=1024), info, [4, 8], 64, max_mem_mib=55 * 1024)
    assert len(out) == 10 and all(len(r) == 5 and r[3] <= 64 and r[4] <= 55 * 1024 for r in out)
    assert [4, 8, 32, 8, 54686] in out            # a measured point that fits is returned as measured


def test_balancer_two_layer_types_selective_recompute_and_per_stage_limits():
    """Memory table in the reference's terms (pipeline_conductor/memory.py): dense and MoE layers with
    their own activation / recompute / selective / weight sizes, a heavier first stage, the head on the
    last, one limit for stage 0, one for the middle stages, one for the last."""
    from hyper_parallel_b200.auto_parallel.fast_tuner.pipeline_balance import _stage_memory
    prof = LayerProfile(dense_fw=0.4, dense_bw=0.74, moe_fw=1.0, moe_bw=1.84, head_fw=1.5, head_bw=2.76,
                        recompute_extra=1.0, select_extra=0.25,
                        act_mem=479.0, recomp_mem=30.0, select_mem=400.0, layer_mem=866.0,
                        moe_act_mem=765.0, moe_recomp_mem=30.0, moe_select_mem=500.0, moe_layer_mem=2600.0,
                        static_mem0=3383.0, static_mem=2382.0, lm_head_mem=8675.0)
    S, V, M, L, D = 4, 2, 8, 30, 3
    free = balance_pipeline(L, D, S, V, M, prof)
    assert sum(map(sum, free.layers)) == L and sum(map(sum, free.dense)) == D
    assert not any(map(any, free.recompute)) and not any(map(any, free.select_recompute))
    assert free.dense[0][0] >= 1 and sum(free.dense[1]) == 0               # dense layers lead the model
    limits = [max(free.peak_mem) * 0.80] * S
    limits[0] = free.peak_mem[0] * 0.85
    limits[-1] = free.peak_mem[-1] * 0.9
    tight = balance_pipeline(L, D, S, V, M, prof, mem_limit_mb=limits)
    assert all(p <= l + 1e-6 for p, l in zip(tight.peak_mem, limits)), (tight.peak_mem, limits)
    assert any(map(any, tight.select_recompute)) or any(map(any, tight.recompute))
    assert tight.makespan > free.makespan                                   # recomputation costs time
    for c in range(V):
        for s in range(S):
            assert tight.recompute[c][s] + tight.select_recompute[c][s] <= tight.layers[c][s]
    # the reported peaks are those of the memory table
    from hyper_parallel_b200.auto_parallel.fast_tuner.pp_simulator import compute_order, simulate
    live = simulate(compute_order("vpp", M, S, V), [1.0] * (S * V), [2.0] * (S * V), S).peak_live
    again = _stage_memory(tight.layers, tight.recompute, live, prof, S, V, tight.dense, tight.select_recompute)
    assert all(abs(a - b) < 1e-6 for a, b in zip(again, tight.peak_mem))
    # when only full recomputation exists it is used, and costs more time than the selective mix
    full_only = balance_pipeline(L, D, S, V, M, LayerProfile(**{**prof.__dict__, "select_mem": None,
                                                                "moe_select_mem": None}), mem_limit_mb=limits)
    assert not any(map(any, full_only.select_recompute)) and any(map(any, full_only.recompute))
    with pytest.raises(ValueError):
        balance_pipeline(L, D, S, V, M, prof, mem_limit_mb=[1.0, 2.0])
