"""Configuration schema / loader / presets / validator, autoconfig solver (levers, pins, refusals,
explain sidecar), hardware descriptor, CLIs.  All CPU."""
import json
import os

import pytest

from layerstorm_b200.autoconfig import AutoconfigRefusal, HardwareInfo, Levers, PINNABLE, detect, explain_text, sizing, solve, synthetic, write_result
from layerstorm_b200.config import (ConfigError, PRESET_OVERLAYS, apply_env, defaults, get_path, json_schema, leaf_paths,
                                    live_changeable_fields, load_config, model_config_from, model_section_from, parse_pin)
from layerstorm_b200.models.config import get_preset


# ---------------------------------------------------------------- schema / loader
def test_defaults_are_valid_and_complete():
    cfg = load_config()
    assert cfg["preset"] == "balanced"
    for path, leaf in leaf_paths():
        assert get_path(cfg, path, "<missing>") != "<missing>", path
    assert cfg["memory"]["kv_cache"]["page_size_tokens"] == 64
    assert set(cfg) >= {"model", "quantization", "hardware", "memory", "orchestrator", "prefetch", "speculation", "parallelism",
                        "transfer", "compute", "serving", "preprocessing", "autoconfig", "gpu_loader"}


def test_unknown_key_type_enum_and_range_are_reported_together():
    with pytest.raises(ConfigError) as e:
        load_config({"serving": {"prot": 1, "port": "x"}, "quantization": {"weights": "int3"},
                     "memory": {"kv_cache": {"speculation_pool_fraction": 1.5}}})
    msg = "\n".join(e.value.problems)
    assert "serving.prot: unknown key" in msg and "serving.port: expected int" in msg
    assert "quantization.weights" in msg and "speculation_pool_fraction" in msg and len(e.value.problems) == 4


def test_internal_sections_and_nulls_pass_through():
    cfg = load_config({"_internal-scheduler": {"anything": 1}, "hardware": {"system_ram_gb": None, "nvme_capacity_gb": None},
                       "serving": {"port": None}})
    assert cfg["_internal-scheduler"] == {"anything": 1}
    assert cfg["serving"]["port"] == 8000 and cfg["hardware"]["system_ram_gb"] is None


def test_preset_overlay_then_user_then_override():
    cfg = load_config({"preset": "min_latency", "orchestrator": {"max_batch_size": 48}}, {"serving.port": 9001})
    assert cfg["orchestrator"]["max_batch_size"] == 48                       # user beats preset (32)
    assert cfg["orchestrator"]["expert_batching"]["max_wait_us"] == 10       # preset beats default (50)
    assert cfg["serving"]["port"] == 9001
    assert load_config({"preset": "max_throughput"})["orchestrator"]["max_batch_size"] == 128
    with pytest.raises(ConfigError):
        load_config(None, {"preset": "warp_speed"})
    assert set(PRESET_OVERLAYS) >= {"balanced", "min_latency", "max_throughput"}


def test_semantic_rules():
    def bad(over, needle):
        with pytest.raises(ConfigError) as e:
            load_config(over)
        assert needle in str(e.value), str(e.value)
    bad({"model": {"num_attention_heads": 6}, "parallelism": {"tensor_parallelism": 4}}, "does not divide")
    bad({"hardware": {"gpus": [{"id": 0}, {"id": 0}]}}, "duplicate")
    bad({"hardware": {"gpus": [{"id": 0, "roles": ["mining"]}]}}, "unknown role")
    bad({"model": {"architecture": "deepseek_v3"}, "compute": {"attention_backend": "csa_hca"}}, "only defined for architecture deepseek_v4")
    bad({"speculation": {"method": "dspark"}}, "checkpoint_path")
    bad({"memory": {"nvme_tier": {"enabled": True}}}, "nvme_paths")
    bad({"model": {"weights_format": "gguf"}}, "gguf* weight format")
    bad({"orchestrator": {"performance_objective": {"latency_weight": 0.9}}}, "must be 1")
    bad({"model": {"num_hidden_layers": 3, "layer_types": ["linear_attention"]}}, "layer_types")


@pytest.mark.parametrize("name", ["glm53_flash_gguf.json", "glm_5_2_gguf.json", "valid_deepseek_v3_2.json", "deepseek_v4_flash_gguf.json"])
def test_reference_style_config_documents_load(name, tmp_path):
    """Documents written for the reference's schema (same section / field names) load unchanged.  The
    samples are rebuilt here from the model presets rather than read from outside the repository."""
    mc = {"glm53_flash_gguf.json": "glm-5.3-flash", "glm_5_2_gguf.json": "glm-5.2", "valid_deepseek_v3_2.json": "deepseek-v3.2",
          "deepseek_v4_flash_gguf.json": "glm-5.3-flash"}[name]
    shape = get_preset(mc)
    doc = {"model": model_section_from(shape), "quantization": {"weights": "nvfp4", "kv_cache": "fp8_e4m3"},
           "hardware": {"gpus": [{"id": i, "type": "b200", "vram_gb": 180, "roles": ["attention", "resident", "expert_streaming"]} for i in range(2)],
                        "nvme_capacity_gb": None, "dcp_kv_mode": "sharded"},
           "parallelism": {"tensor_parallelism": 2}, "serving": {"port": 8123}}
    p = tmp_path / name
    p.write_text(json.dumps(doc))
    cfg = load_config(str(p))
    back = model_config_from(cfg)
    for f in ("hidden", "n_layers", "n_heads", "kv_lora", "qk_nope", "qk_rope", "v_head", "n_routed", "top_k", "moe_inter", "index_kpool",
              "layer_types", "hc_mult", "kda_heads", "kda_rank", "index_n_heads", "scoring", "routed_scale", "swiglu_limit"):
        assert getattr(back, f) == getattr(shape, f), f


def test_json_schema_and_live_fields():
    js = json_schema()
    assert js["properties"]["model"]["properties"]["architecture"]["enum"][0] == "deepseek_v3"
    assert js["properties"]["serving"]["additionalProperties"] is False
    live = live_changeable_fields()
    assert "orchestrator.max_batch_size" in live and "model.hidden_size" not in live


def test_env_switches_and_pins():
    cfg = apply_env(load_config(), {"LS_DETERMINISTIC": "1", "LAYERSTORM_DETERMINISTIC_EP_COMBINE_PRECISION": "bf16"})
    assert cfg["compute"]["deterministic"] and cfg["compute"]["deterministic_ep_combine_precision"] == "bf16"
    cfg = apply_env(load_config(), {"LAYERSTORM_DETERMINISTIC_EP_COMBINE": "0", "LS_REFERENCE_TRAJECTORY_IDENTITY": "1"})
    assert cfg["compute"]["deterministic_ep_combine"] is False and cfg["compute"]["reference_trajectory_identity"]
    assert parse_pin("parallelism.tensor_parallelism=2") == ("parallelism.tensor_parallelism", 2)
    assert parse_pin("compute.attention_backend=snapmla") == ("compute.attention_backend", "snapmla")
    assert parse_pin("memory.kv_tiering.enabled=true")[1] is True


# ---------------------------------------------------------------- sizing / solver
def test_sizing_matches_known_layouts():
    mc = get_preset("glm-5.3-flash")
    assert sizing.kv_row_bytes(mc, "snapmla") == 512 + 16                       # NoPE: fp8 latent + scale slot
    ds = get_preset("deepseek-v3.2")
    assert sizing.kv_row_bytes(ds, "snapmla") == 512 + 16 + 128                 # + 64 bf16 rope
    assert sizing.kv_row_bytes(ds, "bf16_mla") == 576 * 2
    assert sizing.kv_row_bytes(ds, "turboquant_mla") < sizing.kv_row_bytes(ds, "snapmla")
    slot = sizing.expert_slot_bytes(mc)
    assert slot % 4096 == 0 and 13.5e6 < slot < 14.5e6                          # 3 x 4096 x 2048 x 4.5 bit
    total = sizing.resident_bytes(mc, 1, 1, True).total + slot * 288 * mc.n_moe_layers()
    assert 160e9 < total < 190e9                                                # the whole model fits one 180 GB GPU
    assert sizing.recurrent_state_bytes_per_seq(mc, 2) * 2 == pytest.approx(sizing.recurrent_state_bytes_per_seq(mc, 1), rel=1e-6)
    assert sizing.kv_bytes_per_token(ds, "snapmla", 2, "sharded") * 2 == pytest.approx(sizing.kv_bytes_per_token(ds, "snapmla", 1), rel=1e-6)


def test_solver_full_machine_and_single_gpu():
    mc = get_preset("glm-5.3-flash")
    r8 = solve(mc, synthetic(8))
    assert r8.candidate.tp == 8 and r8.config["parallelism"]["expert_parallelism"] == 8
    assert r8.config["hardware"]["dcp_kv_mode"] == "sharded" and r8.config["compute"]["attention_backend"] == "snapmla"
    assert r8.warnings == [] and r8.config["autoconfig"]["vram_expert_ratio"] == 1.0
    assert [s["step"] for s in r8.explain["steps"]][:3] == ["P1", "P2", "K1"]
    r1 = solve(mc, synthetic(1), Levers(total_active_context_tokens=8 * 32768))
    assert r1.candidate.tp == 1 and r1.candidate.concurrency * r1.candidate.seq_len <= 8 * 32768
    big = solve(get_preset("deepseek-v3.2"), synthetic(1))
    assert big.config["autoconfig"]["vram_expert_ratio"] < 1.0 and big.config["memory"]["pin_host_expert_pool"] and big.warnings


def test_prefer_is_a_sort_key_never_a_refusal():
    mc = get_preset("glm-5.2")
    outs = {p: solve(mc, synthetic(8), Levers(prefer=p)) for p in ("speed", "balanced", "capacity")}
    ctx = {(r.candidate.concurrency, r.candidate.seq_len) for r in outs.values()}
    assert len(ctx) == 1                      # every preference lands on the same relaxation level
    assert outs["capacity"].candidate.report.expert_slots_per_layer >= outs["speed"].candidate.report.expert_slots_per_layer


def test_pins_bind_and_refusals_name_them():
    mc = get_preset("glm-5.3-flash")
    r = solve(mc, synthetic(8), pins={"parallelism.tensor_parallelism": 2, "serving.max_concurrent_requests": 4})
    assert r.candidate.tp == 2 and r.config["serving"]["max_concurrent_requests"] == 4 and len(r.config["hardware"]["tp_array"]) == 2
    with pytest.raises(AutoconfigRefusal) as e:
        solve(mc, synthetic(8), pins={"parallelism.tensor_parallelism": 3})
    assert e.value.binding == "parallelism.tensor_parallelism"
    with pytest.raises(AutoconfigRefusal) as e:
        solve(mc, synthetic(8), pins={"model.hidden_size": 1})
    assert "not a pinnable field" in str(e.value)
    with pytest.raises(AutoconfigRefusal) as e:
        solve(mc, synthetic(8), Levers(accuracy="high"), pins={"compute.attention_backend": "turboquant_mla"})
    assert "accuracy floor" in str(e.value)
    with pytest.raises(AutoconfigRefusal) as e:       # a 1M-token pinned length on a small GPU cannot be relaxed away
        solve(get_preset("deepseek-v3.2"), synthetic(1, vram_gb=48, ram_gb=2048), pins={"serving.max_sequence_length": 1 << 20, "serving.max_concurrent_requests": 64})
    assert e.value.binding.startswith("serving.max_")
    with pytest.raises(AutoconfigRefusal) as e:
        solve(get_preset("deepseek-v3.2"), synthetic(1, vram_gb=32, ram_gb=64))
    assert "no configuration fits" in str(e.value)
    with pytest.raises(AutoconfigRefusal):
        solve(mc, HardwareInfo())
    assert "compute.attention_backend" in PINNABLE


def test_accuracy_floor_and_vram_ratio_lever():
    mc = get_preset("deepseek-v3.2")
    assert solve(mc, synthetic(8), Levers(accuracy="compact")).config["quantization"]["kv_cache"] == "turboquant4"
    assert solve(mc, synthetic(8), Levers(accuracy="superior")).config["quantization"]["kv_cache"] == "bf16"
    with pytest.raises(AutoconfigRefusal) as e:
        solve(mc, synthetic(1), Levers(vram_expert_ratio=1.0))
    assert "vram_expert_ratio" in str(e.value)


def test_result_files_and_fingerprint(tmp_path):
    r = solve(get_preset("tiny-glm5-next"), synthetic(2))
    cfg_path, side = write_result(r, str(tmp_path / "ac.json"))
    again = load_config(cfg_path)
    assert again["autoconfig"]["fingerprint"] == synthetic(2).fingerprint() != synthetic(4).fingerprint()
    ex = json.load(open(side))
    assert ex["explain"]["steps"] and "modelled_decode_ms" in ex["explain"]
    assert "tp=" in explain_text(r)
    hw = HardwareInfo.from_dict(json.loads(json.dumps(synthetic(3).to_dict())))
    assert len(hw.gpus) == 3 and hw.fingerprint() == synthetic(3).fingerprint()


def test_detect_does_not_need_a_gpu():
    hw = detect()
    assert hw.system_ram_gb > 0 and hw.cpu_cores > 0 and hw.numa_nodes >= 1
    assert isinstance(hw.hardware_section()["gpus"], list)


# ---------------------------------------------------------------- CLIs
def test_autoconfigure_cli(tmp_path, capsys):
    from layerstorm_b200.cli import autoconfigure
    out = tmp_path / "o.json"
    assert autoconfigure.main(["--model", "glm-5.3-flash", "--assume-gpus", "8", "-o", str(out), "--print", "--pin", "parallelism.tensor_parallelism=4"]) == 0
    assert json.load(open(out))["parallelism"]["tensor_parallelism"] == 4 and os.path.exists(str(out) + ".explain.json")
    assert autoconfigure.main(["--model", "glm-5.3-flash", "--assume-gpus", "8", "-o", str(out), "--pin", "parallelism.tensor_parallelism=3"]) == 3
    assert "relax: parallelism.tensor_parallelism" in capsys.readouterr().err


def test_serve_cli_flags_and_dry_run(tmp_path, capsys):
    from layerstorm_b200.cli import serve
    flags = {a.option_strings[0] for a in serve.build_parser()._actions if a.option_strings}
    for f in ("--config", "--autoconfig", "--model", "--accuracy", "--prefer", "--host", "--port", "--model-name", "--tokenizer-path",
              "--max-concurrent", "--max-queued-requests", "--sse-heartbeat-seconds", "--max-sequence-length", "--tool-call-parser",
              "--enable-auto-tool-choice", "--reasoning-parser", "--reasoning-config", "--tokenizer-mode", "--speculation-depth",
              "--cycle-budget-us", "--log-level", "--test-engine", "--autoconfig-redetect"):
        assert f in flags, f
    assert serve.main(["--model", "tiny-glm5-next", "--autoconfig", "--test-engine", "--dry-run", "--port", "8123", "--max-concurrent", "2"]) == 0
    cfg = json.loads(capsys.readouterr().out)
    assert cfg["serving"]["port"] == 8123 and cfg["serving"]["max_concurrent_requests"] == 2 and cfg["autoconfig"]["enabled"]
    bad = tmp_path / "bad.json"
    bad.write_text(json.dumps({"serving": {"prot": 1}}))
    assert serve.main(["--config", str(bad), "--test-engine", "--dry-run"]) == 2


def test_serve_cli_builds_a_working_server_on_the_null_engine():
    from fastapi.testclient import TestClient
    from layerstorm_b200.cli import serve
    import threading
    args = serve.build_parser().parse_args(["--model", "tiny-mla-moe", "--test-engine", "--model-name", "unit", "--tokenizer-mode", "byte"])
    cfg, shape, ckpt, _ = serve.resolve_config(args)
    eng = serve.build_engine(cfg, shape, ckpt, args)
    server, orch = serve.build_server(cfg, shape, ckpt, eng, args)
    t = threading.Thread(target=orch.run, daemon=True)
    t.start()
    try:
        c = TestClient(server.app)
        assert c.get("/health").json()["status"] == "ok"
        assert c.get("/v1/models").json()["data"][0]["id"] == "unit"
        r = c.post("/v1/completions", json={"prompt": "hello", "max_tokens": 4})
        assert r.status_code == 200 and r.json()["usage"]["completion_tokens"] >= 1
    finally:
        orch.shutdown()
        t.join(timeout=5)


def test_family_template_is_copied_and_pins_win():
    from layerstorm_b200.autoconfig import Levers, solve, synthetic, templates
    from layerstorm_b200.models.config import glm_5_3_flash, deepseek_v3_2
    res = solve(glm_5_3_flash(), synthetic(8), Levers(None, None, "balanced", "standard"), {"serving.max_concurrent_requests": 4})
    assert res.config["serving"]["tool_call_parser"] == "glm47" and res.config["serving"]["reasoning_parser"] == "glm45"
    assert res.config["orchestrator"]["prefill_chunk_tokens"] == 2048          # few concurrent requests: throughput-sized chunks
    t1 = [s for s in res.explain["steps"] if s["step"] == "T1"][0]
    assert t1["decision"]["family"] == "glm5_next" and "serving.tool_call_parser" in t1["decision"]["copied"]
    res2 = solve(deepseek_v3_2(), synthetic(8), Levers(None, None, "balanced", "standard"), {},
                 {"serving": {"reasoning_parser": "glm45", "tool_call_parser": "hermes"}})
    assert res2.config["serving"]["tool_call_parser"] == "hermes" and res2.config["serving"]["reasoning_parser"] == "glm45"
    t1 = [s for s in res2.explain["steps"] if s["step"] == "T1"][0]
    assert "serving.reasoning_parser" not in t1["decision"]["copied"] and "serving.tool_call_parser" not in t1["decision"]["copied"]
    assert res2.config["orchestrator"]["prefill_chunk_tokens"] == 256           # default concurrency 32
    assert templates.family_of("unknown") == "mla_dsa" and templates.template_for("deepseek_v4")["serving"]["tool_call_parser"] == "deepseek_v4"


def test_champion_comparison(tmp_path):
    from layerstorm_b200.autoconfig import compare as cmp
    champ = {"metric": "decode_tok_s", "value": 100.0, "higher_is_better": True, "e2e": {"value": 95.0}, "extra": {"ttft_ms": 400.0, "prefill_tok_s": 5000.0}}
    cand = {"metric": "decode_tok_s", "value": 98.0, "higher_is_better": True, "e2e": {"value": 96.0}, "extra": {"ttft_ms": 380.0, "prefill_tok_s": 5100.0}}
    rep = cmp.compare(champ, cand, 0.03)
    assert rep["pass"] and {r["metric"] for r in rep["metrics"]} == {"decode_tok_s", "e2e", "ttft_ms", "prefill_tok_s"}
    slow = dict(cand, extra={"ttft_ms": 500.0, "prefill_tok_s": 5100.0})
    rep = cmp.compare(champ, slow, 0.03)
    assert not rep["pass"] and [r["metric"] for r in rep["metrics"] if not r["pass"]] == ["ttft_ms"]
    assert not cmp.compare(champ, {"metric": "decode_tok_s", "value": 100.0}, 0.03)["pass"]      # sub-metrics missing
    a, b = tmp_path / "a.log", tmp_path / "b.json"
    a.write_text("warming up\n" + json.dumps(champ) + "\n")
    b.write_text(json.dumps(cand))
    assert cmp.main([str(a), str(b)]) == 0
    assert cmp.config_diff({"x": {"y": 1, "z": 2}}, {"x": {"y": 1, "z": 3}, "w": 0}) == [("w", None, 0), ("x.z", 2, 3)]


def test_calibration_replaces_default_bandwidths(tmp_path):
    from layerstorm_b200.autoconfig import synthetic
    from layerstorm_b200.autoconfig.calibration import apply_calibration
    from layerstorm_b200.cli import autoconfigure
    hw = synthetic(8)
    doc = {"version": 1, "devices": [{"a_ns": 30000, "b_ns": 2500}], "banks": [{"rate_bytes_per_us": [48000, 52000], "latency_ns": [9000, 9000]}],
           "hbm_gbs": 7100.0, "nvlink_gbs": 5.0}
    hw2, notes = apply_calibration(hw, doc)
    assert hw2.h2d_gbs == 48.0 and hw2.hbm_gbs == 7100.0 and hw2.nvlink_gbs == hw.nvlink_gbs and hw.h2d_gbs == 55.0
    assert any("ignored" in n and "nvlink" in n for n in notes) and any("cost curve" in n for n in notes)
    p = tmp_path / "cal.json"
    p.write_text(json.dumps(doc))
    out = tmp_path / "cfg.json"
    assert autoconfigure.main(["--model", "glm-5.3-flash", "--assume-gpus", "8", "--calibration", str(p), "-o", str(out)]) == 0
    assert json.load(open(out))["serving"]["tool_call_parser"] == "glm47"


def test_benchmark_mode_on_the_null_engine(tmp_path, capsys):
    from layerstorm_b200 import build as _build
    _build.build_all(only="runtime")
    from layerstorm_b200.autoconfig import benchmark, compare
    out = tmp_path / "rep.json"
    rc = benchmark.main(["--prompt-len", "300", "--gen", "8", "--requests", "2", "--out", str(out), "--",
                         "--model", "tiny-mla-moe", "--test-engine"])
    assert rc == 0
    rep = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rep == json.load(open(out)) and rep["metric"] == "decode_tok_s" and rep["value"] > 0
    assert rep["extra"]["prefill_tok_s"] > 0 and rep["extra"]["ttft_ms"] > 0 and rep["config"]["model"]
    assert compare.compare(rep, rep)["pass"]
    # too long for the configured sequence length: refused before anything is built
    assert benchmark.main(["--prompt-len", "100000000", "--", "--model", "tiny-mla-moe", "--test-engine"]) == 2


def test_schema_exports_and_check_cli(tmp_path, capsys):
    """Everything generated from the schema tree: JSON-Schema, defaults, live-changeable fields, the markdown field reference, and the
    document check used from the command line."""
    import json
    from layerstorm_b200.config import schema
    assert schema.main(["--emit", "json-schema"]) == 0
    js = json.loads(capsys.readouterr().out)
    assert js["type"] == "object" and "serving" in js["properties"] and js["$schema"].startswith("https://json-schema.org")
    assert schema.main(["--emit", "live-fields"]) == 0
    live = capsys.readouterr().out.split()
    assert live == schema.live_changeable_fields() and "memory.expert_cache.eviction_policy" in live
    assert schema.main(["--emit", "markdown"]) == 0
    md = capsys.readouterr().out
    assert md.count("\n") >= len(list(schema.leaf_paths())) and "| `preset` | str |" in md
    good = tmp_path / "good.json"
    good.write_text(json.dumps({"preset": "min_latency"}))
    assert schema.main(["--check", str(good)]) == 0
    bad = tmp_path / "bad.json"
    bad.write_text(json.dumps({"serving": {"port": "x"}}))
    assert schema.main(["--check", str(bad)]) == 1


def test_auto_run_pipeline_orders_reuses_and_carries_artifacts(tmp_path):
    """calibrate -> derive -> train -> place -> derive with fake GPU steps: a model that does not fit runs all four, the second
    invocation reuses both measured artifacts, --reset measures again, a model that fits stops after the derivation; the final
    configuration names the trained constants and the placement table."""
    import json
    from layerstorm_b200.autoconfig import Levers, synthetic
    from layerstorm_b200.autoconfig.pipeline import AutoRunOptions, Runners, run_pipeline
    from layerstorm_b200.models.config import get_preset
    from layerstorm_b200.utils.cache_sim import synthetic_trace, write_trace
    calls = []

    def calibrate(path):
        calls.append("calibrate")
        return {"version": 2, "h2d_gbs": 50.0}

    def training_decode(config_path, ftrace, rtrace, log):
        calls.append("train")
        cfg = json.load(open(config_path))
        assert cfg["gpu_loader"]["calibration_path"].endswith(".json") and cfg["autoconfig"]["vram_expert_ratio"] < 1.0
        write_trace(rtrace, synthetic_trace(steps=30, layers=4, n_experts=64, top_k=8, seed=1))
        with open(ftrace, "w") as fh:
            for i in range(50):
                n = 1 + i % 6
                fh.write(f"W {i} {n} {n * (20 << 20)} {25.0 + n * (20 << 20) / 42e3:.1f}\n")       # 42 GB/s, 25 us per batch
        return {"value": 7.5, "unit": "tok/s"}

    runners = Runners(calibrate, training_decode)
    big = get_preset("glm-5.2")                              # does not fit one GPU: experts stream
    hw1 = synthetic(1)
    opts = AutoRunOptions(model="glm-5.2", out_dir=str(tmp_path), train_gen=8)
    rec = run_pipeline(big, hw1, Levers(), {}, None, opts, runners)
    assert calls == ["calibrate", "train"]
    names = [(s["step"], s["ran"]) for s in rec["steps"]]
    assert names == [("calibrate", True), ("derive", True), ("train", True), ("place", True), ("derive", True)]
    train = next(s for s in rec["steps"] if s["step"] == "train")
    assert abs(train["h2d_gb_s"] - 42.0) < 0.5
    cfg = json.load(open(rec["config"]))
    assert cfg["gpu_loader"]["calibration_path"] == rec["artifacts"]["trained"]
    assert cfg["memory"]["arena_placement"]["freq_table"] == rec["artifacts"]["placement"]
    assert open(rec["artifacts"]["placement"]).read().count("\n") > 10
    assert json.load(open(rec["artifacts"]["autorun"]))["fingerprint"] == rec["fingerprint"]
    # again: both measured artifacts match this machine and model -> nothing runs on the GPU
    rec2 = run_pipeline(big, hw1, Levers(), {}, None, opts, runners)
    assert calls == ["calibrate", "train"]
    assert [(s["step"], s["ran"]) for s in rec2["steps"]][:1] == [("calibrate", False)] and not any(s["ran"] for s in rec2["steps"] if s["step"] in ("train", "place"))
    # other hardware: the artifacts do not match -> measured again; so does --reset
    run_pipeline(big, synthetic(1, vram_gb=96.0), Levers(), {}, None, opts, runners)
    assert calls == ["calibrate", "train", "calibrate", "train"]
    run_pipeline(big, synthetic(1, vram_gb=96.0), Levers(), {}, None, AutoRunOptions(model="glm-5.2", out_dir=str(tmp_path), reset=True), runners)
    assert calls[-2:] == ["calibrate", "train"] and len(calls) == 6
    # a model that fits: no loader to train
    calls.clear()
    small = get_preset("tiny-mla-moe")
    rec3 = run_pipeline(small, synthetic(1), Levers(), {}, None, AutoRunOptions(model="tiny-mla-moe", out_dir=str(tmp_path / "s")), runners)
    assert calls == ["calibrate"] and [s["ran"] for s in rec3["steps"] if s["step"] in ("train", "place")] == [False, False]


def test_engine_cross_check_table_semantics():
    """Exact rows fail on any divergence, bound rows warn when the solver over-estimates and fail when it under-estimates, rows
    without a figure are reported unchecked."""
    from layerstorm_b200.autoconfig.enginecheck import CheckRow, render, run_checks

    class Eng:
        cfg = None

    rows = [CheckRow("a", "B", "exact", 0.0, lambda mc, c: 100.0, lambda e: 100.0),
            CheckRow("b", "B", "exact", 0.0, lambda mc, c: 101.0, lambda e: 100.0),
            CheckRow("c", "B", "upper_bound", 0.1, lambda mc, c: 105.0, lambda e: 100.0),
            CheckRow("d", "B", "upper_bound", 0.1, lambda mc, c: 130.0, lambda e: 100.0),
            CheckRow("e", "B", "upper_bound", 0.1, lambda mc, c: 99.0, lambda e: 100.0),
            CheckRow("f", "B", "exact", 0.0, lambda mc, c: None, lambda e: 1.0),
            CheckRow("g", "B", "exact", 0.0, lambda mc, c: 1 / 0, lambda e: 1.0)]
    res = run_checks(Eng(), ctx={}, rows=rows)
    assert [r.status for r in res] == ["ok", "FAIL", "ok", "warning", "FAIL", "unchecked", "unchecked"]
    assert "UNDER-estimates" in res[4].note and "ZeroDivisionError" in res[6].note
    assert "quantity" in render(res) and "warning" in render(res)


def test_solver_resident_bytes_bound_the_models_own_tensors():
    """The sizing formula for the weights every GPU keeps (everything but the expert arenas) against the tensors the model really
    builds: never below, and within 2 % above, for every tiny architecture (MLA, KDA + hyper-connections + pooled indexer, DSA)."""
    from layerstorm_b200.autoconfig import sizing
    from layerstorm_b200.models.config import get_preset
    from layerstorm_b200.models.device_model import DeviceModel
    from layerstorm_b200.models.weights import init_weights
    for name in ("tiny-mla-moe", "tiny-glm5-next", "tiny-deepseek-v32"):
        cfg = get_preset(name)
        m = DeviceModel.from_state_dict(cfg, init_weights(cfg, 0), "cpu", kv_fmt="fp8", page=16)
        arenas = [L["arena"] for L in m.layers if L.get("arena") is not None]
        engine = m.weight_bytes() - sum(a.data.numel() for a in arenas) + m.embed.numel() * 2      # (the count skips a host-side embedding)
        rb = sizing.resident_bytes(cfg, 1, 1, False)
        solver = rb.total - rb.shared_expert
        assert engine <= solver <= engine * 1.02, (name, engine, solver)
