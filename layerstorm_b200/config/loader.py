"""Load, merge, validate and resolve engine configuration documents.

Order of precedence (lowest first): schema defaults < preset overlay < the user's JSON < explicit
overrides (CLI flags, ``path=value`` pins).  Validation is strict about unknown keys (a typo must
not be silently ignored) except for the ``_internal-*`` top-level sections and ``_advanced`` maps,
which are passed through.  Reference: config/schema.json + the generated C++ parser
(tools/gen_config.mjs) and presets in config/presets/.
"""
from __future__ import annotations

import copy
import json
import os
from typing import Any

from ..models.config import ModelConfig, from_hf_config
from .schema import F, SCHEMA, defaults

# Preset overlays: the three operating points of the reference (config/presets/*.json), re-tuned for
# a machine whose experts mostly stay resident in HBM.
PRESET_OVERLAYS: dict[str, dict] = {
    "": {},
    "balanced": {},
    "min_latency": {
        "orchestrator": {"performance_objective": {"latency_weight": 0.9, "throughput_weight": 0.1},
                         "max_batch_size": 32,
                         "expert_batching": {"max_wait_us": 10, "min_batch_tokens_per_expert": 1}},
        "speculation": {"mtp": {"max_depth": 1, "dynamic_depth": False},
                        "verification": {"verification_quality_floor": 0.95},
                        "reasoning_mode": {"enabled": True}},
        "prefetch": {"speculative": {"max_prefetch_depth_layers": 4, "confidence_threshold": 0.3},
                     "probe": {"confidence_threshold": 0.8}},
        "memory": {"expert_cache": {"stable_zone_fraction": 0.8}, "kv_cache": {"speculation_pool_fraction": 0.1}},
    },
    "max_throughput": {
        "orchestrator": {"performance_objective": {"latency_weight": 0.2, "throughput_weight": 0.8},
                         "max_batch_size": 128,
                         "expert_batching": {"max_wait_us": 200, "min_batch_tokens_per_expert": 8},
                         "prefill_chunk_tokens": 1024},
        "speculation": {"mtp": {"max_depth": 2}},
        "memory": {"expert_cache": {"stable_zone_fraction": 0.6}, "kv_cache": {"speculation_pool_fraction": 0.2}},
        "compute": {"prefill_superchunk_tokens": 8192},
    },
}


# attention = MLA/DSA/KDA compute, resident = pinned dense layers / embedding / gating / head,
# expert_streaming = expert cache and MoE execution, draft = speculative draft model
GPU_ROLES = ("attention", "resident", "expert_streaming", "draft")


class ConfigError(ValueError):
    """Raised with every problem found, one per line, each naming the dotted path."""

    def __init__(self, problems: list[str]):
        super().__init__("invalid configuration:\n  " + "\n  ".join(problems))
        self.problems = problems


def deep_merge(base: dict, over: dict) -> dict:
    """Recursive dict merge; lists and scalars in ``over`` replace those in ``base``."""
    out = dict(base)
    for k, v in over.items():
        if isinstance(v, dict) and isinstance(out.get(k), dict):
            out[k] = deep_merge(out[k], v)
        else:
            out[k] = copy.deepcopy(v)
    return out


def set_path(cfg: dict, path: str, value: Any) -> None:
    parts = path.split(".")
    node = cfg
    for p in parts[:-1]:
        node = node.setdefault(p, {})
    node[parts[-1]] = value


def get_path(cfg: dict, path: str, default: Any = None) -> Any:
    node: Any = cfg
    for p in path.split("."):
        if not isinstance(node, dict) or p not in node:
            return default
        node = node[p]
    return node


def parse_pin(text: str) -> tuple[str, Any]:
    """``path=value`` with the value read as JSON when it parses (numbers, booleans, lists), else as a string."""
    if "=" not in text:
        raise ConfigError([f"pin '{text}' is not of the form path=value"])
    path, raw = text.split("=", 1)
    try:
        val = json.loads(raw)
    except json.JSONDecodeError:
        val = raw
    return path.strip(), val


def _check_leaf(path: str, f: F, v: Any, out: list[str]) -> None:
    if v is None:          # null means "not set": the default (or the automatic value) applies
        return
    types = f.type if isinstance(f.type, tuple) else (f.type,)
    ok = False
    for t in types:
        if t is float and isinstance(v, (int, float)) and not isinstance(v, bool):
            ok = True
        elif t is int and isinstance(v, int) and not isinstance(v, bool):
            ok = True
        elif t is int and isinstance(v, float) and v == int(v):
            ok = True
        elif t in (str, bool, list, dict) and isinstance(v, t):
            ok = True
    if not ok:
        out.append(f"{path}: expected {'/'.join(t.__name__ for t in types)}, got {type(v).__name__} ({v!r})")
        return
    if f.enum and v not in f.enum:
        out.append(f"{path}: {v!r} is not one of {list(f.enum)}")
    if isinstance(v, (int, float)) and not isinstance(v, bool):
        if f.lo is not None and v < f.lo:
            out.append(f"{path}: {v} is below the minimum {f.lo}")
        if f.hi is not None and v > f.hi:
            out.append(f"{path}: {v} is above the maximum {f.hi}")


def _check_tree(node: dict, spec: dict, prefix: str, out: list[str]) -> None:
    for k, v in node.items():
        path = f"{prefix}{k}"
        if prefix == "" and k.startswith("_internal-"):
            continue
        if k.startswith("$") or k == "_comment":
            continue
        if k not in spec:
            out.append(f"{path}: unknown key")
            continue
        s = spec[k]
        if isinstance(s, F):
            _check_leaf(path, s, v, out)
        elif not isinstance(v, dict):
            out.append(f"{path}: expected an object")
        else:
            _check_tree(v, s, path + ".", out)


def structural_problems(cfg: dict) -> list[str]:
    out: list[str] = []
    _check_tree(cfg, SCHEMA, "", out)
    return out


def semantic_problems(cfg: dict) -> list[str]:
    """Cross-field rules (the part a JSON-Schema cannot express)."""
    out: list[str] = []
    m = cfg["model"]
    tp = cfg["parallelism"]["tensor_parallelism"]
    heads = m["num_attention_heads"]
    if heads and heads % tp:
        out.append(f"parallelism.tensor_parallelism: {tp} does not divide model.num_attention_heads ({heads})")
    gpus = cfg["hardware"]["gpus"]
    if gpus:
        att = [g for g in gpus if "attention" in (g.get("roles") or GPU_ROLES)]
        if len(att) < tp:
            out.append(f"hardware.gpus: {len(att)} GPU(s) carry the attention role but tensor_parallelism is {tp}")
        ids = [g.get("id", g.get("device_id")) for g in gpus]
        if len(set(ids)) != len(ids):
            out.append("hardware.gpus: duplicate device_id")
        for i, g in enumerate(gpus):
            for r in g.get("roles") or []:
                if r not in GPU_ROLES:
                    out.append(f"hardware.gpus[{i}].roles: unknown role {r!r}")
    ta = cfg["hardware"]["tp_array"]
    if ta is not None and len(ta) != tp:
        out.append(f"hardware.tp_array: has {len(ta)} entries but tensor_parallelism is {tp}")
    lt = m["layer_types"]
    if lt and m["num_hidden_layers"] and len(lt) != m["num_hidden_layers"]:
        out.append(f"model.layer_types: {len(lt)} entries for {m['num_hidden_layers']} layers")
    if m["num_experts_per_tok"] and m["n_routed_experts"] and m["num_experts_per_tok"] > m["n_routed_experts"]:
        out.append("model.num_experts_per_tok exceeds model.n_routed_experts")
    if m["n_group"] > 1 and m["n_routed_experts"] % m["n_group"]:
        out.append("model.n_group does not divide model.n_routed_experts")
    if m["topk_group"] > m["n_group"]:
        out.append("model.topk_group exceeds model.n_group")
    ab = cfg["compute"]["attention_backend"]
    arch = m["architecture"]
    if ab.startswith("csa_hca") and arch != "deepseek_v4":
        out.append(f"compute.attention_backend: {ab} is only defined for architecture deepseek_v4")
    if arch == "deepseek_v4" and not ab.startswith("csa_hca"):
        out.append(f"compute.attention_backend: architecture deepseek_v4 needs a csa_hca* backend, not {ab}")
    if ab == "turboquant_mla" and cfg["quantization"]["kv_cache"] not in ("turboquant4", "fp8_e4m3"):
        out.append("quantization.kv_cache: turboquant_mla stores 4-bit rows; use turboquant4")
    fw = cfg["orchestrator"]["performance_objective"]
    if abs(fw["latency_weight"] + fw["throughput_weight"] - 1.0) > 1e-6:
        out.append("orchestrator.performance_objective: latency_weight + throughput_weight must be 1")
    sp = cfg["speculation"]
    if sp["method"] == "dspark" and sp["enabled"] and not sp["dspark"]["checkpoint_path"]:
        out.append("speculation.dspark.checkpoint_path: required when speculation.method is dspark")
    pl = sp["prompt_lookup"]
    if pl["min_ngram_size"] > pl["max_ngram_size"]:
        out.append("speculation.prompt_lookup: min_ngram_size exceeds max_ngram_size")
    if cfg["memory"]["nvme_tier"]["enabled"] and not cfg["hardware"]["nvme_paths"]:
        out.append("memory.nvme_tier.enabled: needs hardware.nvme_paths")
    if cfg["memory"]["kv_tiering"]["enabled"] and not m["index_topk"]:
        out.append("memory.kv_tiering.enabled: tiering is guided by the sparse-attention indexer; this model has none")
    if cfg["model"]["weights_format"] == "gguf" and not cfg["quantization"]["weights"].startswith("gguf"):
        out.append("quantization.weights: a GGUF checkpoint needs a gguf* weight format")
    return out


def validate(cfg: dict) -> None:
    problems = structural_problems(cfg)
    if not problems:
        problems = semantic_problems(cfg)
    if problems:
        raise ConfigError(problems)


def _nulls_to_defaults(node: dict, spec: dict) -> None:
    for k, s in spec.items():
        if isinstance(s, F):
            if node.get(k) is None and not s.nullable:
                node[k] = copy.deepcopy(s.default)
        elif isinstance(node.get(k), dict):
            _nulls_to_defaults(node[k], s)
        else:
            node[k] = defaults(s)


def load_config(source: str | dict | None = None, overrides: dict[str, Any] | None = None, check: bool = True) -> dict:
    """Return a fully-populated, validated config tree.

    ``source`` is a path to a JSON file, an already-parsed dict, or None (defaults only).
    ``overrides`` maps dotted paths to values and wins over everything else."""
    user: dict = {}
    if isinstance(source, str):
        with open(source) as fh:
            user = json.load(fh)
    elif isinstance(source, dict):
        user = copy.deepcopy(source)
    problems = structural_problems(user) if check else []
    if problems:
        raise ConfigError(problems)
    preset = user.get("preset", "balanced")
    for k, v in (overrides or {}).items():
        if k == "preset":
            preset = v
    if preset not in PRESET_OVERLAYS:
        raise ConfigError([f"preset: {preset!r} is not one of {sorted(PRESET_OVERLAYS)}"])
    cfg = deep_merge(defaults(), PRESET_OVERLAYS[preset])
    cfg = deep_merge(cfg, user)
    for k, v in (overrides or {}).items():
        set_path(cfg, k, v)
    cfg["preset"] = preset
    _nulls_to_defaults(cfg, SCHEMA)
    if check:
        validate(cfg)
    return cfg


def fill_model_from_checkpoint(cfg: dict) -> dict:
    """When ``model.weights_path`` points at (a file inside) a directory with a HuggingFace
    ``config.json``, fill the model dimensions the user left at 0 from it."""
    wp = cfg["model"]["weights_path"]
    if not wp:
        return cfg
    d = wp if os.path.isdir(wp) else os.path.dirname(wp)
    cj = os.path.join(d, "config.json")
    if not os.path.exists(cj):
        return cfg
    hf = json.load(open(cj))
    hf = hf.get("text_config", hf)
    m = cfg["model"]
    for k, v in hf.items():
        if k in m and isinstance(SCHEMA["model"].get(k), F) and m[k] in (0, None, [], ""):
            m[k] = v
    if not m.get("gating_score_fn") and hf.get("scoring_func"):
        m["gating_score_fn"] = hf["scoring_func"]
    return cfg


_LAYER_TYPE = {"linear_attention": "kda", "deepseek_sparse_attention": "mla", "full_attention": "mla", "mla": "mla", "kda": "kda"}


def model_config_from(cfg: dict) -> ModelConfig:
    """The engine's ModelConfig for the ``model`` + ``quantization`` sections."""
    m = cfg["model"]
    q = cfg["quantization"]
    n = m["num_hidden_layers"]
    if not n or not m["hidden_size"]:
        raise ConfigError(["model: num_hidden_layers / hidden_size are not set and no checkpoint config.json was found"])
    rs = m["rope_scaling"] or {}
    la = m["linear_attn_config"] or {}
    lt = [_LAYER_TYPE.get(t, "mla") for t in m["layer_types"]] or ["mla"] * n
    has_idx = m["architecture"] in ("glm_moe_dsa", "glm5_next") or (m["architecture"] == "deepseek_v3" and m["index_topk"] > 0
                                                                     and m["index_n_heads"] > 0 and get_path(cfg, "model.index_enabled", True))
    wq = q["weights"]
    expert_quant = {"fp8_e5m2": "fp8_e4m3"}.get(wq, wq)
    return ModelConfig(
        name=cfg["serving"].get("model_name") or m["architecture"], architecture=m["architecture"], hidden=m["hidden_size"],
        n_layers=n, vocab=m["vocab_size"], rms_eps=m["rms_norm_eps"], n_heads=m["num_attention_heads"],
        q_lora=m["q_lora_rank"] or 0, kv_lora=m["kv_lora_rank"], qk_nope=m["qk_nope_head_dim"],
        qk_rope=0 if m["mla_use_nope"] else m["qk_rope_head_dim"], v_head=m["v_head_dim"], rope_theta=float(m["rope_theta"]),
        rope_yarn_factor=float(rs.get("factor", 1.0)), rope_yarn_orig_max=int(rs.get("original_max_position_embeddings", 4096)),
        rope_yarn_beta_fast=float(rs.get("beta_fast", 32)), rope_yarn_beta_slow=float(rs.get("beta_slow", 1)),
        rope_yarn_mscale_all_dim=float(rs.get("mscale_all_dim", 0.0)), max_position=m["max_position_embeddings"] or 8192,
        dense_inter=m["intermediate_size"], first_k_dense=m["first_k_dense_replace"], n_routed=m["n_routed_experts"],
        top_k=m["num_experts_per_tok"], n_shared=m["n_shared_experts"], moe_inter=m["moe_intermediate_size"],
        scoring=m["gating_score_fn"], n_group=m["n_group"], topk_group=m["topk_group"], routed_scale=m["routed_scaling_factor"],
        norm_topk_prob=m["norm_topk_prob"], router_bias=True, swiglu_limit=float(m["swiglu_limit"]),
        index_n_heads=m["index_n_heads"] if has_idx else 0, index_head_dim=m["index_head_dim"], index_topk=m["index_topk"],
        index_topk_freq=max(1, m["index_topk_freq"]), index_kpool=m["index_kpool"],
        index_rope_dim=0 if m["mla_use_nope"] else m["qk_rope_head_dim"], layer_types=lt,
        kda_heads=la.get("num_heads", m["num_attention_heads"] if "kda" in lt else 0), kda_head_dim=la.get("head_dim", 128),
        kda_conv=la.get("short_conv_kernel_size", 4), kda_rank=la.get("gate_low_rank", 128),
        kda_lower_bound=la.get("gate_lower_bound", -5.0), hc_mult=m["hc_mult"], hc_eps=m["hc_eps"],
        hc_sinkhorn_iters=m["hc_sinkhorn_iters"], expert_quant=expert_quant,
        dense_quant="fp8_e4m3" if q["attention_compute"].startswith("fp8") and wq.startswith("fp8") else "bf16")


def model_section_from(mc: ModelConfig) -> dict:
    """Inverse of :func:`model_config_from` for the fields a ModelConfig carries (used by autoconfig probes)."""
    return {
        "architecture": mc.architecture, "num_hidden_layers": mc.n_layers, "hidden_size": mc.hidden,
        "num_attention_heads": mc.n_heads, "num_key_value_heads": mc.n_heads, "kv_lora_rank": mc.kv_lora,
        "qk_rope_head_dim": mc.qk_rope, "qk_nope_head_dim": mc.qk_nope, "v_head_dim": mc.v_head, "q_lora_rank": mc.q_lora,
        "intermediate_size": mc.dense_inter, "n_routed_experts": mc.n_routed, "n_shared_experts": mc.n_shared,
        "num_experts_per_tok": mc.top_k, "n_group": mc.n_group, "topk_group": mc.topk_group, "vocab_size": mc.vocab,
        "max_position_embeddings": mc.max_position, "rope_theta": mc.rope_theta, "rms_norm_eps": mc.rms_eps,
        "index_topk": mc.index_topk, "index_n_heads": mc.index_n_heads, "index_head_dim": mc.index_head_dim,
        "index_topk_freq": mc.index_topk_freq if mc.index_topk_freq > 1 else 0, "index_kpool": mc.index_kpool,
        "first_k_dense_replace": mc.first_k_dense, "routed_scaling_factor": mc.routed_scale,
        "moe_intermediate_size": mc.moe_inter, "norm_topk_prob": mc.norm_topk_prob, "gating_score_fn": mc.scoring,
        "swiglu_limit": mc.swiglu_limit, "hc_mult": mc.hc_mult, "hc_sinkhorn_iters": mc.hc_sinkhorn_iters, "hc_eps": mc.hc_eps,
        "layer_types": ["linear_attention" if t == "kda" else "deepseek_sparse_attention" for t in mc.layer_types]
        if "kda" in mc.layer_types else [],
        "mla_use_nope": mc.qk_rope == 0,
        "linear_attn_config": ({"num_heads": mc.kda_heads, "head_dim": mc.kda_head_dim, "short_conv_kernel_size": mc.kda_conv,
                                "gate_low_rank": mc.kda_rank, "gate_lower_bound": mc.kda_lower_bound} if mc.kda_heads else None),
    }


# Environment switches read once at first use.  Reference: LS_DETERMINISTIC, LS_REFERENCE_TRAJECTORY_IDENTITY,
# LAYERSTORM_DETERMINISTIC_EP_COMBINE(_PRECISION), LS_PERF_TRACE(_OUT) (README.md:126-127, RUN.md:13-24).
def apply_env(cfg: dict, env: dict[str, str] | None = None) -> dict:
    env = os.environ if env is None else env

    def on(name):
        return env.get(name, "") not in ("", "0", "false", "False")

    if on("LS_DETERMINISTIC"):
        cfg["compute"]["deterministic"] = True
        cfg["compute"]["deterministic_reduce"] = True
        cfg["compute"]["deterministic_ep_combine"] = True
    if on("LS_REFERENCE_TRAJECTORY_IDENTITY"):
        cfg["compute"]["reference_trajectory_identity"] = True
        cfg["compute"]["deterministic"] = True
    if "LAYERSTORM_DETERMINISTIC_EP_COMBINE" in env:
        cfg["compute"]["deterministic_ep_combine"] = on("LAYERSTORM_DETERMINISTIC_EP_COMBINE")
    p = env.get("LAYERSTORM_DETERMINISTIC_EP_COMBINE_PRECISION")
    if p in ("fp32", "bf16"):
        cfg["compute"]["deterministic_ep_combine_precision"] = p
    return cfg
