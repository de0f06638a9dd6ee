"""Declarative configuration schema: one JSON document with the sections
``preset, model, quantization, hardware, memory, orchestrator, prefetch, speculation, parallelism,
transfer, compute, serving, preprocessing, autoconfig, gpu_loader``.

The tree below is the single source of truth: defaults, types, enumerations and ranges.  Validation,
default filling, the list of live-changeable fields and the generated JSON-Schema all derive from it.
Reference surface: config/schema.json (same section and field names, so a reference config file loads
unchanged); values that only make sense on PCIe consumer boards keep their names but get B200 defaults
(64-token KV pages, tensor parallelism up to 8, NVLink peer transfers).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

ARCHITECTURES = ("deepseek_v3", "glm_moe_dsa", "kimi_k25", "deepseek_v4", "glm5_next")
WEIGHT_QUANTS = ("nvfp4", "fp8_e4m3", "fp8_e5m2", "int4_symmetric", "int4_asymmetric", "bf16", "gguf", "gguf_q2_k",
                 "gguf_q3_k", "gguf_q4_k", "gguf_q5_k", "gguf_q6_k", "gguf_q8_0", "gguf_mxfp4")
ATTENTION_BACKENDS = ("snapmla", "turboquant_mla", "csa_hca", "csa_hca_tq", "csa_hca_tq_mix")


@dataclass(frozen=True)
class F:
    """One leaf: python type(s), default, optional enumeration / inclusive range, live-changeable flag."""
    type: Any
    default: Any = None
    enum: tuple | None = None
    lo: float | None = None
    hi: float | None = None
    live: bool = False          # may be changed on a running engine (config update command)
    nullable: bool = False


def _auto_or(t):
    return (t, str)


SCHEMA: dict[str, Any] = {
    "preset": F(str, "balanced", enum=("balanced", "min_latency", "max_throughput", "")),
    "model": {
        "architecture": F(str, "glm5_next", enum=ARCHITECTURES),
        "weights_path": F(str, ""),
        "weights_format": F(str, "safetensors", enum=("safetensors", "gguf")),
        "use_mmap": F(bool, True),
        "num_hidden_layers": F(int, 0, lo=0),
        "hidden_size": F(int, 0, lo=0),
        "num_attention_heads": F(int, 0, lo=0),
        "num_key_value_heads": F(int, 0, lo=0),
        "kv_lora_rank": F(int, 512, lo=0),
        "qk_rope_head_dim": F(int, 64, lo=0),
        "qk_nope_head_dim": F(int, 128, lo=0),
        "v_head_dim": F(int, 128, lo=0),
        "q_lora_rank": F(int, 1536, lo=0),
        "intermediate_size": F(int, 0, lo=0),
        "n_routed_experts": F(int, 0, lo=0),
        "n_shared_experts": F(int, 1, lo=0),
        "num_experts_per_tok": F(int, 8, lo=0),
        "n_group": F(int, 8, lo=1),
        "topk_group": F(int, 4, lo=1),
        "vocab_size": F(int, 0, lo=0),
        "max_position_embeddings": F(int, 0, lo=0),
        "rope_theta": F(float, 10000.0),
        "rms_norm_eps": F(float, 1e-6),
        "num_nextn_predict_layers": F(int, 1, lo=0),
        "index_topk": F(int, 2048, lo=0),
        "index_n_heads": F(int, 64, lo=0),
        "index_head_dim": F(int, 128, lo=0),
        "index_topk_freq": F(int, 0, lo=0),
        "index_skip_topk_offset": F(int, 0, lo=0),
        "index_kpool": F(int, 1, lo=1),
        "index_kpool_compress": F(bool, False),
        "index_kpool_always_select_tail": F(bool, False),
        "rope_scaling": F(dict, None, nullable=True),
        "rope_interleave": F(bool, False),
        "indexer_rope_interleave": F(bool, False),
        "first_k_dense_replace": F(int, 3, lo=0),
        "routed_scaling_factor": F(float, 2.5),
        "moe_intermediate_size": F(int, 2048, lo=0),
        "moe_layer_freq": F(int, 1, lo=1),
        "norm_topk_prob": F(bool, True),
        "gating_score_fn": F(str, "sigmoid", enum=("sigmoid", "softmax", "sqrtsoftplus")),
        "head_dim": F(int, 0, lo=0),
        "compress_ratios": F(list, []),
        "compress_rope_theta": F(float, 0.0),
        "sliding_window": F(int, 0, lo=0),
        "swiglu_limit": F(float, 0.0),
        "num_hash_layers": F(int, 0, lo=0),
        "o_groups": F(int, 1, lo=1),
        "o_lora_rank": F(int, 0, lo=0),
        "hc_mult": F(int, 1, lo=1),
        "hc_sinkhorn_iters": F(int, 20, lo=0),
        "hc_eps": F(float, 1e-6),
        "layer_types": F(list, []),
        "linear_attn_config": F(dict, None, nullable=True),
        "mla_use_nope": F(bool, False),
        "vision": {
            "enabled": F(bool, False),
            "hidden_size": F(int, 1152), "num_layers": F(int, 27), "num_heads": F(int, 16),
            "patch_size": F(int, 14), "image_size": F(int, 384),
        },
    },
    "quantization": {
        "weights": F(str, "nvfp4", enum=WEIGHT_QUANTS),
        "gguf_strategy": F(str, "int", enum=("int", "dequant")),
        "attention_compute": F(str, "bf16", enum=("fp8_e4m3", "fp8_e5m2", "fp16", "bf16")),
        "kv_cache": F(str, "fp8_e4m3", enum=("fp8_e4m3", "fp8_e5m2", "fp16", "bf16", "turboquant4")),
        "gating_compute": F(str, "fp32", enum=("fp32", "fp16")),
    },
    "hardware": {
        "gpus": F(list, []),                      # [{id, type, vram_gb, numa_node, roles:[attention|resident|expert_streaming|draft], vram_budget_gb:{...}}]
        "cpu_expert_devices": F(list, []),
        "tp_array": F(list, None, nullable=True),
        "system_ram_gb": F(int, None, nullable=True),
        "nvme_paths": F(list, []),
        "nvme_capacity_gb": F(float, 0.0),
        "dcp_enabled": F(bool, True),
        "dcp_indexer_mode": F(str, "replicated", enum=("replicated", "local")),
        "dcp_kv_mode": F(str, "sharded", enum=("replicated", "sharded")),
    },
    "memory": {
        "pinned_layers": {
            "attention": F((str, list), "all"),
            "dense_ffn_layers": F(list, []),
            "embedding": F(bool, True),
            "output_head": F(bool, True),
            "gating": F((str, list), "all"),
        },
        "tp_mode_per_layer": {k: F(int, None, nullable=True) for k in
                              ("default_mode", "gating", "pinned_dense_ffn", "attention", "shared_expert", "embedding", "output_head")},
        "kv_cache": {
            "max_pages_per_gpu": F(_auto_or(int), "auto"),
            "page_size_tokens": F(int, 64, enum=(16, 32, 64, 128)),
            "speculation_pool_fraction": F(float, 0.15, lo=0.0, hi=0.9),
            "indexer_k_page_size_tokens": F(int, 8192, lo=16),
            "prefill_scratch_preallocated_gb": F(float, 0.5, lo=0.0),
            "streaming_spill_fraction": F(float, 0.34, lo=0.0, hi=1.0),
            "dcp_chunk_size": F(int, 64, lo=1),
            "naive_prefill_context_ceiling": F(int, None, nullable=True),
            "page_growth_chunk_tokens": F(int, 1024, lo=16),
            "_advanced": F(dict, {}),
        },
        "kv_tiering": {
            "enabled": F(bool, False),
            "hot_buffer_slots": F(int, 0, lo=0),
            "host_to_device_ratio": F(float, 8.0, lo=0.0),
            "replica_cold_dedup": F(bool, True),
            "tiered_prefill": F(bool, False),
            "admission_window_tokens": F(int, 0, lo=0),
        },
        "expert_cache": {
            "eviction_policy": F(str, "impact_weighted_lru", enum=("impact_weighted_lru", "lru", "lfu"), live=True),
            "eviction_alpha_recency": F(float, 0.4, live=True),
            "eviction_beta_frequency": F(float, 0.35, live=True),
            "eviction_gamma_routing_weight": F(float, 0.25, live=True),
            "eviction_delta_temporal_autocorr": F(float, 0.0, live=True),
            "eviction_epsilon_coactivation": F(float, 0.0, live=True),
            "eviction_zeta_prefetch_score": F(float, 0.0, live=True),
            "eviction_eta_hysteresis": F(float, 0.0, live=True),
            "hysteresis_enabled": F(bool, False),
            "hysteresis_stages": F(int, 5, lo=1),
            "hysteresis_up_threshold": F(int, 5),
            "hysteresis_down_threshold": F(int, 1),
            "duplication_frequency_threshold_percentile": F(int, 95, lo=0, hi=100),
            "temporal_autocorrelation_bonus": F(float, 0.8),
            "stable_zone_fraction": F(float, 0.7, lo=0.0, hi=1.0, live=True),
            "inclusive_cache": F(bool, True),
            "_advanced": F(dict, {}),
        },
        "nvme_tier": {
            "enabled": F(bool, False),
            "io_engine": F(str, "io_uring", enum=("io_uring", "libaio", "pread")),
            "queue_depth": F(int, 64, lo=1),
            "prefetch_ahead_layers": F(int, 3, lo=0),
            "host_ram_cache_gb": F(float, None, nullable=True),
            "direct_io": F(bool, True),
        },
        "numa": {
            "interleave_strategy": F(str, "affinity_based", enum=("affinity_based", "round_robin")),
            "fallback": F(str, "round_robin", enum=("round_robin", "sequential")),
        },
        "vram_safety_margin_gb": F(float, 1.0, lo=0.0),
        "host_packed_cache_mb": F(int, 0, lo=0),
        "preload_expert_buffers": F(bool, True),
        "pin_host_expert_pool": F(bool, True),
        "pin_host_expert_pool_sizing": {
            "mode": F(str, "fraction_total", enum=("fraction_free", "fraction_total", "absolute_gb")),
            "value": F(float, 0.9, lo=0.0),
            "per_node": F(list, []),
        },
        "pin_host_expert_pool_extra_scratch_bytes": F(int, 0, lo=0),
        "pin_host_expert_pool_preload": F(bool, True),
        "cross_node_spill": {
            "enabled": F(bool, True),
            "nodes": F(list, []),
            "sizing_mode": F(str, "fraction_total", enum=("fraction_free", "fraction_total", "absolute_gb")),
            "sizing_value": F(float, 0.9, lo=0.0),
            "per_node": F(list, []),
        },
        "pin_host_expert_pool_direct_load": F(bool, None, nullable=True),
        "pin_host_expert_pool_direct_o_direct": F(bool, True),
        "pin_host_expert_pool_iouring": F(bool, False),
        "pin_host_expert_pool_thp": F(bool, True),
        "arena_attach": {
            "enabled": F(bool, True),
            "socket_path": F(str, "@layerstorm-arena"),
            "holder_binary": F(str, ""),
            "auto_spawn": F(bool, True),
            "persist": F(bool, False),
            "on_conflict": F(str, "new", enum=("new", "fail", "kill")),
        },
        "arena_placement": {"freq_table": F(str, ""), "online": F(bool, True)},
    },
    "orchestrator": {
        "performance_objective": {"latency_weight": F(float, 0.6, lo=0, hi=1, live=True),
                                  "throughput_weight": F(float, 0.4, lo=0, hi=1, live=True)},
        "max_batch_size": F(int, 64, lo=1, live=True),
        "expert_batching": {"enabled": F(bool, True), "max_wait_us": F(int, 50, lo=0, live=True),
                            "min_batch_tokens_per_expert": F(int, 4, lo=1, live=True)},
        "coactivation_graph": {"enabled": F(bool, True), "decay_factor": F(float, 0.999, lo=0, hi=1),
                               "reoptimize_interval_seconds": F(int, 300, lo=1), "workload_shift_decay": F(float, 0.1)},
        "workload_detection": {"ewma_alpha": F(float, 0.01, lo=0, hi=1), "shift_threshold_std_devs": F(float, 3.0),
                               "_advanced": F(dict, {})},
        "ipc_transaction": {"writer_yield_interval": F(int, 16), "publish_interval_us": F(int, 5000),
                            "reader_max_retries": F(int, 200000000), "reader_backoff_stage_size": F(int, 4096),
                            "reader_stage0_yield_every": F(int, 64)},
        "prefill_chunk_tokens": F(int, 256, lo=1, live=True),
        "decode_expert_fetch_timeout_s": F(int, 5, lo=1),
    },
    "prefetch": {
        "prescope": {"enabled": F(bool, True), "lookahead_layers": F(int, 1, lo=0), "top_k": F(int, 8, lo=1),
                     "score_threshold": F(float, 0.01), "predictor_enabled": F(bool, False)},
        "probe": {"enabled": F(bool, True), "probe_points": F(list, []), "confidence_threshold": F(float, 0.6)},
        "moe_speq": {"enabled": F(bool, True), "predictor_hidden_size": F(int, 256), "learning_rate": F(float, 1e-4),
                     "training_buffer_size": F(int, 10000), "train_interval_steps": F(int, 100)},
        "speculative": {"enabled": F(bool, True), "max_prefetch_depth_layers": F(int, 3), "confidence_threshold": F(float, 0.4)},
        "fusion_weights": {"prescope_alpha": F(float, 0.5), "probe_beta": F(float, 0.3), "speq_gamma": F(float, 0.2),
                           "sp_moe_delta": F(float, 0.15)},
    },
    "speculation": {
        "enabled": F(bool, True),
        "method": F(str, "none", enum=("none", "null", "mtp", "prompt_lookup", "dspark", "self_speculative")),
        "mtp": {"enabled": F(bool, True), "max_depth": F(int, 3, lo=1, live=True), "dynamic_depth": F(bool, True),
                "confidence_threshold": F(float, 0.4, live=True), "batched_verify": F(bool, True)},
        "dspark": {
            "block_size": F(int, 8, lo=1), "speculative_tokens": F(int, 7, lo=1),
            "aux_hidden_state_layer_ids": F(list, []), "mask_token_id": F(int, 154856),
            "max_anchors": F(int, 1024), "draft_vocab_size": F(int, 154880),
            "checkpoint_path": F(str, ""), "draft_gpus": F(list, []),
            "draft_weights_quant": F(str, "bf16", enum=("bf16", "fp8_e4m3", "nvfp4")),
            "markov_rank": F(int, 256), "head_type": F(str, "markov", enum=("markov", "gated", "rnn")),
            "confidence_enabled": F(bool, False),
            "scheduler_mode": F(str, "off", enum=("off", "static_threshold", "throughput")),
            "confidence_threshold": F(float, 0.5), "sts_temperatures": F(list, []),
            "draft_context_capacity_tokens": F(int, 8192), "aux_capture_max_rows": F(int, 2048),
            "epm_dump_dir": F(str, ""), "verify_chunk_prefetch": F(bool, False), "ctx_rotate": F(bool, True),
        },
        "self_speculative": {"enabled": F(bool, True), "draft_expert_count": F(int, 1, lo=1),
                             "adaptive_exit_enabled": F(bool, True), "draft_confidence_threshold": F(float, 0.4),
                             "residual_correction": F(dict, {})},
        "prompt_lookup": {"enabled": F(bool, True), "min_ngram_size": F(int, 2, lo=1), "max_ngram_size": F(int, 4, lo=1),
                          "max_continuation_length": F(int, 5, lo=1)},
        "verification": {
            "moe_spec_max_loaded_experts_fraction": F(float, 0.8), "adaptive_topk_threshold": F(float, 0.92),
            "verification_quality_floor": F(float, 0.85),
            "in_flight_transfer_mode": F(str, "conservative", enum=("conservative", "optimistic")),
            "sparse_verification": F(bool, False),
            "ranking_strategy": F(str, "router_based", enum=("router_based", "static_calibration")),
            "substitution_policy": F(str, "substitution", enum=("substitution", "discard")),
            "_advanced": F(dict, {}),
        },
        "layer_skip_draft": {
            "enabled": F(bool, False), "method": F(str, "cosine_similarity", enum=("cosine_similarity", "clsap", "static_exit")),
            "threshold": F(float, 0.995), "min_acceptance_rate_to_enable": F(float, 0.5),
            "exit_layer": F(int, None, nullable=True), "target_skip_fraction": F(float, 0.5),
            "no_skip_first": F(int, 3), "no_skip_last": F(int, 3), "min_contiguous": F(int, 1),
            "product_window": F(int, 1), "product_threshold": F(float, 0.985), "_advanced": F(dict, {}),
        },
        "transfer_cancellation": {"cancel_abort_transfers": F(bool, True), "cancel_skip_transfers": F(bool, True),
                                  "cancel_stability_window": F(int, 2), "transfer_origin_expiry_cycles": F(int, 10000)},
        "reasoning_mode": {"enabled": F(bool, False), "think_token_detection": F(bool, True),
                           "aggressive_speculation_depth_multiplier": F(float, 2.0),
                           "relaxed_verification_threshold": F(float, 0.85)},
        "calibration": {"min_acceptance_rate": F(float, 0.3), "target_acceptance_rate": F(float, 0.6),
                        "adjustment_interval_tokens": F(int, 500), "acceptance_ema_alpha": F(float, 0.5),
                        "draft_count_ema_alpha": F(float, 0.9), "adjustment_step_size": F(float, 0.01),
                        "_advanced": F(dict, {})},
        "utility_scorer": {"enabled": F(bool, True), "strategy": F(str, "cascade", enum=("cascade", "ema", "fixed")),
                           "static_depth": F(int, 3), "utility_threshold": F(float, 1.0),
                           "vram_headroom_fraction": F(float, 0.1)},
        "draft_combiner": {"enabled": F(bool, True), "prompt_lookup_priority_boost": F(float, 1.0),
                           "mtp_compute_cost": F(float, 0.1), "self_spec_compute_cost": F(float, 0.5),
                           "dspark_compute_cost": F(float, 0.05)},
    },
    "parallelism": {
        "tensor_parallelism": F(int, 1, enum=(1, 2, 4, 8)),
        "expert_parallelism": F(int, 0, lo=0),       # 0 = all GPUs
        "expert_affinity": {"mode": F(str, "soft"), "initial_assignment": F(str, "round_robin", enum=("round_robin", "coactivation")),
                            "rebalance_interval_seconds": F(int, 300, lo=1)},
        "expert_duplication": {"enabled": F(bool, True), "max_duplicated_fraction": F(float, 0.05, lo=0, hi=1)},
        "node_routing": {"max_nodes_per_token": F(int, 4, lo=1)},
    },
    "transfer": {
        "fine_grained": {"enabled": F(bool, False), "max_in_flight_per_gpu": F(int, 4, lo=1),
                         "prefetch_distance_layers": F(int, 4, lo=0)},
        "streams_per_gpu": F(int, 2, lo=1),
        "priority_levels": F(int, 3, lo=1),
    },
    "compute": {
        "cuda_graphs": {"enabled": F(bool, True), "capture_attention": F(bool, True), "capture_gating": F(bool, True),
                        "capture_tp_allreduce": F(bool, True), "capture_expert_ffn": F(bool, True)},
        "gemm": {"backend": F(str, "tcgen05", enum=("tcgen05", "cutlass")), "grouped_gemm": F(bool, True),
                 "fused_swiglu": F(bool, True)},
        "attention_backend": F(str, "snapmla", enum=ATTENTION_BACKENDS),
        "prefill_superchunk_tokens": F(int, 0, lo=0),
        "prefill_moe_big": F(bool, True),
        "moe_big_chunk_tokens": F(int, 512, lo=1),
        "moe_big_fit_headroom_mb": F(int, 1024, lo=0),
        "moe_big_fit_headroom_expert_only_mb": F(int, 256, lo=0),
        "dsa_sparse_prefill": F(bool, False),
        "dsa_indexer_rewind": F(bool, True),
        "deterministic": F(bool, False),
        "reference_trajectory_identity": F(bool, False),
        "deterministic_reduce": F(bool, True),
        "deterministic_ep_combine": F(bool, True),
        "deterministic_ep_combine_precision": F(str, "fp32", enum=("fp32", "bf16")),
        "ipc_pin": F(bool, True),
    },
    "serving": {
        "host": F(str, "0.0.0.0"), "port": F(int, 8000, lo=1, hi=65535),
        "max_concurrent_requests": F(int, 32, lo=1), "max_queued_requests": F(int, 16, lo=0),
        "sse_heartbeat_seconds": F(float, 15, lo=0), "max_sequence_length": F(int, 32768, lo=1),
        "tokenizer_path": F(str, "auto"), "tool_call_parser": F(str, ""), "enable_auto_tool_choice": F(bool, False),
        "reasoning_parser": F(str, ""), "reasoning_config": F(str, ""), "tokenizer_mode": F(str, "auto"),
        "model_name": F(str, ""),
        "prefix_cache": {"enabled": F(bool, True), "max_cached_tokens": F(int, 131072, lo=0), "max_entries": F(int, 8, lo=0),
                         "kda_checkpoints": F(dict, {})},
    },
    "preprocessing": {
        "prepacked_dir": F(str, ""), "auto_preprocess": F(bool, False), "auto_preprocess_target": F(str, ""),
        "host_cache_mode": F(str, "mmap", enum=("mmap", "explicit_alloc")), "legacy_weights": F(bool, False),
        "live_prepack": F(bool, False), "live_prepack_threads": F(int, 0, lo=0),
    },
    "autoconfig": {
        "enabled": F(bool, False), "vram_expert_ratio": F(float, None, nullable=True, lo=0.0, hi=1.0),
        "total_active_context_tokens": F(int, None, nullable=True, lo=1),
        "output_path": F(str, ""), "fingerprint": F(str, ""),
        "prefer": F(str, "balanced", enum=("speed", "balanced", "capacity")),
        "accuracy": F(str, "standard", enum=("compact", "standard", "high", "superior")),
    },
    "gpu_loader": {
        "enabled": F(bool, False), "calibration_mode": F(str, "loaded", enum=("loaded", "quick", "full")),
        "calibration_path": F(str, ""),
    },
}


def defaults(node: Any = None) -> Any:
    """A fresh, fully-populated config tree of default values."""
    import copy
    node = SCHEMA if node is None else node
    if isinstance(node, F):
        return copy.deepcopy(node.default)
    return {k: defaults(v) for k, v in node.items()}


def leaf_paths(node: Any = None, prefix: str = ""):
    """Yield ``(dotted.path, F)`` for every leaf."""
    node = SCHEMA if node is None else node
    for k, v in node.items():
        p = f"{prefix}{k}"
        if isinstance(v, F):
            yield p, v
        else:
            yield from leaf_paths(v, p + ".")


def live_changeable_fields() -> list[str]:
    """Paths that a running engine accepts in a config-update command (reference: the generated
    changeable-field list, python/orchestrator/_gen_changeable_fields.py)."""
    return [p for p, f in leaf_paths() if f.live]


def json_schema(node: Any = None) -> dict:
    """The same tree as JSON-Schema (draft 2020-12), for editors and external validators."""
    node = SCHEMA if node is None else node
    if isinstance(node, F):
        names = {int: "integer", float: "number", str: "string", bool: "boolean", list: "array", dict: "object"}
        ts = node.type if isinstance(node.type, tuple) else (node.type,)
        t = [names[x] for x in ts] + (["null"] if node.nullable else [])
        if "number" in t and "integer" not in t:
            pass
        out: dict[str, Any] = {"type": t[0] if len(t) == 1 else t}
        if node.enum:
            out["enum"] = list(node.enum)
        if node.lo is not None:
            out["minimum"] = node.lo
        if node.hi is not None:
            out["maximum"] = node.hi
        if node.default is not None:
            out["default"] = node.default
        return out
    props = {k: json_schema(v) for k, v in node.items()}
    out = {"type": "object", "properties": props}
    if node is SCHEMA:
        out["$schema"] = "https://json-schema.org/draft/2020-12/schema"
        out["patternProperties"] = {"^_internal-": {}}
    else:
        out["additionalProperties"] = False
    return out


def markdown_reference() -> str:
    """One table row per leaf: path, type, default, constraints, whether it can change on a running engine."""
    rows = ["| field | type | default | constraints | live |", "|---|---|---|---|---|"]
    for path, f in leaf_paths():
        ts = f.type if isinstance(f.type, tuple) else (f.type,)
        cons = []
        if f.enum:
            cons.append("one of " + ", ".join(repr(e) for e in f.enum))
        if f.lo is not None:
            cons.append(f">= {f.lo}")
        if f.hi is not None:
            cons.append(f"<= {f.hi}")
        rows.append(f"| `{path}` | {' / '.join(t.__name__ for t in ts)}{' / null' if f.nullable else ''} | `{f.default!r}` | {'; '.join(cons)} | {'yes' if f.live else ''} |")
    return "\n".join(rows)


def main(argv=None) -> int:
    """``python -m layerstorm_b200.config --emit json-schema|defaults|live-fields|markdown``: everything that is GENERATED from the
    schema tree (the reference generates its parser, defaults and live-field list from ``config/schema.json`` with tools/gen_config.mjs;
    here the tree is interpreted at run time and these are its exports for editors, external validators and documentation).
    ``--check FILE`` validates a configuration document against the tree and exits 1 with the problems listed."""
    import argparse
    import json
    import sys
    ap = argparse.ArgumentParser(description="exports of the configuration schema")
    ap.add_argument("--emit", choices=["json-schema", "defaults", "live-fields", "markdown"], default=None)
    ap.add_argument("--check", default=None, metavar="FILE")
    a = ap.parse_args(argv)
    if a.check:
        from .loader import load_config
        try:
            load_config(a.check)
        except Exception as e:                       # the loader reports every problem of the document in its message
            print(f"{a.check}: {e}", file=sys.stderr)
            return 1
        print(f"{a.check}: ok")
        return 0
    if a.emit == "json-schema":
        print(json.dumps(json_schema(), indent=1))
    elif a.emit == "defaults":
        print(json.dumps(defaults(), indent=1))
    elif a.emit == "live-fields":
        print("\n".join(live_changeable_fields()))
    elif a.emit == "markdown":
        print(markdown_reference())
    else:
        ap.print_help()
    return 0

