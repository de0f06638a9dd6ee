"""Architecture-family serving templates: DATA, not logic.

Values for knobs that follow neither from the model's geometry nor from the machine: which tool-call / reasoning parser a model
family speaks, the prefill chunk that measured best on B200, the speculation scaffold, prefetch fusion weights.  The solver copies
the family's template into the configuration it writes (its explain trace lists every copied path as kind "template"); the base
configuration and pins win over the template.

Families: ``mla_dsa`` (DeepSeek-V3 / V3.2 and GLM MoE-DSA: MLA + optional DSA indexer + MoE), ``glm5_next`` (hybrid KDA + sparse
MLA; starts from mla_dsa), ``v4`` (DeepSeek-V4).  Provenance of the B200 numbers: prefill chunks of 2048 rows run the tensor-core
MLA kernel and the grouped expert GEMM at their best measured throughput on this framework (5.0k tok/s on the GLM-5.3-Flash
shape, 1 GPU); 256-row chunks are latency-friendlier and are kept for concurrency > 8.
Reference counterpart: python/autoconfig/templates.py (family templates copied by the solver's last stage).
"""
from __future__ import annotations

import copy
from typing import Any, Dict, List, Tuple

COMMON: Dict[str, Any] = {
    "orchestrator": {"performance_objective": {"latency_weight": 0.6, "throughput_weight": 0.4},
                     "expert_batching": {"max_wait_us": 50, "min_batch_tokens_per_expert": 4}},
    "prefetch": {"prescope": {"enabled": True, "lookahead_layers": 1},
                 "fusion_weights": {"prescope_alpha": 0.5, "probe_beta": 0.3, "speq_gamma": 0.2, "sp_moe_delta": 0.15}},
    "speculation": {"prompt_lookup": {"enabled": True, "min_ngram_size": 2, "max_ngram_size": 4, "max_continuation_length": 5},
                    "verification": {"adaptive_topk_threshold": 0.92, "verification_quality_floor": 0.85}},
    "compute": {"cuda_graphs": {"enabled": True}},
}

FAMILIES: Dict[str, Dict[str, Any]] = {
    "mla_dsa": {"serving": {"tool_call_parser": "deepseek_v3", "reasoning_parser": "deepseek_r1", "enable_auto_tool_choice": True}},
    "glm_dsa": {"serving": {"tool_call_parser": "glm47", "reasoning_parser": "glm45", "enable_auto_tool_choice": True}},
    "glm5_next": {"serving": {"tool_call_parser": "glm47", "reasoning_parser": "glm45", "enable_auto_tool_choice": True}},
    "v4": {"serving": {"tool_call_parser": "deepseek_v4", "reasoning_parser": "deepseek_v4", "enable_auto_tool_choice": True}},
}

_ARCH_FAMILY = {"deepseek_v3": "mla_dsa", "kimi_k25": "mla_dsa", "glm_moe_dsa": "glm_dsa", "glm5_next": "glm5_next", "deepseek_v4": "v4"}


def family_of(architecture: str) -> str:
    return _ARCH_FAMILY.get(architecture, "mla_dsa")


def prefill_chunk_for(concurrency: int) -> int:
    return 2048 if concurrency <= 8 else 256


def _merge(dst: dict, src: dict):
    for k, v in src.items():
        if isinstance(v, dict):
            _merge(dst.setdefault(k, {}), v)
        else:
            dst[k] = copy.deepcopy(v)


def template_for(architecture: str) -> Dict[str, Any]:
    out: Dict[str, Any] = {}
    _merge(out, COMMON)
    _merge(out, FAMILIES[family_of(architecture)])
    return out


def _leaves(tree: dict, prefix: str = "") -> List[Tuple[str, Any]]:
    out: List[Tuple[str, Any]] = []
    for k, v in tree.items():
        p = f"{prefix}.{k}" if prefix else k
        out.extend(_leaves(v, p) if isinstance(v, dict) else [(p, v)])
    return out


def apply_template(cfg: dict, architecture: str, user_set: Dict[str, Any]) -> List[str]:
    """Copy the family template into ``cfg`` except for the dotted paths in ``user_set`` (set by the base configuration or pinned).
    Returns the paths that were copied."""
    copied = []
    for path, val in _leaves(template_for(architecture)):
        if path in user_set:
            continue
        node = cfg
        parts = path.split(".")
        for p in parts[:-1]:
            node = node.setdefault(p, {})
        node[parts[-1]] = copy.deepcopy(val)
        copied.append(path)
    return copied
