"""Model identity from a bare weights path: what is it, what shape, how is it quantised, how big is it.

``probe(path)`` accepts a HuggingFace directory (``config.json`` + ``*.safetensors``), a ``.gguf`` file (first shard of a split
included), a prepacked directory (``manifest.json``) or the name of a built-in shape, and returns a ``ModelProbe``: the ``ModelConfig``,
the weights format, a quantisation summary (HF ``quantization_config`` or the histogram of ggml tensor types, with the type of the routed
experts singled out), bytes on disk, shard count and whether a tokenizer sits beside the weights.  Everything is read from headers and
metadata; no tensor data is touched, no GPU is needed.

``shape_from_gguf(reader)`` builds the ``ModelConfig`` from GGUF metadata alone (llama.cpp key names under the ``general.architecture``
prefix), so a GGUF file needs no ``config.json`` beside it.
Reference counterparts: python/autoconfig/modelprobe.py (identity from a bare path), gguf_meta.py (header-only GGUF reader) and
modelshape.py (shape ingestion).
"""
from __future__ import annotations

import glob
import json
import os
import re
from dataclasses import dataclass, field
from typing import Dict, Optional

from ..models.config import PRESETS, ModelConfig, from_hf_config, get_preset

# general.architecture -> architecture name of this framework
_GGUF_ARCH = {"deepseek2": "deepseek_v3", "deepseek3": "deepseek_v3", "deepseek_v3": "deepseek_v3", "deepseek3_2": "deepseek_v3",
              "glm_moe_dsa": "glm_moe_dsa", "glm-dsa": "glm_moe_dsa", "glm5_next": "glm5_next", "kimi_k25": "kimi_k25", "deepseek4": "deepseek_v4"}


@dataclass
class ModelProbe:
    kind: str                         # hf | gguf | prepacked | preset
    path: Optional[str]
    shape: Optional[ModelConfig]
    weights_format: str               # safetensors | gguf | prepacked | none
    quant: Dict[str, object] = field(default_factory=dict)
    bytes_on_disk: int = 0
    shards: int = 0
    has_tokenizer: bool = False
    notes: list = field(default_factory=list)

    def to_dict(self) -> dict:
        d = dict(self.__dict__)
        d["shape"] = self.shape.name if self.shape is not None else None
        return d


def shape_from_gguf(r) -> ModelConfig:
    """``r``: anything with ``meta(key, default)`` (``GgufReader`` / ``GgufSource``)."""
    ga = r.meta("general.architecture")
    if ga is None:
        raise ValueError("GGUF file has no general.architecture")
    m = lambda k, d=None: r.meta(f"{ga}.{k}", d)
    need = lambda k: _need(m(k), f"{ga}.{k}")
    n_layers, hidden, heads = int(need("block_count")), int(need("embedding_length")), int(need("attention.head_count"))
    rope = int(m("rope.dimension_count", 64))
    kv_lora = int(need("attention.kv_lora_rank"))
    # llama.cpp stores the absorbed (MQA) key width kv_lora + rope as key_length and the per-head widths as *_mla
    key_mla = m("attention.key_length_mla")
    key_len = int(m("attention.key_length", 0) or 0)
    qk_nope = int(key_mla) - rope if key_mla is not None else (key_len - rope if key_len and key_len != kv_lora + rope else 128)
    v_head = int(m("attention.value_length_mla", m("attention.value_length", 128)) or 128)
    if key_mla is None and v_head == kv_lora:
        v_head = 128                                                     # absorbed layout without the *_mla keys: per-head value width unknown
    gating = int(m("expert_gating_func", 1) or 1)
    vocab = m("vocab_size")
    if vocab is None:
        toks = r.meta("tokenizer.ggml.tokens")
        vocab = len(toks) if toks is not None else 0
    eos = r.meta("tokenizer.ggml.eos_token_id", 0)
    n_routed = int(m("expert_count", 0) or 0)
    return ModelConfig(
        name=str(r.meta("general.name", ga)), architecture=_GGUF_ARCH.get(ga, "deepseek_v3"), hidden=hidden, n_layers=n_layers, vocab=int(vocab),
        rms_eps=float(m("attention.layer_norm_rms_epsilon", 1e-6)), n_heads=heads, q_lora=int(m("attention.q_lora_rank", 0) or 0), kv_lora=kv_lora,
        qk_nope=qk_nope, qk_rope=rope, v_head=v_head, rope_theta=float(m("rope.freq_base", 10000.0)),
        rope_yarn_factor=float(m("rope.scaling.factor", 1.0) or 1.0), rope_yarn_orig_max=int(m("rope.scaling.original_context_length", 4096) or 4096),
        rope_yarn_mscale_all_dim=float(m("rope.scaling.yarn_log_multiplier", 0.0) or 0.0) * 10.0,
        max_position=int(m("context_length", 8192)), dense_inter=int(m("feed_forward_length", 0) or 0),
        first_k_dense=int(m("leading_dense_block_count", 0) or 0), n_routed=n_routed, top_k=int(m("expert_used_count", 0) or 0),
        n_shared=int(m("expert_shared_count", 0) or 0), moe_inter=int(m("expert_feed_forward_length", 0) or 0),
        scoring={1: "softmax", 2: "sigmoid"}.get(gating, "softmax"), n_group=int(m("expert_group_count", 1) or 1),
        topk_group=int(m("expert_group_used_count", 1) or 1), routed_scale=float(m("expert_weights_scale", 1.0) or 1.0),
        norm_topk_prob=bool(m("expert_weights_norm", True)), router_bias=gating == 2,
        index_n_heads=int(m("attention.indexer.head_count", 0) or 0), index_head_dim=int(m("attention.indexer.key_length", 128) or 128),
        index_topk=int(m("attention.indexer.top_k", 2048) or 2048), index_rope_dim=rope, layer_types=["mla"] * n_layers,
        eos_token_ids=[int(eos)] if not isinstance(eos, list) else [int(e) for e in eos])


def _need(v, key):
    if v is None:
        raise ValueError(f"GGUF metadata lacks {key}")
    return v


def _dir_bytes(pattern: str) -> tuple[int, int]:
    files = glob.glob(pattern)
    return sum(os.path.getsize(f) for f in files), len(files)


def _has_tokenizer(d: str) -> bool:
    return any(os.path.exists(os.path.join(d, f)) for f in ("tokenizer.json", "tokenizer.model", "tokenizer_config.json"))


def probe(path: str) -> ModelProbe:
    if path.lower() in PRESETS and not os.path.exists(path):
        return ModelProbe("preset", None, get_preset(path), "none", notes=["built-in shape: random weights only"])
    if not os.path.exists(path):
        raise FileNotFoundError(path)
    if path.endswith(".gguf"):
        return _probe_gguf(path)
    d = path if os.path.isdir(path) else os.path.dirname(path) or "."
    if os.path.exists(os.path.join(d, "manifest.json")) and not os.path.exists(os.path.join(d, "config.json")):
        man = json.load(open(os.path.join(d, "manifest.json")))
        nbytes, n = _dir_bytes(os.path.join(d, "L*", "*.bin"))
        quant = {k: man.get(k) for k in ("version", "quant", "hidden", "moe_inter", "stride")}
        return ModelProbe("prepacked", d, None, "prepacked", quant, nbytes, n, _has_tokenizer(d),
                          ["expert slot images only: the shape comes from the checkpoint they were packed from"])
    ggufs = sorted(glob.glob(os.path.join(d, "*.gguf")))
    cj = os.path.join(d, "config.json")
    if not os.path.exists(cj):
        if ggufs:
            return _probe_gguf(ggufs[0])
        raise ValueError(f"{d}: neither config.json, manifest.json nor a .gguf file")
    raw = json.load(open(cj))
    shape = from_hf_config(raw)
    nbytes, n = _dir_bytes(os.path.join(d, "*.safetensors"))
    qc = raw.get("quantization_config") or raw.get("text_config", {}).get("quantization_config") or {}
    quant: Dict[str, object] = {"method": qc.get("quant_method", "none")}
    if qc.get("quant_method") == "fp8":
        quant["block"] = qc.get("weight_block_size")
    hq = os.path.join(d, "hf_quant_config.json")
    if os.path.exists(hq):                                                 # ModelOpt export
        q = json.load(open(hq)).get("quantization", {})
        quant = {"method": "modelopt", "algo": q.get("quant_algo"), "kv": q.get("kv_cache_quant_algo")}
    notes = []
    if n == 0 and ggufs:
        p = _probe_gguf(ggufs[0])
        p.shape, p.notes = shape, p.notes + ["shape taken from the config.json beside the GGUF file"]
        return p
    if n == 0:
        notes.append("config.json without weights: shape only")
    return ModelProbe("hf", d, shape, "safetensors" if n else "none", quant, nbytes, n, _has_tokenizer(d), notes)


def _probe_gguf(path: str) -> ModelProbe:
    from ..formats.gguf import GGML_NAMES, GgufReader
    m = re.match(r"^(.*)-(\d{5})-of-(\d{5})\.gguf$", path)
    files = [f for f in (f"{m.group(1)}-{i:05d}-of-{m.group(3)}.gguf" for i in range(1, int(m.group(3)) + 1)) if os.path.exists(f)] if m else [path]
    hist: Dict[str, int] = {}
    expert_types: Dict[str, int] = {}
    shape, notes = None, []
    for i, f in enumerate(files):
        r = GgufReader(f)
        try:
            if i == 0:
                try:
                    shape = shape_from_gguf(r)
                except ValueError as e:
                    notes.append(str(e))
            for name, t in r.tensors.items():
                tn = GGML_NAMES.get(t["type"], f"type{t['type']}")
                hist[tn] = hist.get(tn, 0) + t["nbytes"]
                if "_exps" in name:
                    expert_types[tn] = expert_types.get(tn, 0) + t["nbytes"]
        finally:
            r.close()
    if m and len(files) != int(m.group(3)):
        notes.append(f"{int(m.group(3)) - len(files)} of {int(m.group(3))} shards are missing")
    quant = {"method": "gguf", "bytes_by_type": hist, "experts": max(expert_types, key=expert_types.get) if expert_types else None}
    d = os.path.dirname(path) or "."
    return ModelProbe("gguf", path, shape, "gguf", quant, sum(os.path.getsize(f) for f in files), len(files), _has_tokenizer(d), notes)
