"""Model shape descriptions for the MLA-family MoE architectures the engine runs.

One dataclass covers the five architecture names of the reference's config schema
(``config/schema.json`` -> ``model.architecture``: deepseek_v3, glm_moe_dsa, kimi_k25,
deepseek_v4, glm5_next) through feature switches: RoPE or NoPE MLA, DSA indexer (with
IndexShare / IndexPool), KDA linear-attention layers and mHC residual streams.  The
presets reproduce the dimensions of the reference's test-data model configs
(``test-data/{DeepSeek-V3.2,GLM-5.2,GLM-5.3-Flash}/config.json``), and
``from_hf_config`` reads the same HuggingFace ``config.json`` files.
Reference: src/model/model_config.h:19-204.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field, asdict
from typing import List, Optional

ARCHITECTURES = ("deepseek_v3", "glm_moe_dsa", "kimi_k25", "deepseek_v4", "glm5_next")


@dataclass
class ModelConfig:
    name: str = "tiny"
    architecture: str = "deepseek_v3"
    hidden: int = 256
    n_layers: int = 4
    vocab: int = 1024
    rms_eps: float = 1e-6
    # MLA
    n_heads: int = 8
    q_lora: int = 128
    kv_lora: int = 64
    qk_nope: int = 32
    qk_rope: int = 16
    v_head: int = 32
    rope_theta: float = 10000.0
    rope_yarn_factor: float = 1.0
    rope_yarn_orig_max: int = 4096
    rope_yarn_beta_fast: float = 32.0
    rope_yarn_beta_slow: float = 1.0
    rope_yarn_mscale_all_dim: float = 0.0
    max_position: int = 8192
    # FFN / MoE
    dense_inter: int = 512
    first_k_dense: int = 1
    n_routed: int = 16
    top_k: int = 4
    n_mtp: int = 0                      # multi-token-prediction blocks after the main stack (layer ids n_layers .. n_layers + n_mtp - 1)
    n_shared: int = 1
    num_hash_layers: int = 0            # MoE layers with index < this route by a token-id table (`moe.tid2eid`, DeepSeek-V4 hash layers) instead of top-k
    moe_inter: int = 128
    scoring: str = "softmax"          # sigmoid | softmax | sqrtsoftplus
    n_group: int = 1
    topk_group: int = 1
    routed_scale: float = 1.0
    norm_topk_prob: bool = True
    router_bias: bool = False         # e_score_correction_bias
    swiglu_limit: float = 0.0
    # DSA indexer (0 heads = dense attention)
    index_n_heads: int = 0
    index_head_dim: int = 128
    index_topk: int = 2048
    index_topk_freq: int = 1          # IndexShare: every freq-th sparse layer recomputes
    index_kpool: int = 1              # IndexPool: tokens per pooled indexer entry
    index_rope_dim: int = 0
    # layer types: "mla" | "kda"
    layer_types: List[str] = field(default_factory=list)
    # KDA
    kda_heads: int = 0
    kda_head_dim: int = 128
    kda_conv: int = 4
    kda_rank: int = 128
    kda_lower_bound: float = -5.0
    # mHC
    hc_mult: int = 1
    hc_eps: float = 1e-6
    hc_sinkhorn_iters: int = 20
    hc_post_mult: float = 2.0
    # weight formats for the synthetic / loaded checkpoint
    expert_quant: str = "bf16"        # bf16 | fp8_e4m3 | nvfp4 | gguf_q4_k ...
    dense_quant: str = "bf16"         # attention / dense FFN / shared expert
    eos_token_ids: List[int] = field(default_factory=list)

    def __post_init__(self):
        if not self.layer_types:
            self.layer_types = ["mla"] * self.n_layers
        assert len(self.layer_types) == self.n_layers
        assert self.architecture in ARCHITECTURES

    # ---- derived ----
    @property
    def qk_head(self) -> int:
        return self.qk_nope + self.qk_rope

    @property
    def has_indexer(self) -> bool:
        return self.index_n_heads > 0

    @property
    def mhc(self) -> bool:
        return self.hc_mult > 1

    def is_moe_layer(self, i: int) -> bool:
        return i >= self.first_k_dense and self.n_routed > 0

    def is_hash_layer(self, i: int) -> bool:
        """The layer's experts come from the token id (table row), not from a top-k over the router scores."""
        return self.is_moe_layer(i) and i < self.num_hash_layers

    def is_kda_layer(self, i: int) -> bool:
        return i < len(self.layer_types) and self.layer_types[i] == "kda"       # multi-token-prediction blocks (i >= n_layers) are MLA layers

    def mla_layers(self) -> List[int]:
        return [i for i in range(self.n_layers) if not self.is_kda_layer(i)]

    def index_source_layer(self, i: int) -> int:
        """Sparse layer whose indexer selection layer ``i`` uses (IndexShare)."""
        mla = self.mla_layers()
        j = mla.index(i)
        return mla[(j // self.index_topk_freq) * self.index_topk_freq]

    @property
    def softmax_scale(self) -> float:
        s = self.qk_head ** -0.5
        if self.rope_yarn_factor > 1.0 and self.rope_yarn_mscale_all_dim > 0:
            m = 0.1 * self.rope_yarn_mscale_all_dim * math.log(self.rope_yarn_factor) + 1.0
            s *= m * m
        return s

    def rope_inv_freq(self, dim: Optional[int] = None) -> List[float]:
        """Inverse frequencies for ``dim`` rotary dims, with the YaRN correction.
        Reference: src/compute/rope_table.cpp (YaRN ramp between beta_fast and beta_slow)."""
        d = dim if dim is not None else self.qk_rope
        if d <= 0:
            return []
        base = [self.rope_theta ** (-(2.0 * i) / d) for i in range(d // 2)]
        f = self.rope_yarn_factor
        if f <= 1.0:
            return base

        def corr_dim(rot):
            return d * math.log(self.rope_yarn_orig_max / (rot * 2 * math.pi)) / (2 * math.log(self.rope_theta))

        lo = max(math.floor(corr_dim(self.rope_yarn_beta_fast)), 0)
        hi = min(math.ceil(corr_dim(self.rope_yarn_beta_slow)), d - 1)
        if lo == hi:
            hi += 0.001
        out = []
        for i, fr in enumerate(base):
            ramp = min(max((i - lo) / (hi - lo), 0.0), 1.0)
            smooth = 1.0 - ramp
            out.append(fr / f * (1 - smooth) + fr * smooth)
        return out

    # ---- parameter counts (for sizing / autoconfig) ----
    def expert_params(self) -> int:
        return 3 * self.hidden * self.moe_inter

    def n_moe_layers(self) -> int:
        return sum(1 for i in range(self.n_layers) if self.is_moe_layer(i))

    def to_json(self) -> str:
        return json.dumps(asdict(self), indent=1)

    @classmethod
    def from_json(cls, s: str) -> "ModelConfig":
        return cls(**json.loads(s))


def tiny_mla_moe() -> ModelConfig:
    """The CPU-plumbing model: 4 layers (layer 0 dense FFN 512, layers 1-3 MoE), hidden 256,
    8 heads, q_lora 128, kv_lora 64, nope 32, rope 16, v 32, 16 experts top-4 softmax + 1 shared,
    expert FFN 128, vocab 1024."""
    return ModelConfig(name="tiny-mla-moe")


def tiny_glm5_next(n_layers: int = 4) -> ModelConfig:
    """A shrunken glm5_next (KDA + NoPE sparse MLA + mHC + IndexPool) for tests."""
    lt = ["mla" if (i % 4) == 3 else "kda" for i in range(n_layers)]
    return ModelConfig(
        name="tiny-glm5-next", architecture="glm5_next", hidden=256, n_layers=n_layers, vocab=1024, rms_eps=1e-5,
        n_heads=4, q_lora=128, kv_lora=64, qk_nope=64, qk_rope=0, v_head=64, dense_inter=512, first_k_dense=1,
        n_routed=16, top_k=4, n_shared=1, moe_inter=128, scoring="sigmoid", routed_scale=2.5, router_bias=True,
        swiglu_limit=10.0, index_n_heads=4, index_head_dim=128, index_topk=32, index_kpool=4, layer_types=lt,
        kda_heads=2, kda_head_dim=128, kda_rank=32, hc_mult=4)


def tiny_deepseek_v32(n_layers: int = 3) -> ModelConfig:
    """A shrunken DeepSeek-V3.2 shape (RoPE MLA + DSA indexer + grouped sigmoid routing)."""
    return ModelConfig(
        name="tiny-deepseek-v32", architecture="deepseek_v3", hidden=256, n_layers=n_layers, vocab=1024,
        n_heads=8, q_lora=128, kv_lora=64, qk_nope=32, qk_rope=16, v_head=32, dense_inter=512, first_k_dense=1,
        n_routed=32, top_k=4, n_shared=1, moe_inter=128, scoring="sigmoid", n_group=4, topk_group=2,
        routed_scale=2.5, router_bias=True, index_n_heads=4, index_topk=32, index_rope_dim=16,
        rope_yarn_factor=40.0, rope_yarn_mscale_all_dim=1.0)


def deepseek_v3_2() -> ModelConfig:
    return ModelConfig(
        name="DeepSeek-V3.2", architecture="deepseek_v3", hidden=7168, n_layers=61, vocab=129280, rms_eps=1e-6,
        n_heads=128, q_lora=1536, kv_lora=512, qk_nope=128, qk_rope=64, v_head=128, rope_theta=10000.0,
        rope_yarn_factor=40.0, rope_yarn_orig_max=4096, rope_yarn_mscale_all_dim=1.0, max_position=163840,
        dense_inter=18432, first_k_dense=3, n_routed=256, top_k=8, n_shared=1, moe_inter=2048, scoring="sigmoid",
        n_group=8, topk_group=4, routed_scale=2.5, router_bias=True, index_n_heads=64, index_head_dim=128,
        index_topk=2048, index_rope_dim=64, expert_quant="fp8_e4m3", dense_quant="fp8_e4m3", eos_token_ids=[1])


def glm_5_2() -> ModelConfig:
    return ModelConfig(
        name="GLM-5.2", architecture="glm_moe_dsa", hidden=6144, n_layers=78, vocab=154880, rms_eps=1e-5,
        n_heads=64, q_lora=2048, kv_lora=512, qk_nope=192, qk_rope=64, v_head=256, rope_theta=8000000.0,
        max_position=1048576, dense_inter=12288, first_k_dense=3, n_routed=256, top_k=8, n_shared=1, moe_inter=2048,
        scoring="sigmoid", routed_scale=2.5, router_bias=True, index_n_heads=32, index_head_dim=128, index_topk=2048,
        index_topk_freq=4, index_rope_dim=64, expert_quant="gguf_q4_k", dense_quant="bf16",
        eos_token_ids=[154820, 154827, 154829])


def glm_5_3_flash() -> ModelConfig:
    n = 45
    lt = ["mla" if (i % 4) == 3 else "kda" for i in range(n)]
    return ModelConfig(
        name="GLM-5.3-Flash", architecture="glm5_next", hidden=4096, n_layers=n, vocab=154880, rms_eps=1e-5,
        n_heads=64, q_lora=1536, kv_lora=512, qk_nope=256, qk_rope=0, v_head=256, max_position=1048576,
        dense_inter=12288, first_k_dense=3, n_routed=288, top_k=8, n_shared=1, moe_inter=2048, scoring="sigmoid",
        routed_scale=2.5, router_bias=True, swiglu_limit=10.0, index_n_heads=32, index_head_dim=128,
        index_topk=2048, index_kpool=4, layer_types=lt, kda_heads=64, kda_head_dim=128, kda_rank=128,
        kda_lower_bound=-5.0, hc_mult=4, hc_eps=1e-6, hc_sinkhorn_iters=20, expert_quant="nvfp4", dense_quant="bf16",
        eos_token_ids=[154820, 154827, 154829])


PRESETS = {
    "tiny-mla-moe": tiny_mla_moe,
    "tiny-glm5-next": tiny_glm5_next,
    "tiny-deepseek-v32": tiny_deepseek_v32,
    "deepseek-v3.2": deepseek_v3_2,
    "glm-5.2": glm_5_2,
    "glm-5.3-flash": glm_5_3_flash,
}


def get_preset(name: str) -> ModelConfig:
    return PRESETS[name.lower()]()


def from_hf_config(path_or_dict) -> ModelConfig:
    """Build a ModelConfig from a HuggingFace ``config.json`` (path or dict)."""
    c = json.load(open(path_or_dict)) if isinstance(path_or_dict, str) else dict(path_or_dict)
    c = c.get("text_config", c)
    mt = c.get("model_type", "")
    arch = {"deepseek_v3": "deepseek_v3", "deepseek_v32": "deepseek_v3", "glm_moe_dsa": "glm_moe_dsa",
            "glm5_next_text": "glm5_next", "glm5_next": "glm5_next", "kimi_k25": "kimi_k25",
            "deepseek_v4": "deepseek_v4"}.get(mt, "deepseek_v3")
    n = c["num_hidden_layers"]
    lt_raw = c.get("layer_types")
    lt = ["kda" if t == "linear_attention" else "mla" for t in lt_raw] if lt_raw else ["mla"] * n
    rs = c.get("rope_scaling") or {}
    rp = c.get("rope_parameters") or {}
    la = c.get("linear_attn_config") or {}
    return ModelConfig(
        name=mt or "hf", architecture=arch, hidden=c["hidden_size"], n_layers=n, vocab=c["vocab_size"],
        rms_eps=c.get("rms_norm_eps", 1e-6), n_heads=c["num_attention_heads"], q_lora=c.get("q_lora_rank") or 0,
        kv_lora=c["kv_lora_rank"], qk_nope=c["qk_nope_head_dim"], qk_rope=c.get("qk_rope_head_dim", 0),
        v_head=c["v_head_dim"], rope_theta=float(rp.get("rope_theta", c.get("rope_theta", 10000.0))),
        rope_yarn_factor=float(rs.get("factor", 1.0)), rope_yarn_orig_max=int(rs.get("original_max_position_embeddings", 4096)),
        rope_yarn_beta_fast=float(rs.get("beta_fast", 32)), rope_yarn_beta_slow=float(rs.get("beta_slow", 1)),
        rope_yarn_mscale_all_dim=float(rs.get("mscale_all_dim", 0.0)), max_position=c.get("max_position_embeddings", 8192),
        dense_inter=c["intermediate_size"], first_k_dense=c.get("first_k_dense_replace", 0),
        n_routed=c.get("n_routed_experts", 0), top_k=c.get("num_experts_per_tok", 0), n_shared=c.get("n_shared_experts", 0),
        n_mtp=int(c.get("num_nextn_predict_layers", 0) or 0), num_hash_layers=int(c.get("num_hash_layers", 0) or 0),
        moe_inter=c.get("moe_intermediate_size", 0), scoring=c.get("scoring_func", "softmax"), n_group=c.get("n_group", 1),
        topk_group=c.get("topk_group", 1), routed_scale=c.get("routed_scaling_factor", 1.0),
        norm_topk_prob=c.get("norm_topk_prob", True), router_bias=c.get("topk_method") == "noaux_tc",
        swiglu_limit=float(c.get("swiglu_limit", 0.0) or 0.0), index_n_heads=c.get("index_n_heads", 0),
        index_head_dim=c.get("index_head_dim", 128), index_topk=c.get("index_topk", 2048),
        index_topk_freq=c.get("index_topk_freq", 1) or 1, index_kpool=c.get("index_kpool", 1) or 1,
        index_rope_dim=c.get("qk_rope_head_dim", 0), layer_types=lt, kda_heads=la.get("num_heads", 0),
        kda_head_dim=la.get("head_dim", 128), kda_conv=la.get("short_conv_kernel_size", 4),
        kda_rank=la.get("gate_low_rank", la.get("head_dim", 128)), kda_lower_bound=la.get("gate_lower_bound", -5.0), hc_mult=c.get("hc_mult", 1) if c.get("mhc") else 1,
        hc_eps=c.get("hc_eps", 1e-6), hc_sinkhorn_iters=c.get("hc_sinkhorn_iters", 20),
        eos_token_ids=(c["eos_token_id"] if isinstance(c.get("eos_token_id"), list) else [c.get("eos_token_id", 0)]))
