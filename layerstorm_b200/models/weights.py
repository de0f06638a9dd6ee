"""Random-init checkpoints in the engine's canonical tensor naming.

``init_weights`` produces an fp32 CPU state dict (small models, used by the oracle and by
the loaders' round-trip tests).  Large presets are initialised directly on the device in
their quantised storage format by ``layerstorm_b200.models.device_model`` because a
300B-parameter fp32 copy does not fit in host memory.

Tensor names (all ``[out, in]`` row-major like HuggingFace linear weights):

  embed.weight, head.weight, final_norm.weight
  layers.N.attn_norm.weight, layers.N.ffn_norm.weight
  layers.N.hc_attn.{fn,scale,base}, layers.N.hc_ffn.{fn,scale,base}          (mHC)
  layers.N.attn.{q_a,q_a_norm,q_b,kv_a,kv_a_norm,k_b,v_b,o}                  (MLA; k_b [H,dl,dn], v_b [H,dv,dl])
  layers.N.indexer.{wq_b,wk,k_norm.weight,k_norm.bias,weights_proj,gate,ape} (DSA / IndexPool)
  layers.N.kda.{q,k,v,beta,f_a,f_b,g_a,g_b,conv_q,conv_k,conv_v,a_log,dt_bias,o_norm,o}
  layers.N.mlp.{gate,up,down}                                                (dense FFN)
  layers.N.moe.{router,router_bias}, layers.N.moe.experts.E.{gate,up,down}, layers.N.moe.shared.S.{gate,up,down}

Reference naming map: src/model/weight_loader/tensor_id.h (HF + GGUF names -> canonical ids).
"""
from __future__ import annotations

from typing import Dict

import torch

from .config import ModelConfig


def init_weights(cfg: ModelConfig, seed: int = 0, std: float = 0.02) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)

    def mat(*shape, s=std):
        return torch.randn(*shape, generator=g, dtype=torch.float32) * s

    def norm(n):
        return 1.0 + 0.1 * torch.randn(n, generator=g, dtype=torch.float32)

    def uni(lo, hi, *shape):
        return lo + (hi - lo) * torch.rand(*shape, generator=g, dtype=torch.float32)

    H = cfg.hidden
    w: Dict[str, torch.Tensor] = {}
    w["embed.weight"] = mat(cfg.vocab, H, s=1.0)
    w["head.weight"] = mat(cfg.vocab, H)
    w["final_norm.weight"] = norm(H)
    n = cfg.hc_mult
    for i in range(cfg.n_layers):
        p = f"layers.{i}."
        w[p + "attn_norm.weight"] = norm(H)
        w[p + "ffn_norm.weight"] = norm(H)
        if cfg.mhc:
            for nm in ("hc_attn", "hc_ffn"):
                w[p + nm + ".fn"] = mat(2 * n + n * n, n * H, s=0.05)
                w[p + nm + ".scale"] = uni(0.5, 1.5, 3)
                w[p + nm + ".base"] = mat(2 * n + n * n, s=0.5)
        if cfg.is_kda_layer(i):
            C = cfg.kda_heads * cfg.kda_head_dim
            k = p + "kda."
            for nm in ("q", "k", "v"):
                w[k + nm] = mat(C, H, s=0.05)
                w[k + "conv_" + nm] = uni(-0.5, 0.5, C, cfg.kda_conv)
            w[k + "beta"] = mat(cfg.kda_heads, H, s=0.05)
            w[k + "f_a"] = mat(cfg.kda_rank, H, s=0.05)
            w[k + "f_b"] = mat(C, cfg.kda_rank, s=0.2)
            w[k + "g_a"] = mat(cfg.kda_rank, H, s=0.05)
            w[k + "g_b"] = mat(C, cfg.kda_rank, s=0.2)
            w[k + "a_log"] = uni(-1.0, 1.5, cfg.kda_heads)
            w[k + "dt_bias"] = uni(-1.0, 1.0, cfg.kda_heads, cfg.kda_head_dim)
            w[k + "o_norm"] = norm(cfg.kda_head_dim)
            w[k + "o"] = mat(H, C)
        else:
            a = p + "attn."
            Hh = cfg.n_heads
            w[a + "q_a"] = mat(cfg.q_lora, H, s=0.05)
            w[a + "q_a_norm"] = norm(cfg.q_lora)
            w[a + "q_b"] = mat(Hh * cfg.qk_head, cfg.q_lora, s=0.05)
            w[a + "kv_a"] = mat(cfg.kv_lora + cfg.qk_rope, H, s=0.05)
            w[a + "kv_a_norm"] = norm(cfg.kv_lora)
            w[a + "k_b"] = mat(Hh, cfg.kv_lora, cfg.qk_nope, s=0.05)
            w[a + "v_b"] = mat(Hh, cfg.v_head, cfg.kv_lora, s=0.05)
            w[a + "o"] = mat(H, Hh * cfg.v_head)
            if cfg.has_indexer and cfg.index_source_layer(i) == i:
                x = p + "indexer."
                w[x + "wq_b"] = mat(cfg.index_n_heads * cfg.index_head_dim, cfg.q_lora, s=0.05)
                w[x + "wk"] = mat(cfg.index_head_dim, H, s=0.05)
                w[x + "k_norm.weight"] = norm(cfg.index_head_dim)
                w[x + "k_norm.bias"] = mat(cfg.index_head_dim, s=0.1)
                w[x + "weights_proj"] = mat(cfg.index_n_heads, H, s=0.05)
                if cfg.index_kpool > 1:
                    w[x + "gate"] = mat(cfg.index_head_dim, H, s=0.05)
                    w[x + "ape"] = mat(cfg.index_kpool, cfg.index_head_dim, s=0.5)
        if cfg.is_moe_layer(i):
            m = p + "moe."
            w[m + "router"] = mat(cfg.n_routed, H, s=0.1)
            if cfg.router_bias:
                w[m + "router_bias"] = mat(cfg.n_routed, s=0.05)
            if cfg.is_hash_layer(i):
                # token id -> its top_k experts (distinct per row), int32 [vocab, top_k]
                w[m + "tid2eid"] = torch.stack([torch.randperm(cfg.n_routed, generator=g)[: cfg.top_k] for _ in range(cfg.vocab)]).int()
            for e in range(cfg.n_routed):
                w[m + f"experts.{e}.gate"] = mat(cfg.moe_inter, H)
                w[m + f"experts.{e}.up"] = mat(cfg.moe_inter, H)
                w[m + f"experts.{e}.down"] = mat(H, cfg.moe_inter)
            for s_ in range(cfg.n_shared):
                w[m + f"shared.{s_}.gate"] = mat(cfg.moe_inter, H)
                w[m + f"shared.{s_}.up"] = mat(cfg.moe_inter, H)
                w[m + f"shared.{s_}.down"] = mat(H, cfg.moe_inter)
        else:
            f = p + "mlp."
            w[f + "gate"] = mat(cfg.dense_inter, H)
            w[f + "up"] = mat(cfg.dense_inter, H)
            w[f + "down"] = mat(H, cfg.dense_inter)
    # multi-token-prediction blocks: an MLA + FFN decoder layer each (dense attention), plus the input norms / projection and output norm
    for k in range(cfg.n_mtp):
        L = cfg.n_layers + k
        p = f"layers.{L}."
        a = p + "attn."
        Hh = cfg.n_heads
        w[p + "attn_norm.weight"] = norm(H)
        w[p + "ffn_norm.weight"] = norm(H)
        w[a + "q_a"] = mat(cfg.q_lora, H, s=0.05)
        w[a + "q_a_norm"] = norm(cfg.q_lora)
        w[a + "q_b"] = mat(Hh * cfg.qk_head, cfg.q_lora, s=0.05)
        w[a + "kv_a"] = mat(cfg.kv_lora + cfg.qk_rope, H, s=0.05)
        w[a + "kv_a_norm"] = norm(cfg.kv_lora)
        w[a + "k_b"] = mat(Hh, cfg.kv_lora, cfg.qk_nope, s=0.05)
        w[a + "v_b"] = mat(Hh, cfg.v_head, cfg.kv_lora, s=0.05)
        w[a + "o"] = mat(H, Hh * cfg.v_head)
        if cfg.is_moe_layer(L):
            m = p + "moe."
            w[m + "router"] = mat(cfg.n_routed, H, s=0.1)
            if cfg.router_bias:
                w[m + "router_bias"] = mat(cfg.n_routed, s=0.05)
            if cfg.is_hash_layer(L):
                # token id -> its top_k experts (distinct per row), int32 [vocab, top_k]
                w[m + "tid2eid"] = torch.stack([torch.randperm(cfg.n_routed, generator=g)[: cfg.top_k] for _ in range(cfg.vocab)]).int()
            for e in range(cfg.n_routed):
                w[m + f"experts.{e}.gate"] = mat(cfg.moe_inter, H)
                w[m + f"experts.{e}.up"] = mat(cfg.moe_inter, H)
                w[m + f"experts.{e}.down"] = mat(H, cfg.moe_inter)
            for s_ in range(cfg.n_shared):
                w[m + f"shared.{s_}.gate"] = mat(cfg.moe_inter, H)
                w[m + f"shared.{s_}.up"] = mat(cfg.moe_inter, H)
                w[m + f"shared.{s_}.down"] = mat(H, cfg.moe_inter)
        else:
            f = p + "mlp."
            w[f + "gate"] = mat(cfg.dense_inter, H)
            w[f + "up"] = mat(cfg.dense_inter, H)
            w[f + "down"] = mat(H, cfg.dense_inter)
        w[p + "mtp.enorm"] = norm(H)
        w[p + "mtp.hnorm"] = norm(H)
        w[p + "mtp.eh_proj"] = mat(H, 2 * H, s=0.05)
        w[p + "mtp.final_norm"] = norm(H)
    return w


def round_weights_bf16(w: Dict[str, torch.Tensor], keep_fp32=("router", "hc_", "norm", "a_log", "dt_bias", "conv_", "ape", "bias")) -> Dict[str, torch.Tensor]:
    """Round the matrices that the engine stores in bf16 through bf16, so the oracle and the
    engine start from identical values."""
    out = {}
    for k, v in w.items():
        if any(t in k for t in keep_fp32) or not v.is_floating_point():
            out[k] = v.clone()
        else:
            out[k] = v.to(torch.bfloat16).to(torch.float32)
    return out
