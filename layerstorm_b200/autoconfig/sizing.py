"""Byte model of a deployment: what one GPU must hold for a given model, tensor-parallel degree,
KV format and context budget.  Pure arithmetic (no torch, no GPU), shared by the autoconfig solver,
the validator's VRAM-feasibility rule and the server's boot log.
Reference: the "K2 position-state sizing" step of docs/AUTOCONFIG_MODEL.md:395-499, which transcribes
src/core/vram_allocator.cpp; here the terms are re-derived from this engine's own layouts.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..models.config import ModelConfig

GiB = float(2**30)

# bits per weight including block scales
QUANT_BITS = {
    "bf16": 16.0, "fp16": 16.0, "fp8_e4m3": 8.0 + 32.0 / (128 * 128), "fp8_e5m2": 8.0 + 32.0 / (128 * 128),
    "nvfp4": 4.5, "int4_symmetric": 4.5, "int4_asymmetric": 5.0,
    "gguf": 4.5, "gguf_q2_k": 84 * 8 / 256, "gguf_q3_k": 110 * 8 / 256, "gguf_q4_k": 144 * 8 / 256, "gguf_q5_k": 176 * 8 / 256,
    "gguf_q6_k": 210 * 8 / 256, "gguf_q8_0": 34 * 8 / 32, "gguf_mxfp4": 17 * 8 / 32,
}

# attention backends in increasing accuracy; value = KV row format
ACCURACY_FLOOR = {"compact": 0, "standard": 1, "high": 1, "superior": 2}
MLA_LADDER = ("turboquant_mla", "snapmla", "bf16_mla")
V4_LADDER = ("csa_hca_tq", "csa_hca_tq_mix", "csa_hca")


def _align(x: int, a: int) -> int:
    return (x + a - 1) // a * a


def expert_slot_bytes(mc: ModelConfig, quant: str | None = None) -> int:
    """One routed expert (gate, up, down) in its cache slot, 4096-aligned."""
    q = quant or mc.expert_quant
    bits = QUANT_BITS.get(q, 16.0)
    return _align(int(3 * mc.hidden * mc.moe_inter * bits / 8) + 64, 4096)


def kv_row_bytes(mc: ModelConfig, backend: str = "snapmla") -> int:
    """Bytes of one token's latent KV row in one MLA layer."""
    dl, dr = mc.kv_lora, mc.qk_rope
    if backend in ("turboquant_mla", "csa_hca_tq"):
        return dl // 2 + 2 + 2 * dr            # 4-bit codes + bf16 norm + bf16 rope
    if backend in ("bf16_mla", "csa_hca"):
        return (dl + dr) * 2
    return dl + 16 + 2 * dr                    # fp8 latent + fp32 scale (16-byte slot) + bf16 rope


def indexer_row_bytes(mc: ModelConfig) -> float:
    """Bytes per token of the lightning-indexer key cache in one sparse layer (FP8 key + scale, pooled)."""
    if not mc.has_indexer:
        return 0.0
    return (mc.index_head_dim + 16) / max(1, mc.index_kpool)


def kv_bytes_per_token(mc: ModelConfig, backend: str = "snapmla", tp: int = 1, kv_mode: str = "sharded") -> float:
    """All MLA layers, one token, on one GPU.  Sharded mode keeps 1/tp of the rows per rank."""
    mla = mc.mla_layers()
    idx_layers = len({mc.index_source_layer(i) for i in mla}) if mc.has_indexer else 0
    per = len(mla) * kv_row_bytes(mc, backend) + idx_layers * indexer_row_bytes(mc)
    return per / tp if (kv_mode == "sharded" and tp > 1) else per


def recurrent_state_bytes_per_seq(mc: ModelConfig, tp: int = 1) -> int:
    """KDA state (fp32 [heads, 128, 128]) and conv history per sequence on one GPU (heads split over tp)."""
    n_kda = sum(1 for t in mc.layer_types if t == "kda")
    if not n_kda:
        return 0
    h = max(1, mc.kda_heads // tp)
    return n_kda * (h * mc.kda_head_dim * mc.kda_head_dim * 4 + 3 * h * mc.kda_head_dim * 3 * 4)


@dataclass
class ResidentBytes:
    attention: int = 0
    dense_ffn: int = 0
    shared_expert: int = 0
    router: int = 0
    embedding: int = 0
    head: int = 0
    norms: int = 0

    @property
    def total(self) -> int:
        return self.attention + self.dense_ffn + self.shared_expert + self.router + self.embedding + self.head + self.norms


def resident_bytes(mc: ModelConfig, tp: int = 1, n_gpus: int = 1, embed_on_host: bool = False) -> ResidentBytes:
    """Weights every GPU keeps regardless of the expert cache: its tensor-parallel shard of attention /
    KDA / dense FFN / LM head, the replicated router and norms, and the shared experts it owns."""
    db = QUANT_BITS.get(mc.dense_quant, 16.0) / 8
    H = mc.hidden
    r = ResidentBytes()
    n = mc.hc_mult
    for i in range(mc.n_layers):
        if mc.is_kda_layer(i):
            C = mc.kda_heads * mc.kda_head_dim
            sharded = 3 * C * H + C * H                                  # q, k, v in; o out (dense format)
            repl = 2 * mc.kda_rank * H + mc.kda_heads * H
            r.attention += int((sharded / tp + repl) * db)
            # always bf16: the low-rank gate tails and their [W | W] copies for the chunk-parallel path (3 x each); fp32: short
            # convolutions, dt bias, output norm, decay
            r.attention += int((2 * 3 * C * mc.kda_rank * 2 + 3 * C * mc.kda_conv * 4 + C * 4 + mc.kda_heads * 4) / tp) + mc.kda_head_dim * 4
        else:
            q_in = (mc.q_lora * H + mc.n_heads * mc.qk_head * mc.q_lora / tp) if mc.q_lora else mc.n_heads * mc.qk_head * H / tp
            kv_a = (mc.kv_lora + mc.qk_rope) * H
            o = H * mc.n_heads * mc.v_head / tp
            idx = 0
            extra = (mc.q_lora + mc.kv_lora) * 4                         # fp32 norms of the two latents
            if mc.has_indexer and mc.index_source_layer(i) == i:
                idx = mc.index_n_heads * mc.index_head_dim * (mc.q_lora or H) + (mc.index_head_dim + mc.index_n_heads) * H
                extra += 2 * mc.index_head_dim * 4                       # key LayerNorm weight and bias
                if mc.index_kpool > 1:
                    idx += mc.index_head_dim * H                         # pooling gate projection
                    extra += mc.index_kpool * mc.index_head_dim * 4      # pooled-position embedding
            r.attention += int((q_in + kv_a + o + idx + 8 * H) * db)     # (+ the fused input projection's rows padded to 8)
            r.attention += int(mc.n_heads * (mc.qk_nope + mc.v_head) * mc.kv_lora * 2 / tp) + extra      # W_UK / W_UV stay bf16
        if mc.is_moe_layer(i):
            r.router += mc.n_routed * H * 4 + mc.n_routed * 4
            r.shared_expert += int(mc.n_shared * expert_slot_bytes(mc) / n_gpus + 0.5)
        else:
            r.dense_ffn += int(3 * H * mc.dense_inter * db / tp)
        r.norms += 2 * H * 4
        if mc.mhc:
            # two hyper-connection passes per layer: mixing matrix [(2n + n^2), n H] fp32, its base vector and three scales
            r.norms += 2 * ((2 * n + n * n) * (n * H + 1) + 3) * 4
    r.norms += H * 4                                                     # output norm
    r.embedding = 0 if embed_on_host else mc.vocab * H * 2
    r.head = int(mc.vocab * H * 2 / tp)
    return r


def workspace_bytes(mc: ModelConfig, max_rows: int, max_ctx: int) -> int:
    """Activation scratch of one forward of ``max_rows`` tokens (prefill chunk / verify rows)."""
    H = mc.hidden
    per_row = H * 4 * (2 + 2 * mc.hc_mult) + mc.n_heads * (mc.qk_head + mc.kv_lora + mc.v_head) * 4 + mc.top_k * (2 * mc.moe_inter + H) * 4
    per_row += 3 * mc.kda_heads * mc.kda_head_dim * 4 + mc.dense_inter * 2 * 4
    score = mc.index_n_heads and max_ctx * 4 * min(max_rows, 256)
    return int(per_row * max_rows + score + (64 << 20))


@dataclass
class FitReport:
    ok: bool
    vram_budget: int
    resident: int
    workspace: int
    kv: int
    recurrent: int
    draft: int
    expert_slots_per_layer: int
    expert_slots_wanted: int
    host_expert_bytes: int
    binding: str = ""

    @property
    def vram_expert_ratio(self) -> float:
        return self.expert_slots_per_layer / max(1, self.expert_slots_wanted)


def fit(mc: ModelConfig, *, vram_gb: float, n_gpus: int, tp: int, backend: str, kv_mode: str, context_tokens: int,
        concurrency: int, max_rows: int, safety_gb: float = 1.0, draft_bytes: int = 0, embed_on_host: bool = False,
        min_slot_fraction: float = 0.0, expert_quant: str | None = None) -> FitReport:
    """Does one GPU hold its share?  Experts owned by a GPU = ceil(n_routed / n_gpus) per MoE layer; the
    slots that do not fit stay in pinned host memory and are streamed on demand."""
    budget = int((vram_gb - safety_gb) * GiB)
    res = resident_bytes(mc, tp, n_gpus, embed_on_host).total
    ws = workspace_bytes(mc, max_rows, max(1, context_tokens // max(1, concurrency)))
    kv = int(kv_bytes_per_token(mc, backend, tp, kv_mode) * context_tokens)
    rec = recurrent_state_bytes_per_seq(mc, tp) * (concurrency + 2)
    fixed = res + ws + kv + rec + draft_bytes
    n_moe = mc.n_moe_layers()
    owned = -(-mc.n_routed // n_gpus) if mc.n_routed else 0
    slot = expert_slot_bytes(mc, expert_quant)
    left = budget - fixed
    if n_moe == 0:
        return FitReport(left >= 0, budget, res, ws, kv, rec, draft_bytes, 0, 0, 0, "" if left >= 0 else "resident weights")
    slots = min(owned, max(0, left // (slot * n_moe)))
    need = max(mc.top_k + 1, int(min_slot_fraction * owned + 0.999))
    ok = left >= 0 and slots >= min(need, owned)
    binding = ""
    if not ok:
        parts = {"resident weights": res, "KV cache": kv, "recurrent state": rec, "workspace": ws, "draft model": draft_bytes}
        binding = max(parts, key=parts.get) if left < slot * n_moe * min(need, owned) else "expert cache"
    host = (owned - slots) * slot * n_moe
    return FitReport(ok, budget, res, ws, kv, rec, draft_bytes, int(slots), owned, int(host), binding)
