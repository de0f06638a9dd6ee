"""DSpark block draft: a small dense transformer proposes a whole block of tokens in ONE non-causal pass over features of the target.

What the draft is (speculators-format ``dspark`` checkpoint: ``config.json`` + ``model.safetensors``):
  * context features - for every committed position the target's hidden states at ``aux_hidden_state_layer_ids`` (the stream that
    ENTERS each of those layers; hyper-connection targets: the mean over the residual streams) are concatenated, fused by ``fc``
    ([H, N_aux * H]) and normalised (``hidden_norm``); every draft layer projects them to keys (``k_proj`` -> per-head RMSNorm -> rotary
    at the absolute position) and values (``v_proj``) ONCE, when the position is committed - the draft never re-reads the context;
  * one block pass - rows ``[anchor token, mask, mask, ...]`` at positions ``anchor_pos, anchor_pos + 1, ...`` go through ``L`` dense
    layers (per-head q / k RMSNorm, rotary in the half-split pairing, full multi-head attention over ALL context positions and ALL
    rows of the block - no causal mask -, SwiGLU MLP), then ``norm`` and ``lm_head``: row k >= 1 sits AT the position it predicts;
  * a first-order Markov head corrects each row's logits by a rank-r bias that depends on the token actually chosen for the row
    before it (``markov_w2 @ markov_w1[x_{k-1}]``, the anchor for the first row), a short serial chain over the block;
  * an optional confidence head gives a trained survival probability per row (sigmoid of a linear map of [hidden ; markov feature]),
    whose running product cuts the block where the draft stops believing itself.
The target verifies the block in one step; whatever the draft proposes, the committed tokens are the target's (lossless).

B200 shape of the problem: the draft is ~7.6 GB of bf16 weights and a block pass reads all of them once for 8 rows, so a pass is one
weight sweep (~1 ms at HBM speed) against gamma target steps it can save; context keys and values cost 2 * L * kv_dim * 2 bytes per
position (80 KB with the shipped geometry), so a 180 GB GPU keeps a million-token context of the DRAFT next to the target without a
sliding window - the window (``ctx_rotate``) is there for configurations that cap ``draft_context_capacity_tokens``.

Everything here is tensor code on whatever device the tensors live on (plain library GEMMs: the draft is dense and small); the CPU
runs the same code in fp32, which is what the tests compare against a separately written per-head reference.

Reference: src/speculation/dspark_runtime.cpp (context ingest, block forward, Markov / confidence heads, window rotation),
src/model/weight_loader/dspark_loader.h (checkpoint layout and its fail-closed validation), src/compute/kernels/dspark/*.h.
"""
from __future__ import annotations

import contextlib
import dataclasses
import json
import math
import os
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from .model_draft import ConfidenceHead, MarkovHead


# ------------------------------------------------------------------------------------------------------------- checkpoint
@dataclasses.dataclass
class DsparkCheckpointConfig:
    block_size: int = 8                      # rows of one block pass: the anchor row + block_size - 1 predicting rows
    speculative_tokens: int = 7
    markov_rank: int = 256
    markov_head_type: str = "vanilla"
    enable_confidence_head: bool = False
    confidence_head_with_markov: bool = False
    draft_vocab_size: int = 0
    mask_token_id: int = -1
    max_anchors: int = 1024
    aux_hidden_state_layer_ids: List[int] = dataclasses.field(default_factory=list)
    tie_word_embeddings: bool = False
    # the dense backbone
    num_hidden_layers: int = 5
    hidden_size: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    intermediate_size: int = 0
    rms_norm_eps: float = 1e-5
    rope_theta: float = 8e6
    vocab_size: int = 0

    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def n_aux(self) -> int:
        return len(self.aux_hidden_state_layer_ids)

    @classmethod
    def from_json(cls, j: dict) -> "DsparkCheckpointConfig":
        if j.get("speculators_model_type") != "dspark":
            raise ValueError(f"not a dspark speculator checkpoint (speculators_model_type = {j.get('speculators_model_type')!r})")
        t = j["transformer_layer_config"]
        theta = (t.get("rope_parameters") or {}).get("rope_theta", t.get("rope_theta", 0.0))
        pm = (j.get("speculators_config") or {}).get("proposal_methods") or [{}]
        c = cls(block_size=int(j["block_size"]), speculative_tokens=int(pm[0].get("speculative_tokens", int(j["block_size"]) - 1)),
                markov_rank=int(j["markov_rank"]), markov_head_type=str(j["markov_head_type"]),
                enable_confidence_head=bool(j["enable_confidence_head"]), confidence_head_with_markov=bool(j["confidence_head_with_markov"]),
                draft_vocab_size=int(j["draft_vocab_size"]), mask_token_id=int(j["mask_token_id"]), max_anchors=int(j.get("max_anchors", 1024)),
                aux_hidden_state_layer_ids=[int(x) for x in j["aux_hidden_state_layer_ids"]], tie_word_embeddings=bool(j.get("tie_word_embeddings", False)),
                num_hidden_layers=int(t["num_hidden_layers"]), hidden_size=int(t["hidden_size"]), num_attention_heads=int(t["num_attention_heads"]),
                num_key_value_heads=int(t["num_key_value_heads"]), head_dim=int(t["head_dim"]), intermediate_size=int(t["intermediate_size"]),
                rms_norm_eps=float(t["rms_norm_eps"]), rope_theta=float(theta), vocab_size=int(t["vocab_size"]))
        c.check()
        return c

    def to_json(self) -> dict:
        return {"speculators_model_type": "dspark", "block_size": self.block_size, "markov_rank": self.markov_rank, "markov_head_type": self.markov_head_type,
                "enable_confidence_head": self.enable_confidence_head, "confidence_head_with_markov": self.confidence_head_with_markov,
                "draft_vocab_size": self.draft_vocab_size, "mask_token_id": self.mask_token_id, "max_anchors": self.max_anchors,
                "aux_hidden_state_layer_ids": list(self.aux_hidden_state_layer_ids), "tie_word_embeddings": self.tie_word_embeddings,
                "speculators_config": {"proposal_methods": [{"speculative_tokens": self.speculative_tokens}]},
                "transformer_layer_config": {"model_type": "qwen3", "num_hidden_layers": self.num_hidden_layers, "hidden_size": self.hidden_size,
                                             "num_attention_heads": self.num_attention_heads, "num_key_value_heads": self.num_key_value_heads,
                                             "head_dim": self.head_dim, "intermediate_size": self.intermediate_size, "rms_norm_eps": self.rms_norm_eps,
                                             "rope_parameters": {"rope_theta": self.rope_theta}, "vocab_size": self.vocab_size}}

    def check(self):
        bad = []
        if self.markov_head_type != "vanilla":
            bad.append(f"markov_head_type {self.markov_head_type!r}: only the vanilla low-rank head is built")
        if self.head_dim <= 0 or self.head_dim % 2 or self.head_dim > 256:
            bad.append(f"head_dim {self.head_dim}")
        if self.num_key_value_heads <= 0 or self.num_attention_heads % max(1, self.num_key_value_heads):
            bad.append("num_attention_heads must be a multiple of num_key_value_heads")
        if not self.aux_hidden_state_layer_ids:
            bad.append("aux_hidden_state_layer_ids is empty")
        if not 0 <= self.mask_token_id < self.vocab_size:
            bad.append(f"mask_token_id {self.mask_token_id} outside the vocabulary")
        if not 0 < self.draft_vocab_size <= self.vocab_size:
            bad.append(f"draft_vocab_size {self.draft_vocab_size} against vocab_size {self.vocab_size}")
        if not 1 <= self.speculative_tokens < max(2, self.block_size + 1) or self.speculative_tokens + 1 > self.block_size:
            bad.append(f"speculative_tokens {self.speculative_tokens} needs block_size >= {self.speculative_tokens + 1}, have {self.block_size}")
        if self.rope_theta <= 0:
            bad.append("rope_theta missing")
        if bad:
            raise ValueError("dspark checkpoint configuration: " + "; ".join(bad))

    def expected_tensors(self) -> Dict[str, Tuple[int, ...]]:
        """Every tensor the checkpoint must hold, with its shape - nothing more, nothing less."""
        H, V, Vd, r, I = self.hidden_size, self.vocab_size, self.draft_vocab_size, self.markov_rank, self.intermediate_size
        t: Dict[str, Tuple[int, ...]] = {"embed_tokens.weight": (V, H), "fc.weight": (H, self.n_aux * H), "hidden_norm.weight": (H,), "norm.weight": (H,),
                                         "markov_head.markov_w1.weight": (V, r), "markov_head.markov_w2.weight": (Vd, r)}
        if not self.tie_word_embeddings:
            t["lm_head.weight"] = (Vd, H)
        if Vd < V:
            t["d2t"] = (Vd,)
        if self.enable_confidence_head:
            t["confidence_head.proj.weight"] = (1, H + (r if self.confidence_head_with_markov else 0))
            t["confidence_head.proj.bias"] = (1,)
        for l in range(self.num_hidden_layers):
            p = f"layers.{l}."
            t.update({p + "self_attn.q_proj.weight": (self.q_dim, H), p + "self_attn.k_proj.weight": (self.kv_dim, H), p + "self_attn.v_proj.weight": (self.kv_dim, H),
                      p + "self_attn.o_proj.weight": (H, self.q_dim), p + "self_attn.q_norm.weight": (self.head_dim,), p + "self_attn.k_norm.weight": (self.head_dim,),
                      p + "input_layernorm.weight": (H,), p + "post_attention_layernorm.weight": (H,),
                      p + "mlp.gate_proj.weight": (I, H), p + "mlp.up_proj.weight": (I, H), p + "mlp.down_proj.weight": (H, I)})
        return t

    def weight_bytes(self, bytes_per_element: int = 2) -> int:
        n = 0
        for shape in self.expected_tensors().values():
            n += math.prod(shape)
        return n * bytes_per_element

    def context_bytes_per_token(self, bytes_per_element: int = 2) -> int:
        return 2 * self.num_hidden_layers * self.kv_dim * bytes_per_element


def draft_memory_bytes(cfg: DsparkCheckpointConfig, weights_quant: str = "bf16", context_tokens: int = 8192, contexts: int = 4) -> Dict[str, int]:
    """What the block draft takes on its GPU: the matrices in their storage format (embedding, norms and the Markov / confidence heads
    stay bf16), and keys + values of ``contexts`` draft contexts of ``context_tokens`` positions.  The auto-configurator's draft term."""
    per = {"bf16": 2.0, "fp8_e4m3": 1.0 + 4.0 / (128 * 128), "nvfp4": 0.5 + 1.0 / 16}[weights_quant]
    mats = small = 0
    for k, shape in cfg.expected_tensors().items():
        n = math.prod(shape)
        if k.endswith("proj.weight") and "confidence" not in k or k in ("fc.weight", "lm_head.weight"):
            mats += n
        elif k != "d2t":
            small += n
    w = int(mats * per + small * 2 + (8 * cfg.draft_vocab_size if cfg.draft_vocab_size < cfg.vocab_size else 0))
    ctx = cfg.context_bytes_per_token() * int(context_tokens) * int(contexts)
    return {"weights": w, "contexts": ctx, "total": w + ctx}


def validate_tensors(cfg: DsparkCheckpointConfig, tensors: Dict[str, torch.Tensor]):
    """Fail closed: an unknown, missing, mis-shaped or wrongly typed tensor stops the load (a draft that silently runs on a partly
    matched checkpoint proposes garbage that the target then pays to reject)."""
    want = cfg.expected_tensors()
    bad = [f"unexpected tensor {k}" for k in tensors if k not in want]
    for k, shape in want.items():
        if k not in tensors:
            bad.append(f"missing tensor {k}")
        elif tuple(tensors[k].shape) != shape:
            bad.append(f"{k}: shape {tuple(tensors[k].shape)}, expected {shape}")
        elif k == "d2t":
            if tensors[k].dtype not in (torch.int64, torch.int32):
                bad.append(f"d2t: dtype {tensors[k].dtype}, expected an integer type")
        elif not tensors[k].is_floating_point():
            bad.append(f"{k}: dtype {tensors[k].dtype}")
    if "d2t" in tensors and not bad:
        tgt = torch.arange(cfg.draft_vocab_size, dtype=torch.int64) + tensors["d2t"].to(torch.int64).cpu()
        if int(tgt.min()) < 0 or int(tgt.max()) >= cfg.vocab_size:
            bad.append("d2t maps a draft id outside the target vocabulary")
    if bad:
        raise ValueError("dspark checkpoint: " + "; ".join(bad[:12]) + (f"; ... {len(bad) - 12} more" if len(bad) > 12 else ""))


def is_dspark_checkpoint(path: str) -> bool:
    cj = os.path.join(path, "config.json") if os.path.isdir(path) else ""
    if not cj or not os.path.exists(cj):
        return False
    try:
        return json.load(open(cj)).get("speculators_model_type") == "dspark"
    except (OSError, ValueError):
        return False


def load_dspark_checkpoint(path: str) -> Tuple[DsparkCheckpointConfig, Dict[str, torch.Tensor]]:
    from ..formats.safetensors import SafetensorsReader
    cfg = DsparkCheckpointConfig.from_json(json.load(open(os.path.join(path, "config.json"))))
    rd = SafetensorsReader(os.path.join(path, "model.safetensors"))
    try:
        tensors = {k: rd.get(k).clone() for k in rd.keys()}
    finally:
        rd.close()
    validate_tensors(cfg, tensors)
    return cfg, tensors


def write_dspark_checkpoint(path: str, cfg: DsparkCheckpointConfig, tensors: Dict[str, torch.Tensor]):
    from ..formats.safetensors import write_safetensors
    os.makedirs(path, exist_ok=True)
    json.dump(cfg.to_json(), open(os.path.join(path, "config.json"), "w"), indent=1)
    write_safetensors(os.path.join(path, "model.safetensors"), {k: v.contiguous() for k, v in tensors.items()}, {"format": "pt"})


def random_dspark_tensors(cfg: DsparkCheckpointConfig, seed: int = 0, dtype: torch.dtype = torch.bfloat16, device="cpu") -> Dict[str, torch.Tensor]:
    """Random draft weights of the checkpoint's shapes (``device``: made there, matrix by matrix - a full-size draft never exists on
    the host)."""
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed)
    out: Dict[str, torch.Tensor] = {}
    for k, shape in cfg.expected_tensors().items():
        if k == "d2t":
            # an increasing subset of the target vocabulary, stored as offsets: target id = draft id + d2t[draft id]
            tgt = torch.sort(torch.randperm(cfg.vocab_size, generator=g, device=dev)[: cfg.draft_vocab_size]).values
            out[k] = (tgt - torch.arange(cfg.draft_vocab_size, device=dev)).to(torch.int64)
        elif k.endswith("norm.weight") or k.endswith("layernorm.weight"):
            out[k] = (1.0 + 0.1 * torch.randn(shape, generator=g, device=dev)).to(dtype)
        elif k.endswith(".bias"):
            out[k] = torch.zeros(shape, dtype=dtype, device=dev)
        else:
            fan_in = shape[-1]
            out[k] = (torch.randn(shape, generator=g, device=dev) * (0.5 if "embed" in k or "markov_w1" in k else 1.0 / math.sqrt(fan_in))).to(dtype)
    return out


def draft_config_for_target(hidden: int, vocab: int, n_target_layers: int, layers: int = 2, heads: int = 0, head_dim: int = 64, inter: int = 0,
                            block_size: int = 8, markov_rank: int = 64, n_aux: int = 3, draft_vocab: int = 0, confidence: bool = True,
                            mask_token_id: Optional[int] = None) -> DsparkCheckpointConfig:
    """A draft geometry for a target of the given width (random-weight runs and tests): aux layers spread evenly over the target."""
    heads = heads or max(1, hidden // head_dim)
    ids = sorted({max(1, min(n_target_layers - 1, round((j + 1) * n_target_layers / (n_aux + 1)))) for j in range(n_aux)})
    c = DsparkCheckpointConfig(block_size=block_size, speculative_tokens=block_size - 1, markov_rank=markov_rank, enable_confidence_head=confidence,
                               confidence_head_with_markov=confidence, draft_vocab_size=draft_vocab or vocab,
                               mask_token_id=vocab - 1 if mask_token_id is None else mask_token_id, aux_hidden_state_layer_ids=ids,
                               num_hidden_layers=layers, hidden_size=hidden, num_attention_heads=heads, num_key_value_heads=heads, head_dim=head_dim,
                               intermediate_size=inter or 2 * hidden, vocab_size=vocab)
    c.check()
    return c


# ------------------------------------------------------------------------------------------------------------- the backbone
def _rms(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


def _rope_half_split(x: torch.Tensor, pos: torch.Tensor, theta: float) -> torch.Tensor:
    """Rotary embedding over [rows, heads, head_dim]: element i pairs with i + head_dim / 2, angle = pos * theta^(-2 i / head_dim);
    the angles are made in fp32 from the position itself (no table, so a position of a million costs nothing)."""
    half = x.shape[-1] // 2
    inv = torch.exp(torch.arange(half, dtype=torch.float32, device=x.device) * (-2.0 * math.log(theta) / x.shape[-1]))
    ang = pos.to(torch.float32)[:, None] * inv[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    xf = x.float()
    a, b = xf[..., :half], xf[..., half:]
    return torch.cat([a * c - b * s, b * c + a * s], -1).to(x.dtype)


class _Linear:
    """y = x @ W^T for the draft's matrices.  ``kernels`` = None: a library GEMM on the tensor as it is (the CPU, fp32 comparisons).
    ``kernels`` = "bf16" | "fp8_e4m3" | "nvfp4": the weights are stored in that format and applied by the framework's own kernels
    (``models/device_model.py`` ``QLinear``: weight-streaming kernels for the few rows of a block pass, tcgen05 GEMMs with the
    de-quantisation in the operand pipeline for the many rows of a context ingest) - ``speculation.dspark.draft_weights_quant``."""

    def __init__(self, w: torch.Tensor, device, dtype, kernels: Optional[str]):
        self.N, self.K = w.shape
        self.q = None
        if kernels is None:
            self.w = w.to(device, dtype)
        else:
            from ..models.device_model import QLinear
            self.q = QLinear.from_float(w.float(), kernels, device)

    def __call__(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        if self.q is None:
            y = x @ self.w.T
            return y if out_dtype is None else y.to(out_dtype)
        M = x.shape[0]
        want = out_dtype or x.dtype
        out = torch.empty(M, self.N, dtype=torch.bfloat16 if want == torch.bfloat16 else torch.float32, device=x.device)
        self.q(out, x.to(torch.bfloat16).contiguous(), M)
        return out if out.dtype == want else out.to(want)

    def dense(self) -> torch.Tensor:
        """The matrix in effect, as fp32 (de-quantised)."""
        return (self.w if self.q is None else self.q.dequant()).float()

    def nbytes(self) -> int:
        return self.w.numel() * self.w.element_size() if self.q is None else self.q.nbytes()


class DsparkContext:
    """Keys and values of one sequence's committed positions, per draft layer: a window [base, base + capacity) of absolute
    positions; ``length`` = positions [0, length) have been seen (those below ``base`` have left the window)."""

    def __init__(self, layers: int, capacity: int, kv_heads: int, head_dim: int, device, dtype):
        self.k = torch.zeros(layers, capacity, kv_heads, head_dim, device=device, dtype=dtype)
        self.v = torch.zeros_like(self.k)
        self.capacity = capacity
        self.base = 0
        self.length = 0
        self.rotations = 0
        self.valid = True
        self.tokens: List[int] = []          # the committed tokens behind ``length`` (prefix matching by the draft source)

    def reset(self):
        self.base = self.length = 0
        self.valid = True
        self.tokens = []

    def rewind(self, length: int):
        """Forget the positions from ``length`` on (a rejected suffix, a fork point): later ingests overwrite them in place."""
        if length < self.base:
            self.reset()                      # everything still held lies behind the fork point
            return
        self.length = min(self.length, length)
        del self.tokens[self.length:]


class DsparkBackbone:
    def __init__(self, cfg: DsparkCheckpointConfig, tensors: Dict[str, torch.Tensor], device="cpu", dtype: Optional[torch.dtype] = None,
                 ctx_capacity: int = 8192, rotate: bool = True, kernels: Optional[str] = None):
        """``kernels``: None = library GEMMs over the tensors in ``dtype``; "bf16" / "fp8_e4m3" / "nvfp4" = the draft's matrices are
        stored in that format on the GPU and applied by the framework's own kernels (see ``_Linear``)."""
        validate_tensors(cfg, tensors)
        self.cfg = cfg
        self.device = torch.device(device)
        self.dtype = dtype or (torch.float32 if self.device.type == "cpu" else torch.bfloat16)
        self.ctx_capacity = int(ctx_capacity)
        self.rotate = rotate
        if self.ctx_capacity < 2 * cfg.block_size:
            raise ValueError(f"draft context capacity {ctx_capacity} is smaller than two blocks")
        if kernels is not None and self.device.type != "cuda":
            raise ValueError("the framework's GEMM kernels run on the GPU; on the CPU leave ``kernels`` unset")
        self.kernels = kernels
        if kernels is not None:
            self.dtype = torch.bfloat16                                     # the kernels take bf16 activations
        mv = lambda k: tensors[k].to(self.device, self.dtype)             # noqa: E731
        lin = lambda w: _Linear(w, self.device, self.dtype, kernels)     # noqa: E731
        self.embed = mv("embed_tokens.weight")
        self.lm_head = lin(tensors["embed_tokens.weight"][: cfg.draft_vocab_size] if cfg.tie_word_embeddings else tensors["lm_head.weight"])
        self.fc, self.hidden_norm, self.norm = lin(tensors["fc.weight"]), mv("hidden_norm.weight"), mv("norm.weight")
        self.layers = []
        for l in range(cfg.num_hidden_layers):
            p = f"layers.{l}."
            a, m = p + "self_attn.", p + "mlp."
            # k and v of the context are projected together (one GEMM over the fused features), gate and up of the MLP likewise
            self.layers.append({"q": lin(tensors[a + "q_proj.weight"]), "kv": lin(torch.cat([tensors[a + "k_proj.weight"], tensors[a + "v_proj.weight"]], 0)),
                                "o": lin(tensors[a + "o_proj.weight"]),
                                "q_norm": mv(a + "q_norm.weight"), "k_norm": mv(a + "k_norm.weight"), "in_norm": mv(p + "input_layernorm.weight"),
                                "post_norm": mv(p + "post_attention_layernorm.weight"),
                                "gate_up": lin(torch.cat([tensors[m + "gate_proj.weight"], tensors[m + "up_proj.weight"]], 0)), "down": lin(tensors[m + "down_proj.weight"])})
        d2t = tensors.get("d2t")
        self.markov = MarkovHead(mv("markov_head.markov_w1.weight"), mv("markov_head.markov_w2.weight"), None, d2t.to(self.device) if d2t is not None else None)
        self.confidence = None
        if cfg.enable_confidence_head:
            self.confidence = ConfidenceHead(mv("confidence_head.proj.weight")[0], float(tensors["confidence_head.proj.bias"].float()[0]))
        self.block_passes = 0
        self.ingested_rows = 0
        self.collect_layers = False      # keep the residual stream after every layer of the last block pass (corpus recording)
        self.last_layer_hidden: Optional[torch.Tensor] = None     # [rows, layers, hidden]

    def effective_tensors(self) -> Dict[str, torch.Tensor]:
        """The checkpoint tensors as this backbone applies them (fp32, on the CPU): identical to what was loaded for library GEMMs,
        the de-quantised values for quantised kernels - what a reference run has to use to be comparable."""
        c = self.cfg
        f = lambda t: t.float().cpu()                                     # noqa: E731
        out = {"embed_tokens.weight": f(self.embed), "fc.weight": f(self.fc.dense()), "hidden_norm.weight": f(self.hidden_norm), "norm.weight": f(self.norm),
               "markov_head.markov_w1.weight": f(self.markov.w1), "markov_head.markov_w2.weight": f(self.markov.w2)}
        if not c.tie_word_embeddings:
            out["lm_head.weight"] = f(self.lm_head.dense())
        if self.markov.d2t is not None:
            out["d2t"] = self.markov.d2t.cpu()
        if self.confidence is not None:
            out["confidence_head.proj.weight"] = f(self.confidence.w)[None, :]
            out["confidence_head.proj.bias"] = torch.tensor([self.confidence.b])
        for l, L in enumerate(self.layers):
            p = f"layers.{l}."
            kv, gu = f(L["kv"].dense()), f(L["gate_up"].dense())
            out.update({p + "self_attn.q_proj.weight": f(L["q"].dense()), p + "self_attn.k_proj.weight": kv[: c.kv_dim], p + "self_attn.v_proj.weight": kv[c.kv_dim:],
                        p + "self_attn.o_proj.weight": f(L["o"].dense()), p + "self_attn.q_norm.weight": f(L["q_norm"]), p + "self_attn.k_norm.weight": f(L["k_norm"]),
                        p + "input_layernorm.weight": f(L["in_norm"]), p + "post_attention_layernorm.weight": f(L["post_norm"]),
                        p + "mlp.gate_proj.weight": gu[: c.intermediate_size], p + "mlp.up_proj.weight": gu[c.intermediate_size:], p + "mlp.down_proj.weight": f(L["down"].dense())})
        return out

    def weight_bytes(self) -> int:
        n = self.embed.numel() * self.embed.element_size() + self.fc.nbytes() + (0 if self.cfg.tie_word_embeddings and self.kernels is None else self.lm_head.nbytes())
        return n + sum(L[k].nbytes() for L in self.layers for k in ("q", "kv", "o", "gate_up", "down"))

    # ---------------------------------------------------------------- context
    def new_context(self) -> DsparkContext:
        c = self.cfg
        return DsparkContext(c.num_hidden_layers, self.ctx_capacity, c.num_key_value_heads, c.head_dim, self.device, self.dtype)

    def _make_room(self, ctx: DsparkContext, start: int, rows: int) -> bool:
        """The window must hold [start, start + rows): when it would overflow, the oldest positions leave - the newest surviving rows
        move to the front and the base follows, so that half the capacity (at least the incoming rows) is in use afterwards."""
        end = start + rows
        if end - ctx.base <= ctx.capacity:
            return True
        if not self.rotate or rows > ctx.capacity:
            ctx.valid = False
            return False
        keep = max(ctx.capacity // 2, rows)
        new_base = end - keep
        n = start - new_base                                              # surviving rows that are already in the window
        if n > 0:
            s = new_base - ctx.base
            ctx.k[:, :n] = ctx.k[:, s: s + n].clone()
            ctx.v[:, :n] = ctx.v[:, s: s + n].clone()
        ctx.base = new_base
        ctx.rotations += 1
        return True

    @torch.no_grad()
    def ingest(self, ctx: DsparkContext, aux: torch.Tensor, start_pos: int, tokens: Optional[Sequence[int]] = None) -> bool:
        """Commit positions [start_pos, start_pos + rows): ``aux`` [rows, N_aux * H] = the target's hidden states at the aux layers,
        concatenated in the order of ``aux_hidden_state_layer_ids``.  ``start_pos`` may lie at or below the context's length (the
        rows overwrite a rejected suffix) but not beyond it (a gap ends drafting for the sequence).  False: the context is invalid."""
        c = self.cfg
        rows = aux.shape[0]
        if not ctx.valid or rows == 0:
            return ctx.valid
        if aux.shape[1] != c.n_aux * c.hidden_size:
            raise ValueError(f"aux rows have {aux.shape[1]} features, the checkpoint fuses {c.n_aux} x {c.hidden_size}")
        if start_pos > ctx.length or start_pos < ctx.base:
            ctx.valid = False
            return False
        if not self._make_room(ctx, start_pos, rows):
            return False
        feat = _rms(self.fc(aux.to(self.device, self.dtype)), self.hidden_norm, c.rms_norm_eps)
        pos = torch.arange(start_pos, start_pos + rows, device=self.device)
        lo = start_pos - ctx.base
        for l, L in enumerate(self.layers):
            kv = L["kv"](feat)
            k = kv[:, : c.kv_dim].view(rows, c.num_key_value_heads, c.head_dim)
            ctx.k[l, lo: lo + rows] = _rope_half_split(_rms(k, L["k_norm"], c.rms_norm_eps), pos, c.rope_theta)
            ctx.v[l, lo: lo + rows] = kv[:, c.kv_dim:].view(rows, c.num_key_value_heads, c.head_dim)
        ctx.length = start_pos + rows
        del ctx.tokens[start_pos:]
        if tokens is not None and len(ctx.tokens) == start_pos:
            ctx.tokens.extend(int(t) for t in tokens)
        self.ingested_rows += rows
        return True

    # ---------------------------------------------------------------- one block
    @torch.no_grad()
    def run_block(self, ctx: DsparkContext, anchor_token: int, anchor_pos: int, n_draft: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """One non-causal pass: (fp32 logits [n_draft + 1, V_draft], normalised hidden rows [n_draft + 1, H]); row 0 belongs to the
        anchor and predicts nothing, row k >= 1 predicts the token at position anchor_pos + k."""
        c = self.cfg
        nq = n_draft + 1
        if nq > c.block_size:
            raise ValueError(f"{nq} rows exceed the checkpoint's block size {c.block_size}")
        if not ctx.valid or anchor_pos > ctx.length or anchor_pos < ctx.base:
            raise RuntimeError(f"no context for an anchor at position {anchor_pos} (window [{ctx.base}, {ctx.length}), valid {ctx.valid})")
        if not 0 <= anchor_token < c.vocab_size:
            raise ValueError("anchor token outside the vocabulary")
        ids = torch.tensor([anchor_token] + [c.mask_token_id] * n_draft, device=self.device)
        pos = torch.arange(anchor_pos, anchor_pos + nq, device=self.device)
        x = self.embed[ids]
        n_ctx = anchor_pos - ctx.base
        rep = c.num_attention_heads // c.num_key_value_heads
        scale = 1.0 / math.sqrt(c.head_dim)
        per_layer: List[torch.Tensor] = []
        for l, L in enumerate(self.layers):
            h = _rms(x, L["in_norm"], c.rms_norm_eps)
            q = _rope_half_split(_rms(L["q"](h).view(nq, c.num_attention_heads, c.head_dim), L["q_norm"], c.rms_norm_eps), pos, c.rope_theta)
            kv = L["kv"](h)
            k = _rope_half_split(_rms(kv[:, : c.kv_dim].view(nq, c.num_key_value_heads, c.head_dim), L["k_norm"], c.rms_norm_eps), pos, c.rope_theta)
            v = kv[:, c.kv_dim:].view(nq, c.num_key_value_heads, c.head_dim)
            keys = torch.cat([ctx.k[l, :n_ctx], k], 0)                      # every context position, then every row of the block
            vals = torch.cat([ctx.v[l, :n_ctx], v], 0)
            if rep > 1:
                keys, vals = keys.repeat_interleave(rep, 1), vals.repeat_interleave(rep, 1)
            att = torch.softmax(torch.einsum("qhd,khd->hqk", q.float(), keys.float()) * scale, -1)
            o = torch.einsum("hqk,khd->qhd", att, vals.float()).reshape(nq, c.q_dim).to(self.dtype)
            x = x + L["o"](o)
            h = _rms(x, L["post_norm"], c.rms_norm_eps)
            gu = L["gate_up"](h)
            x = x + L["down"]((torch.nn.functional.silu(gu[:, : c.intermediate_size].float()) * gu[:, c.intermediate_size:].float()).to(self.dtype))
            if self.collect_layers:
                per_layer.append(x)
        hidden = _rms(x, self.norm, c.rms_norm_eps)
        self.block_passes += 1
        self.last_layer_hidden = torch.stack(per_layer, 1) if per_layer else None
        return self.lm_head(hidden, torch.float32), hidden

    @torch.no_grad()
    def draft(self, ctx: DsparkContext, anchor_token: int, anchor_pos: int, n_draft: int, confidence_threshold: float = 0.0) -> Tuple[List[int], List[float]]:
        """Block pass + Markov chain (+ confidence cut): target-vocabulary ids and, with a confidence head, the per-row survival."""
        logits, hidden = self.run_block(ctx, anchor_token, anchor_pos, n_draft)
        ids, feats = self.markov.chain(logits[1:], anchor_token)
        conf: List[float] = []
        if self.confidence is not None:
            f = feats if self.cfg.confidence_head_with_markov else feats[:, :0]
            cv = self.confidence.survival(hidden[1:], f)
            conf = [float(x) for x in cv]
            if confidence_threshold > 0:
                ids = ids[: ConfidenceHead.cut(cv, confidence_threshold)]
        return ids, conf


# ------------------------------------------------------------------------------------------------------------- how much of a block to verify
class DsparkScheduler:
    """Decides, per round, how many of the block's tokens go to the target (``speculation.dspark.scheduler_mode``):
      ``off``               all of them;
      ``static_threshold``  the longest prefix whose cumulative survival stays at or above ``confidence_threshold``;
      ``throughput``        the prefix that maximises expected committed tokens per unit of verify cost:
                            (1 + sum_{j<=k} a_j) / (1 + row_cost * k), a_j = survival of position j, row_cost = what one more verify
                            row costs relative to a one-row step (decode steps on this GPU are bound by the weight sweep, so a row is
                            a few per cent of a step; the block pass is already paid when the choice is made).
    Survival of position j = product of the confidence head's conditional probabilities c_1 .. c_j, each first temperature-scaled
    on the logit (``sts_temperatures``, fitted offline by ``verify_plan.fit_sts_temperatures`` on the trace kept here); without a
    confidence head (or with it switched off) the running acceptance rate p stands in: a_j = p^j.
    Reference: python/orchestrator/dspark_draft.py (survival confidences, STS temperatures, acceptance EMA, confidence trace)."""

    def __init__(self, cfg: Optional[dict] = None):
        cfg = cfg or {}
        self.mode = cfg.get("scheduler_mode", "off")
        if self.mode not in ("off", "static_threshold", "throughput"):
            raise ValueError(f"speculation.dspark.scheduler_mode {self.mode!r}")
        self.use_head = bool(cfg.get("confidence_enabled", False))
        if self.use_head and self.mode == "off":
            self.mode = "static_threshold"                 # confidence_enabled alone means: cut at the threshold
        self.threshold = float(cfg.get("confidence_threshold", 0.5))
        self.temps = [float(t) for t in cfg.get("sts_temperatures") or []]
        self.alpha = float(cfg.get("acceptance_ema_alpha", 0.3))
        self.row_cost = float(cfg.get("verify_row_cost", 0.03))
        self.trace_capacity = int(cfg.get("confidence_trace_capacity", 4096))
        self.trace: List[Tuple[Tuple[float, ...], int]] = []
        self.ema = 0.5                                     # the uninformed prior; every round moves it by ``acceptance_ema_alpha``
        self.probe_every = int(cfg.get("probe_every_rounds", 16))
        self._idle = 0
        self.rounds = self.proposed = self.accepted = 0

    def proxy(self) -> float:
        return self.ema

    def survival(self, conf: Sequence[float], n: int) -> List[float]:
        from .verify_plan import apply_temperature
        out, a = [], 1.0
        if self.use_head and len(conf) >= n:
            for k in range(n):
                c = min(max(float(conf[k]), 0.0), 1.0)
                if k < len(self.temps) and self.temps[k] != 1.0:
                    c = float(apply_temperature(c, self.temps[k]))
                a *= c
                out.append(a)
        else:
            p = self.proxy()
            for _ in range(n):
                a *= p
                out.append(a)
        return out

    def depth(self, conf: Sequence[float], n: int) -> int:
        if self.mode == "off" or n <= 0:
            return n
        k = self._choose(self.survival(conf, n), n)
        if k == 0:
            # nothing verified means nothing learned: every ``probe_every`` such rounds one token goes through anyway, so that an
            # acceptance rate that has recovered (another topic, another request) is noticed
            self._idle += 1
            if self.probe_every > 0 and self._idle >= self.probe_every:
                self._idle, k = 0, 1
        else:
            self._idle = 0
        return k

    def _choose(self, a: Sequence[float], n: int) -> int:
        if self.mode == "static_threshold":
            k = 0
            while k < n and a[k] >= self.threshold:
                k += 1
            return k
        best_k, best, tot = 0, 1.0, 1.0
        for k in range(1, n + 1):
            tot += a[k - 1]
            v = tot / (1.0 + self.row_cost * k)
            if v > best + 1e-12:
                best_k, best = k, v
        return best_k

    def record(self, conf: Sequence[float], proposed: int, accepted: int):
        if proposed <= 0:
            return
        accepted = min(max(int(accepted), 0), proposed)
        self.rounds += 1
        self.proposed += proposed
        self.accepted += accepted
        if self.use_head and len(conf) >= proposed:
            self.trace.append((tuple(float(c) for c in conf[:proposed]), accepted))
            if len(self.trace) > self.trace_capacity:
                del self.trace[: len(self.trace) - self.trace_capacity]
        # per-token acceptance of the positions that were actually decided (the first rejected one included)
        rate = accepted / min(proposed, accepted + 1)
        self.ema = self.alpha * rate + (1.0 - self.alpha) * self.ema

    def fit_temperatures(self, gamma: Optional[int] = None) -> List[float]:
        """Refit the per-position temperatures on the recorded rounds and use them from now on."""
        from .verify_plan import fit_sts_temperatures
        g = gamma or max((len(c) for c, _ in self.trace), default=0)
        self.temps = fit_sts_temperatures(self.trace, g) if g else []
        return self.temps


# ------------------------------------------------------------------------------------------------------------- draft sources
class _CorpusHook:
    """Writes what a block pass knew and what became of it to an expert-routing prediction corpus (``speculation/epm_corpus.py``)."""

    corpus = None

    def attach_corpus(self, writer):
        self.corpus = writer
        self.bb.collect_layers = writer is not None
        self._pending = None
        self._block_no: Dict[int, int] = {}
        self._ctx_len: Dict[int, int] = {}

    def _corpus_block(self, seq: int, anchor_pos: int, anchor: int, drafted: Sequence[int], conf: Sequence[float], proposed: Sequence[int],
                      context: Optional[Sequence[int]] = None):
        if self.corpus is None or self.bb.last_layer_hidden is None or not drafted:
            return
        n = self._block_no.get(seq, 0)
        self._block_no[seq] = n + 1
        if context is not None:
            # the tokens the sequence gained since its last block (all of them at its first): an offline labeller can re-run the target
            known = self._ctx_len.get(seq, 0) if n else 0
            self.corpus.write_context(seq, n, known, context[known:])
            self._ctx_len[seq] = len(context)
        self.corpus.write_block(seq, n, anchor_pos, anchor, drafted, conf or None, self.bb.last_layer_hidden[1: 1 + len(drafted)])
        self._pending = (seq, n, anchor_pos, list(proposed), list(conf))

    def last_expected_tokens(self) -> Optional[float]:
        """Expected committed tokens of the last proposal (the target's own token + the survival of each proposed row), for whoever
        weighs this proposal against another source's; None without a proposal."""
        n = getattr(self, "_last_n", 0)
        if n <= 0:
            return None
        return 1.0 + sum(self.sched.survival(self.last_confidences, n))

    def _corpus_feedback(self, proposed: int, accepted: int):
        if self.corpus is None or getattr(self, "_pending", None) is None:
            return
        seq, n, pos, ids, conf = self._pending
        self._pending = None
        self.corpus.write_manifest(seq, n, pos, proposed, accepted, ids[:accepted], conf)


class DsparkDraft(_CorpusHook):
    """``speculation.method = dspark`` as a draft source of the serving loop: ``propose(context, gamma)``.

    ``aux_of(tokens, first) -> [len(tokens) - first, N_aux * H]`` supplies the target's aux hidden states of positions
    ``first .. len(tokens) - 1`` for a token prefix (the CPU engine recomputes them with the reference model; the GPU engine
    captures them during its own steps, see ``DeviceDsparkDraft``).  One context is kept and followed by prefix matching: the
    positions the new request shares with it stay, the rest is overwritten - a rewind after a rejection, a fork from a cached prefix
    and a new conversation are the same operation."""

    def __init__(self, backbone: DsparkBackbone, aux_of: Callable[[Sequence[int], int], torch.Tensor], cfg: Optional[dict] = None):
        cfg = cfg or {}
        self.bb = backbone
        self.aux_of = aux_of
        self.ctx = backbone.new_context()
        self.sequence_no = 0
        self.max_tokens = min(int(cfg.get("speculative_tokens", backbone.cfg.speculative_tokens)), backbone.cfg.block_size - 1)
        self.sched = DsparkScheduler(dict(cfg, confidence_enabled=bool(cfg.get("confidence_enabled")) and backbone.confidence is not None))
        self.proposed = self.accepted = self.failures = 0
        self.last_confidences: List[float] = []

    def _follow(self, committed: Sequence[int]) -> bool:
        ctx = self.ctx
        m = 0
        n = min(len(ctx.tokens), len(committed), ctx.length)
        while m < n and ctx.tokens[m] == int(committed[m]):
            m += 1
        if not ctx.valid or m < ctx.base or len(ctx.tokens) != ctx.length:
            ctx.reset()
            m = 0
        if m == 0:
            self.sequence_no += 1                       # nothing shared with what was held: another conversation
        ctx.rewind(m)
        if len(committed) > ctx.length:
            first = ctx.length
            aux = self.aux_of(committed, first)
            return self.bb.ingest(ctx, aux, first, committed[first:])
        return True

    def propose(self, context: Sequence[int], gamma: int) -> List[int]:
        n = min(int(gamma), self.max_tokens)
        if n <= 0 or len(context) < 2:
            return []
        committed, anchor = context[:-1], int(context[-1])
        try:
            if not self._follow(committed):
                return []
            ids, self.last_confidences = self.bb.draft(self.ctx, anchor, len(committed), n)
        except (RuntimeError, ValueError):
            self.failures += 1
            self.ctx.reset()
            return []
        drafted = ids
        ids = ids[: self.sched.depth(self.last_confidences, len(ids))]
        self._corpus_block(self.sequence_no, len(committed), anchor, drafted, self.last_confidences, ids, context)
        self.proposed += len(ids)
        self._last_n = len(ids)
        return ids

    def feedback(self, proposed: int, accepted: int):
        self.accepted += accepted
        self.sched.record(self.last_confidences, proposed, accepted)
        self._corpus_feedback(proposed, accepted)

    def acceptance_rate(self) -> float:
        return self.accepted / self.proposed if self.proposed else 0.0


def oracle_aux_provider(oracle, layer_ids: Sequence[int], output_of_layer: bool = False) -> Callable[[Sequence[int], int], torch.Tensor]:
    """Aux hidden states from the fp32 reference model (the CPU engine's model): the stream entering each aux layer, or with
    ``output_of_layer`` the stream leaving it (checkpoints trained on layer outputs)."""
    ids = [int(l) + (1 if output_of_layer else 0) for l in layer_ids]

    def aux_of(tokens: Sequence[int], first: int) -> torch.Tensor:
        cap: Dict[int, torch.Tensor] = {l: None for l in ids}
        oracle.forward(torch.tensor([int(t) for t in tokens]), aux=cap)
        missing = [l for l, v in cap.items() if v is None]
        if missing:
            raise ValueError(f"aux layers {missing} are outside the target's {oracle.cfg.n_layers} layers")
        return torch.cat([cap[l][first:] for l in ids], -1)
    return aux_of


class DeviceDsparkDraft(_CorpusHook):
    """The block draft beside the GPU engine.  The engine reports the aux hidden states of every committed step
    (``Engine.enable_aux_capture``); they are fused and projected into the owning sequence's draft context at once, on the engine's
    stream, so the draft's context is complete the moment the step's token is known and a proposal costs one block pass.
    Sequences: a context per engine sequence, at most ``max_contexts`` (least recently used ones are dropped and their sequences
    stop drafting); a fork copies the parent's window up to the fork point, a rewind pulls the frontier back, a verify step's
    rejected rows are overwritten by the next step.  A sequence without a complete context proposes nothing - the target's output
    is the same either way."""

    def __init__(self, engine, backbone: DsparkBackbone, cfg: Optional[dict] = None, max_contexts: int = 4, output_of_layer: bool = False):
        cfg = cfg or {}
        self.engine, self.bb = engine, backbone
        ids = [l + (1 if output_of_layer else 0) for l in backbone.cfg.aux_hidden_state_layer_ids]
        if backbone.cfg.hidden_size != engine.cfg.hidden or backbone.cfg.vocab_size != engine.cfg.vocab:
            raise ValueError(f"the draft was trained for hidden {backbone.cfg.hidden_size} / vocabulary {backbone.cfg.vocab_size}, the target has "
                             f"{engine.cfg.hidden} / {engine.cfg.vocab}")
        self.max_tokens = min(int(cfg.get("speculative_tokens", backbone.cfg.speculative_tokens)), backbone.cfg.block_size - 1)
        self.sched = DsparkScheduler(dict(cfg, confidence_enabled=bool(cfg.get("confidence_enabled")) and backbone.confidence is not None))
        self.max_contexts = max(1, int(max_contexts))
        self.ctx: Dict[int, DsparkContext] = {}
        self._spare: List[DsparkContext] = []
        self._use = 0
        self._used: Dict[int, int] = {}
        self.proposed = self.accepted = self.failures = 0
        self.last_confidences: List[float] = []
        engine.enable_aux_capture(ids, self)

    # ---- the engine's notifications
    def _context(self, sid: int, create: bool) -> Optional[DsparkContext]:
        c = self.ctx.get(sid)
        if c is None and create:
            if len(self.ctx) >= self.max_contexts:
                old = min(self.ctx, key=lambda k: self._used.get(k, 0))
                self._spare.append(self.ctx.pop(old))
            c = self._spare.pop() if self._spare else self.bb.new_context()
            c.reset()
            self._seq_counter = getattr(self, "_seq_counter", 0) + 1
            c.corpus_seq = self._seq_counter
            self.ctx[sid] = c
        if c is not None:
            self._use += 1
            self._used[sid] = self._use
        return c

    def on_rows(self, sid: int, pos0: int, aux: torch.Tensor, tokens):
        c = self._context(sid, create=pos0 == 0)
        if c is not None:
            self.bb.ingest(c, aux, pos0, tokens)

    def on_rewind(self, sid: int, length: int):
        c = self.ctx.get(sid)
        if c is not None:
            c.rewind(length)

    def on_fork(self, parent: int, child: int, prefix_len: int):
        p = self.ctx.get(parent)
        if p is None or not p.valid or p.length < prefix_len or prefix_len < p.base:
            return
        c = self._context(child, create=True)
        p = self.ctx.get(parent)
        if p is None:                                  # the parent's context was the one that made room
            self.ctx.pop(child, None)
            return
        n = prefix_len - p.base
        c.k[:, :n].copy_(p.k[:, :n])
        c.v[:, :n].copy_(p.v[:, :n])
        c.base, c.length, c.valid, c.tokens = p.base, prefix_len, True, list(p.tokens[:prefix_len])

    def on_free(self, sid: int):
        c = self.ctx.pop(sid, None)
        self._used.pop(sid, None)
        if c is not None:
            self._spare.append(c)

    # ---- the serving loop's draft source
    def _sequence_of(self, context: Sequence[int]) -> Optional[int]:
        n = len(context) - 1
        tail = [int(t) for t in context[max(0, n - 8): n]]
        for sid, s in self.engine.seqs.items():
            if s.length == n and len(s.tokens) == n and s.tokens[-8:] == tail and sid in self.ctx:
                return sid
        return None

    def propose(self, context: Sequence[int], gamma: int) -> List[int]:
        n = min(int(gamma), self.max_tokens)
        if n <= 0 or len(context) < 2:
            return []
        sid = self._sequence_of(context)
        c = self.ctx.get(sid) if sid is not None else None
        if c is None or not c.valid or c.length != len(context) - 1:
            return []
        try:
            stream = getattr(self.engine, "stream", None)
            with (torch.cuda.stream(stream) if stream is not None else contextlib.nullcontext()):
                ids, self.last_confidences = self.bb.draft(c, int(context[-1]), c.length, n)
        except (RuntimeError, ValueError):
            self.failures += 1
            c.valid = False
            return []
        self._used[sid] = self._use = self._use + 1
        drafted = ids
        ids = ids[: self.sched.depth(self.last_confidences, len(ids))]
        self._corpus_block(getattr(c, "corpus_seq", sid), c.length, int(context[-1]), drafted, self.last_confidences, ids, context)
        self.proposed += len(ids)
        self._last_n = len(ids)
        return ids

    def feedback(self, proposed: int, accepted: int):
        self.accepted += accepted
        self.sched.record(self.last_confidences, proposed, accepted)
        self._corpus_feedback(proposed, accepted)

    def acceptance_rate(self) -> float:
        return self.accepted / self.proposed if self.proposed else 0.0
