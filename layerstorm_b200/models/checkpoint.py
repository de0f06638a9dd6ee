"""Checkpoint readers that present any supported on-disk format under the engine's canonical
tensor names (see ``models/weights.py``), lazily: a tensor is read, dequantised and reshaped only
when ``DeviceModel.from_state_dict`` asks for it, so a 700 GB checkpoint never sits in host memory.

Formats: HuggingFace safetensors directories (bf16/fp16/fp32, DeepSeek-style FP8 with
``weight_scale_inv`` 128x128 block scales, ModelOpt NVFP4 with ``weight_scale`` / ``weight_scale_2``)
and GGUF files (single or ``-0000N-of-0000M`` split; F32/F16/BF16/Q8_0/K-quants/MXFP4).
Name maps follow the reference's tensor-id parser (src/model/weight_loader/tensor_id.cpp:175-640):
HF ``model.layers.N.self_attn.*`` / ``mlp.*`` and GGUF ``blk.N.*``.
"""
from __future__ import annotations

import glob
import json
import os
import re
from collections.abc import Mapping
from typing import Callable, Dict, Iterator, List, Optional

import numpy as np
import torch

from ..formats import quant
from ..formats.gguf import GgufReader
from ..formats.safetensors import SafetensorsReader
from .config import ModelConfig, from_hf_config

# canonical suffix -> HF module path (under model.layers.N.)
_HF_LAYER = {
    "attn_norm.weight": "input_layernorm.weight", "ffn_norm.weight": "post_attention_layernorm.weight",
    "attn.q_a": "self_attn.q_a_proj", "attn.q_a_norm": "self_attn.q_a_layernorm.weight", "attn.q_b": "self_attn.q_b_proj",
    "attn.kv_a": "self_attn.kv_a_proj_with_mqa", "attn.kv_a_norm": "self_attn.kv_a_layernorm.weight", "attn.o": "self_attn.o_proj",
    "indexer.wq_b": "self_attn.indexer.wq_b", "indexer.wk": "self_attn.indexer.wk",
    "indexer.k_norm.weight": "self_attn.indexer.k_norm.weight", "indexer.k_norm.bias": "self_attn.indexer.k_norm.bias",
    "indexer.weights_proj": "self_attn.indexer.weights_proj", "indexer.gate": "self_attn.indexer.index_kpool_compress_gate",
    "indexer.ape": "self_attn.indexer.index_kpool_compress_ape",
    "kda.q": "self_attn.q_proj", "kda.k": "self_attn.k_proj", "kda.v": "self_attn.v_proj", "kda.beta": "self_attn.b_proj",
    "kda.f_a": "self_attn.f_a_proj", "kda.f_b": "self_attn.f_b_proj", "kda.g_a": "self_attn.g_a_proj", "kda.g_b": "self_attn.g_b_proj",
    "kda.conv_q": "self_attn.q_conv1d.weight", "kda.conv_k": "self_attn.k_conv1d.weight", "kda.conv_v": "self_attn.v_conv1d.weight",
    "kda.a_log": "self_attn.A_log", "kda.dt_bias": "self_attn.dt_bias", "kda.o_norm": "self_attn.o_norm.weight", "kda.o": "self_attn.o_proj",
    "hc_attn.fn": "hc_attn_fn", "hc_attn.scale": "hc_attn_scale", "hc_attn.base": "hc_attn_base",
    "hc_ffn.fn": "hc_ffn_fn", "hc_ffn.scale": "hc_ffn_scale", "hc_ffn.base": "hc_ffn_base",
    "mlp.gate": "mlp.gate_proj", "mlp.up": "mlp.up_proj", "mlp.down": "mlp.down_proj",
    "moe.router": "mlp.gate.weight", "moe.router_bias": "mlp.gate.e_score_correction_bias", "moe.tid2eid": "mlp.gate.tid2eid",
    # multi-token-prediction blocks (layer ids >= num_hidden_layers)
    "mtp.enorm": "enorm.weight", "mtp.hnorm": "hnorm.weight", "mtp.eh_proj": "eh_proj", "mtp.final_norm": "shared_head.norm.weight",
}
_GGUF_LAYER = {
    "attn_norm.weight": "attn_norm.weight", "ffn_norm.weight": "ffn_norm.weight",
    "attn.q_a": "attn_q_a.weight", "attn.q_a_norm": "attn_q_a_norm.weight", "attn.q_b": "attn_q_b.weight",
    "attn.kv_a": "attn_kv_a_mqa.weight", "attn.kv_a_norm": "attn_kv_a_norm.weight", "attn.o": "attn_output.weight",
    "indexer.wq_b": "indexer.attn_q_b.weight", "indexer.wk": "indexer.attn_k.weight", "indexer.k_norm.weight": "indexer.k_norm.weight",
    "indexer.k_norm.bias": "indexer.k_norm.bias", "indexer.weights_proj": "indexer.proj.weight",
    "indexer.gate": "indexer_compressor_gate.weight", "indexer.ape": "indexer_compressor_ape.weight",
    "kda.q": "attn_q.weight", "kda.k": "attn_k.weight", "kda.v": "attn_v.weight", "kda.beta": "ssm_beta.weight",
    "kda.f_a": "ssm_f_a.weight", "kda.f_b": "ssm_f_b.weight", "kda.g_a": "ssm_g_a.weight", "kda.g_b": "ssm_g_b.weight",
    "kda.conv_q": "ssm_conv1d_q.weight", "kda.conv_k": "ssm_conv1d_k.weight", "kda.conv_v": "ssm_conv1d_v.weight",
    "kda.a_log": "ssm_a", "kda.dt_bias": "ssm_dt.bias", "kda.o_norm": "ssm_norm.weight", "kda.o": "attn_output.weight",
    "hc_attn.fn": "hc_attn_fn.weight", "hc_attn.scale": "hc_attn_scale.weight", "hc_attn.base": "hc_attn_base.weight",
    "hc_ffn.fn": "hc_ffn_fn.weight", "hc_ffn.scale": "hc_ffn_scale.weight", "hc_ffn.base": "hc_ffn_base.weight",
    "mlp.gate": "ffn_gate.weight", "mlp.up": "ffn_up.weight", "mlp.down": "ffn_down.weight",
    "moe.router": "ffn_gate_inp.weight", "moe.router_bias": "exp_probs_b.bias", "moe.tid2eid": "ffn_gate_tid2eid.weight",
    "mtp.enorm": "nextn.enorm.weight", "mtp.hnorm": "nextn.hnorm.weight", "mtp.eh_proj": "nextn.eh_proj.weight",
    "mtp.final_norm": "nextn.shared_head_norm.weight",
}
_LAYER_RE = re.compile(r"^layers\.(\d+)\.(.+)$")
_EXPERT_RE = re.compile(r"^moe\.(experts|shared)\.(\d+)\.(gate|up|down)$")


class _Source:
    """A set of files addressed by source tensor name, returning fp32 torch tensors."""

    def names(self) -> List[str]:
        raise NotImplementedError

    def has(self, name: str) -> bool:
        raise NotImplementedError

    def load(self, name: str) -> torch.Tensor:
        raise NotImplementedError


class SafetensorsSource(_Source):
    def __init__(self, directory: str):
        self.dir = directory
        idx = os.path.join(directory, "model.safetensors.index.json")
        self.where: Dict[str, str] = {}
        self.readers: Dict[str, SafetensorsReader] = {}
        if os.path.exists(idx):
            self.where = dict(json.load(open(idx))["weight_map"])
        else:
            for f in sorted(glob.glob(os.path.join(directory, "*.safetensors"))):
                r = self._reader(os.path.basename(f))
                for k in r.keys():
                    self.where[k] = os.path.basename(f)
        # multimodal checkpoints nest the text model
        self.prefix = "model.language_model." if any(k.startswith("model.language_model.") for k in self.where) else "model."

    def _reader(self, fname: str) -> SafetensorsReader:
        if fname not in self.readers:
            self.readers[fname] = SafetensorsReader(os.path.join(self.dir, fname))
        return self.readers[fname]

    def names(self):
        return list(self.where)

    def has(self, name):
        return name in self.where

    def raw(self, name: str) -> torch.Tensor:
        return self._reader(self.where[name]).get(name)

    def load(self, name: str) -> torch.Tensor:
        """``name`` is a module path without the ``.weight`` suffix for linears (so the scale
        companions can be found) or a full tensor name."""
        if name in self.where:
            return self.raw(name).float()
        wn = name + ".weight"
        w = self.raw(wn)
        if name + ".weight_scale_inv" in self.where:                 # FP8 e4m3 with 128x128 block scales
            return quant.dequantize_fp8_block(w.view(torch.uint8) if w.dtype != torch.uint8 else w, self.raw(name + ".weight_scale_inv").float())
        if name + ".weight_scale_2" in self.where:                   # NVFP4: packed nibbles + e4m3 group scales (row-major) + global
            sf = self.raw(name + ".weight_scale")
            g = float(self.raw(name + ".weight_scale_2").float().reshape(-1)[0])
            return dequant_nvfp4_rowmajor(w.view(torch.uint8), sf.view(torch.uint8), g)
        if name + ".weight_scale" in self.where and w.dtype in (torch.uint8, torch.float8_e4m3fn):
            s = self.raw(name + ".weight_scale").float()
            wf = w.view(torch.float8_e4m3fn).float() if w.dtype == torch.uint8 else w.float()
            return wf * (s if s.numel() == 1 else s.reshape(-1, 1))
        return w.float()


def dequant_nvfp4_rowmajor(packed: torch.Tensor, sf: torch.Tensor, gscale: float) -> torch.Tensor:
    """ModelOpt layout: packed [N, K/2] (low nibble = even k), group scales e4m3 [N, K/16] row-major."""
    N, K2 = packed.shape
    lut = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], dtype=torch.float32)
    lo = lut[(packed & 0xF).long()]
    hi = lut[(packed >> 4).long()]
    w = torch.stack([lo, hi], -1).reshape(N, K2 * 2)
    s = sf.view(torch.float8_e4m3fn).float().reshape(N, -1)
    return (w.reshape(N, -1, 16) * s.unsqueeze(-1)).reshape(N, K2 * 2) * gscale


class GgufSource(_Source):
    def __init__(self, path: str):
        m = re.match(r"^(.*)-(\d{5})-of-(\d{5})\.gguf$", path)
        files = [f"{m.group(1)}-{i:05d}-of-{m.group(3)}.gguf" for i in range(1, int(m.group(3)) + 1)] if m else [path]
        self.readers = [GgufReader(f) for f in files if os.path.exists(f)]
        self.where: Dict[str, GgufReader] = {}
        for r in self.readers:
            for n in r.tensor_names():
                self.where[n] = r

    def names(self):
        return list(self.where)

    def has(self, name):
        return name in self.where

    def meta(self, key, default=None):
        for r in self.readers:
            v = r.meta(key, None)
            if v is not None:
                return v
        return default

    def ggml_type(self, name: str) -> int:
        return self.where[name].tensor_type(name)

    def load(self, name: str) -> torch.Tensor:
        return torch.from_numpy(np.ascontiguousarray(self.where[name].get(name))).float()


class LazyCheckpoint(Mapping):
    """Canonical-name view over a source.  ``w["layers.3.attn.k_b"]`` etc."""

    def __init__(self, cfg: ModelConfig, src: _Source, kind: str):
        self.cfg, self.src, self.kind = cfg, src, kind
        self._kvb_cache: Dict[int, torch.Tensor] = {}

    # ---- Mapping ----
    def __iter__(self) -> Iterator[str]:
        raise TypeError("LazyCheckpoint is addressed by name; iterate the model's expected names instead")

    def __len__(self) -> int:
        return len(self.src.names())

    def __contains__(self, key) -> bool:
        try:
            return self._resolve(key) is not None
        except KeyError:
            return False

    def __getitem__(self, key: str) -> torch.Tensor:
        fn = self._resolve(key)
        if fn is None:
            raise KeyError(key)
        return fn()

    # ---- resolution ----
    def _resolve(self, key: str) -> Optional[Callable[[], torch.Tensor]]:
        return self._resolve_hf(key) if self.kind == "hf" else self._resolve_gguf(key)

    def _lin(self, path: str):
        s = self.src
        if s.has(path + ".weight") or s.has(path):
            return lambda: s.load(path)
        return None

    def _resolve_hf(self, key: str):
        s: SafetensorsSource = self.src
        P = s.prefix
        top = {"embed.weight": P + "embed_tokens.weight", "final_norm.weight": P + "norm.weight"}
        if key in top:
            return (lambda: s.load(top[key])) if s.has(top[key]) else None
        if key == "head.weight":
            if s.has("lm_head.weight"):
                return lambda: s.load("lm_head.weight")
            return lambda: s.load(P + "embed_tokens.weight")            # tied embeddings
        m = _LAYER_RE.match(key)
        if not m:
            return None
        i, rest = int(m.group(1)), m.group(2)
        L = f"{P}layers.{i}."
        if rest in ("attn.k_b", "attn.v_b"):
            return lambda: self._split_kv_b(i, lambda: s.load(L + "self_attn.kv_b_proj"), rest)
        e = _EXPERT_RE.match(rest)
        if e:
            kind, idx, proj = e.group(1), int(e.group(2)), e.group(3) + "_proj"
            if kind == "experts":
                return self._lin(f"{L}mlp.experts.{idx}.{proj}")
            return self._lin(f"{L}mlp.shared_experts.{proj}") or self._lin(f"{L}mlp.shared_experts.{idx}.{proj}")
        if rest not in _HF_LAYER:
            return None
        path = L + _HF_LAYER[rest]
        if rest.startswith("kda.conv_"):
            return (lambda: s.load(path).reshape(-1, self.cfg.kda_conv)) if s.has(path) else None
        if rest == "kda.dt_bias":
            return (lambda: s.load(path).reshape(self.cfg.kda_heads, -1)) if s.has(path) else None
        if rest == "kda.a_log":
            return (lambda: s.load(path).reshape(-1)) if s.has(path) else None
        if s.has(path):
            return lambda: s.load(path)
        return self._lin(path)

    def _split_kv_b(self, i: int, loader, which: str) -> torch.Tensor:
        c = self.cfg
        if i not in self._kvb_cache:
            self._kvb_cache = {i: loader().reshape(c.n_heads, c.qk_nope + c.v_head, c.kv_lora)}
        kvb = self._kvb_cache[i]
        if which == "attn.k_b":
            return kvb[:, :c.qk_nope, :].transpose(1, 2).contiguous()          # [H, dl, dn]
        return kvb[:, c.qk_nope:, :].contiguous()                             # [H, dv, dl]

    def _resolve_gguf(self, key: str):
        s: GgufSource = self.src
        c = self.cfg
        top = {"embed.weight": "token_embd.weight", "final_norm.weight": "output_norm.weight"}
        if key in top:
            return (lambda: s.load(top[key])) if s.has(top[key]) else None
        if key == "head.weight":
            n = "output.weight" if s.has("output.weight") else "token_embd.weight"
            return lambda: s.load(n)
        m = _LAYER_RE.match(key)
        if not m:
            return None
        i, rest = int(m.group(1)), m.group(2)
        B = f"blk.{i}."
        if rest == "attn.k_b":
            if s.has(B + "attn_k_b.weight"):      # stored [H, dn, dl] (ggml ne = [dn? ...]); normalise to [H, dl, dn]
                def f():
                    t = s.load(B + "attn_k_b.weight")
                    t = t.reshape(c.n_heads, -1, t.shape[-1])
                    return t if t.shape[1] == c.kv_lora else t.transpose(1, 2).contiguous()
                return f
            return lambda: self._split_kv_b(i, lambda: s.load(B + "attn_kv_b.weight"), rest)
        if rest == "attn.v_b":
            if s.has(B + "attn_v_b.weight"):
                return lambda: s.load(B + "attn_v_b.weight").reshape(c.n_heads, c.v_head, c.kv_lora)
            return lambda: self._split_kv_b(i, lambda: s.load(B + "attn_kv_b.weight"), rest)
        e = _EXPERT_RE.match(rest)
        if e:
            kind, idx, proj = e.group(1), int(e.group(2)), e.group(3)
            name = f"{B}ffn_{proj}_{'exps' if kind == 'experts' else 'shexp'}.weight"
            if not s.has(name):
                return None
            if kind == "experts":
                return lambda: self._expert_slice(name, idx)
            return lambda: s.load(name)
        if rest not in _GGUF_LAYER:
            return None
        name = B + _GGUF_LAYER[rest]
        if not s.has(name):
            return None
        if rest.startswith("kda.conv_"):
            return lambda: s.load(name).reshape(-1, c.kda_conv)
        if rest == "kda.a_log":
            # GGUF stores A = -exp(A_log) per head (src/model/weight_loader/tensor_id.cpp:467); invert it
            return lambda: torch.log(-s.load(name).reshape(-1))
        if rest == "kda.dt_bias":
            return lambda: s.load(name).reshape(c.kda_heads, -1)
        return lambda: s.load(name)

    def native_ggml(self, key: str):
        """(ggml type, file-order blocks as a flat uint8 array, rows, cols) of an expert matrix whose GGUF tensor is stored in a
        block type the GPU kernels read natively (Q4_K, Q5_K, Q6_K, Q8_0), else None.  Lets the device model take such experts
        bit-exactly instead of de-quantising and re-quantising them."""
        if self.kind != "gguf":
            return None
        m = _LAYER_RE.match(key)
        if not m:
            return None
        e = _EXPERT_RE.match(m.group(2))
        if not e:
            return None
        kind, idx, proj = e.group(1), int(e.group(2)), e.group(3)
        name = f"blk.{int(m.group(1))}.ffn_{proj}_{'exps' if kind == 'experts' else 'shexp'}.weight"
        s: GgufSource = self.src
        if not s.has(name):
            return None
        from ..formats import gguf as _g
        t = s.ggml_type(name)
        if t not in _g.DEVICE_NATIVE:
            return None
        r = s.where[name]
        shape = r.tensor_shape(name)                       # [E, rows, cols] or [rows, cols]
        rows, cols = int(shape[-2]), int(shape[-1])
        if cols % 256:
            return None
        per = _g.nbytes_for(t, rows * cols)
        raw = r.raw(name)
        off = idx * per if (kind == "experts" and len(shape) == 3) else 0
        return t, np.ascontiguousarray(raw[off: off + per]), rows, cols

    def native_q4k(self, key: str) -> Optional[torch.Tensor]:
        """Raw Q4_K super-blocks ([rows, cols / 256 * 144] uint8) of an expert matrix whose GGUF tensor is stored as Q4_K, else
        None.  Lets the device model take such experts bit-exactly instead of de-quantising and re-quantising them."""
        if self.kind != "gguf":
            return None
        m = _LAYER_RE.match(key)
        if not m:
            return None
        e = _EXPERT_RE.match(m.group(2))
        if not e:
            return None
        kind, idx, proj = e.group(1), int(e.group(2)), e.group(3)
        name = f"blk.{int(m.group(1))}.ffn_{proj}_{'exps' if kind == 'experts' else 'shexp'}.weight"
        s: GgufSource = self.src
        if not s.has(name):
            return None
        from ..formats import gguf as _g
        if s.ggml_type(name) != _g.GGML_TYPES["Q4_K"]:
            return None
        r = s.where[name]
        shape = r.tensor_shape(name)                       # [E, rows, cols] or [rows, cols]
        rows, cols = int(shape[-2]), int(shape[-1])
        if cols % 256:
            return None
        per = rows * cols // 256 * 144
        raw = r.raw(name)
        off = idx * per if (kind == "experts" and len(shape) == 3) else 0
        return torch.from_numpy(np.ascontiguousarray(raw[off: off + per])).view(rows, cols // 256 * 144)

    def _expert_slice(self, name: str, e: int) -> torch.Tensor:
        """One expert's matrix out of a stacked [E, rows, cols] GGUF tensor, dequantising only its blocks."""
        s: GgufSource = self.src
        r = s.where[name]
        shape = r.tensor_shape(name)                       # numpy order: [E, rows, cols]
        per = int(np.prod(shape[1:]))
        return torch.from_numpy(np.ascontiguousarray(r.get_slice(name, e * per, per))).float().reshape(shape[1:])


class QuantSkipList:
    """The modules a mixed-precision (FP8) HuggingFace checkpoint keeps unquantised: ``quantization_config.modules_to_not_convert`` of
    its ``config.json``.  This loader never converts dtypes (the safetensors header is the authority), so the list is a correctness
    cross-check: every matrix-shaped weight must be FP8 exactly when it is NOT on the list.

    The list names MODULE paths of the loaded model (``model.layers.N...``, ``visual...``) while multimodal checkpoints store their
    TENSORS under a wrapper (``model.language_model.layers.N...``, ``model.visual...``): a literal comparison matches nothing.  Both
    sides are therefore brought into one namespace first (wrapper prefixes and the role suffix ``.weight`` / ``.weight_scale`` /
    ``.weight_scale_inv`` / ``.bias`` stripped).  An entry matches a tensor when it equals the tensor's module path or is a whole-path
    prefix of it (``model.layers.3.self_attn`` covers ``model.layers.3.self_attn.kv_b_proj.weight``).
    Reference: src/model/weight_loader/quant_skip_list.h (same cross-check, fails the load on disagreement or on a list that matches
    no tensor)."""
    _ROLES = (".weight_scale_inv", ".weight_scale_2", ".weight_scale", ".weight", ".bias")

    def __init__(self, entries, quant_method: str = ""):
        self.quant_method = quant_method
        self.entries = sorted({self.canonical(e) for e in entries if e})

    @staticmethod
    def canonical(name: str) -> str:
        n = name.strip()
        for r in QuantSkipList._ROLES:
            if n.endswith(r):
                n = n[: -len(r)]
                break
        for pre in ("model.language_model.", "language_model.model.", "language_model."):
            if n.startswith(pre):
                n = "model." + n[len(pre):]
                break
        if n == "visual" or n.startswith("visual."):
            n = "model." + n
        return n

    @classmethod
    def from_model_dir(cls, directory: str) -> Optional["QuantSkipList"]:
        cj = os.path.join(directory, "config.json")
        if not os.path.exists(cj):
            return None
        c = json.load(open(cj))
        qc = c.get("quantization_config") or (c.get("text_config") or {}).get("quantization_config")
        if not isinstance(qc, dict) or "modules_to_not_convert" not in qc:
            return None
        ents = qc["modules_to_not_convert"]
        if ents is not None and not isinstance(ents, list):
            raise ValueError("quantization_config.modules_to_not_convert must be a list")
        return cls(ents or [], str(qc.get("quant_method", "")))

    def matches(self, tensor_name: str) -> bool:
        n = self.canonical(tensor_name)
        import bisect
        i = bisect.bisect_right(self.entries, n)
        if i and self.entries[i - 1] == n:
            return True
        # a prefix entry sorts before the name; walk the path upwards instead of scanning the list
        parts = n.split(".")
        for k in range(len(parts) - 1, 0, -1):
            pre = ".".join(parts[:k])
            j = bisect.bisect_left(self.entries, pre)
            if j < len(self.entries) and self.entries[j] == pre:
                return True
        return False

    def cross_check(self, dtype_of: Dict[str, str], shape_of: Dict[str, tuple]) -> dict:
        """``dtype_of`` / ``shape_of``: safetensors dtype string and shape per tensor name.  Raises ``ValueError`` when an FP8 matrix is
        on the list, a listed-free matrix with a scale companion is not FP8, or a non-empty list matches no tensor at all."""
        fp8 = {"F8_E4M3", "F8_E5M2"}
        matched = 0
        bad = []
        for name, dt in dtype_of.items():
            if not name.endswith(".weight") or len(shape_of.get(name, ())) < 2:
                continue
            listed = self.matches(name)
            matched += listed
            is_fp8 = dt in fp8
            has_scale = (name[: -len(".weight")] + ".weight_scale_inv") in dtype_of or (name[: -len(".weight")] + ".weight_scale") in dtype_of
            if listed and is_fp8:
                bad.append(f"{name}: FP8 although its module is listed as not converted")
            elif not listed and not is_fp8 and has_scale:
                bad.append(f"{name}: carries a quantisation scale but is stored as {dt}")
        if self.entries and matched == 0:
            bad.append(f"none of the {len(self.entries)} modules_to_not_convert entries matches a tensor of this checkpoint (namespace mismatch?)")
        if bad:
            raise ValueError("quantisation skip list disagrees with the checkpoint: " + "; ".join(bad[:6]) + (f" (+{len(bad) - 6} more)" if len(bad) > 6 else ""))
        return {"entries": len(self.entries), "matrices_kept": matched}


def open_checkpoint(path: str, cfg: Optional[ModelConfig] = None) -> tuple[ModelConfig, LazyCheckpoint]:
    """``path`` = HF directory, a ``.safetensors`` file inside one, or a ``.gguf`` file (first shard)."""
    if path.endswith(".gguf"):
        src = GgufSource(path)
        if cfg is None:
            cj = os.path.join(os.path.dirname(path), "config.json")
            if os.path.exists(cj):
                cfg = from_hf_config(cj)
            else:
                from ..autoconfig.modelprobe import shape_from_gguf
                cfg = shape_from_gguf(src)                      # llama.cpp metadata keys of the file itself
        return cfg, LazyCheckpoint(cfg, src, "gguf")
    d = path if os.path.isdir(path) else os.path.dirname(path)
    if cfg is None:
        cfg = from_hf_config(os.path.join(d, "config.json"))
    src = SafetensorsSource(d)
    skip = QuantSkipList.from_model_dir(d)
    if skip is not None and skip.quant_method in ("fp8", ""):
        dts, shp = {}, {}
        for fname in sorted(set(src.where.values())):
            for name, (dt, shape) in src._reader(fname).header_items().items():
                dts[name], shp[name] = dt, shape
        if any(dt in ("F8_E4M3", "F8_E5M2") for dt in dts.values()):
            skip.cross_check(dts, shp)                       # load-stopping on disagreement
    ck = LazyCheckpoint(cfg, src, "hf")
    ck.quant_skip = skip
    return cfg, ck


def export_hf(cfg: ModelConfig, w: Dict[str, torch.Tensor], directory: str, dtype=torch.bfloat16, shard_bytes: int = 1 << 30):
    """Write a canonical state dict as a HuggingFace-layout safetensors directory (+ index, + config.json).
    Used by tests and by the tiny-model tooling."""
    from ..formats.safetensors import write_safetensors
    os.makedirs(directory, exist_ok=True)
    out: Dict[str, torch.Tensor] = {"model.embed_tokens.weight": w["embed.weight"], "lm_head.weight": w["head.weight"],
                                    "model.norm.weight": w["final_norm.weight"]}
    kvb: Dict[int, dict] = {}
    for k, v in w.items():
        m = _LAYER_RE.match(k)
        if not m:
            continue
        i, rest = int(m.group(1)), m.group(2)
        L = f"model.layers.{i}."
        if rest in ("attn.k_b", "attn.v_b"):
            kvb.setdefault(i, {})[rest] = v
            continue
        e = _EXPERT_RE.match(rest)
        if e:
            kind, idx, proj = e.group(1), int(e.group(2)), e.group(3) + "_proj"
            out[f"{L}mlp.experts.{idx}.{proj}.weight" if kind == "experts" else f"{L}mlp.shared_experts.{proj}.weight"] = v
            continue
        hp = _HF_LAYER[rest]
        full = L + hp
        is_tensor_name = hp.endswith((".weight", ".bias")) or hp.split(".")[-1] in ("A_log", "dt_bias", "tid2eid") or hp.startswith("hc_")
        out[full if is_tensor_name else full + ".weight"] = v
    for i, d in kvb.items():
        kb = d["attn.k_b"].transpose(1, 2)                  # [H, dn, dl]
        out[f"model.layers.{i}.self_attn.kv_b_proj.weight"] = torch.cat([kb, d["attn.v_b"]], 1).reshape(-1, cfg.kv_lora)
    keep32 = ("A_log", "dt_bias", "hc_", "e_score_correction_bias", "mlp.gate.weight", "conv1d", "compress_ape", "norm")
    shards: List[Dict[str, torch.Tensor]] = [{}]
    size = 0
    for k in sorted(out):
        t = out[k].contiguous()
        if k.endswith("tid2eid"):
            t = t.to(torch.int32)                            # integer table: stays integer in the file
        else:
            t = t.float() if any(s in k for s in keep32) else t.to(dtype)
        if size + t.numel() * t.element_size() > shard_bytes and shards[-1]:
            shards.append({})
            size = 0
        shards[-1][k] = t
        size += t.numel() * t.element_size()
    weight_map = {}
    for n, sh in enumerate(shards):
        fn = f"model-{n + 1:05d}-of-{len(shards):05d}.safetensors"
        write_safetensors(os.path.join(directory, fn), sh)
        weight_map.update({k: fn for k in sh})
    json.dump({"metadata": {}, "weight_map": weight_map}, open(os.path.join(directory, "model.safetensors.index.json"), "w"))
    json.dump(hf_config_dict(cfg), open(os.path.join(directory, "config.json"), "w"), indent=1)


def hf_config_dict(c: ModelConfig) -> dict:
    mt = {"deepseek_v3": "deepseek_v3", "glm_moe_dsa": "glm_moe_dsa", "glm5_next": "glm5_next", "kimi_k25": "kimi_k25", "deepseek_v4": "deepseek_v4"}[c.architecture]
    d = {"model_type": mt, "hidden_size": c.hidden, "num_hidden_layers": c.n_layers, "num_nextn_predict_layers": c.n_mtp, "vocab_size": c.vocab,
         "rms_norm_eps": c.rms_eps,
         "num_attention_heads": c.n_heads, "q_lora_rank": c.q_lora, "kv_lora_rank": c.kv_lora, "qk_nope_head_dim": c.qk_nope,
         "qk_rope_head_dim": c.qk_rope, "v_head_dim": c.v_head, "rope_theta": c.rope_theta, "max_position_embeddings": c.max_position,
         "intermediate_size": c.dense_inter, "first_k_dense_replace": c.first_k_dense, "n_routed_experts": c.n_routed,
         "num_experts_per_tok": c.top_k, "n_shared_experts": c.n_shared, "moe_intermediate_size": c.moe_inter, "scoring_func": c.scoring,
         "n_group": c.n_group, "topk_group": c.topk_group, "routed_scaling_factor": c.routed_scale, "norm_topk_prob": c.norm_topk_prob,
         "topk_method": "noaux_tc" if c.router_bias else "greedy", "swiglu_limit": c.swiglu_limit, "index_n_heads": c.index_n_heads,
         "index_head_dim": c.index_head_dim, "index_topk": c.index_topk, "index_topk_freq": c.index_topk_freq, "index_kpool": c.index_kpool,
         "eos_token_id": c.eos_token_ids or [0]}
    if c.rope_yarn_factor > 1:
        d["rope_scaling"] = {"type": "yarn", "factor": c.rope_yarn_factor, "original_max_position_embeddings": c.rope_yarn_orig_max,
                             "beta_fast": c.rope_yarn_beta_fast, "beta_slow": c.rope_yarn_beta_slow, "mscale_all_dim": c.rope_yarn_mscale_all_dim}
    if "kda" in c.layer_types:
        d["layer_types"] = ["linear_attention" if t == "kda" else "deepseek_sparse_attention" for t in c.layer_types]
        d["linear_attn_config"] = {"num_heads": c.kda_heads, "head_dim": c.kda_head_dim, "short_conv_kernel_size": c.kda_conv,
                                   "gate_low_rank": c.kda_rank, "gate_lower_bound": c.kda_lower_bound}
    if c.num_hash_layers:
        d["num_hash_layers"] = c.num_hash_layers
    if c.mhc:
        d.update({"mhc": True, "hc_mult": c.hc_mult, "hc_eps": c.hc_eps, "hc_sinkhorn_iters": c.hc_sinkhorn_iters})
    return d
