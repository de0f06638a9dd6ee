"""Model identity from a bare path: HF directory, GGUF file (shape from its metadata), prepacked directory, built-in shape."""
import json

import numpy as np
import pytest

from layerstorm_b200 import build as _build

_build.build_all(only="runtime")

from layerstorm_b200.autoconfig.modelprobe import probe, shape_from_gguf
from layerstorm_b200.formats.gguf import GgufReader, GgufWriter
from layerstorm_b200.models.checkpoint import hf_config_dict, open_checkpoint
from layerstorm_b200.models.config import deepseek_v3_2, tiny_mla_moe


def _gguf_meta(gw, c, arch="deepseek2"):
    gw.meta("general.architecture", arch)
    gw.meta("general.name", "probe-me")
    kv = {"block_count": c.n_layers, "embedding_length": c.hidden, "attention.head_count": c.n_heads, "attention.q_lora_rank": c.q_lora,
          "attention.kv_lora_rank": c.kv_lora, "attention.key_length": c.kv_lora + c.qk_rope, "attention.value_length": c.kv_lora,
          "attention.key_length_mla": c.qk_nope + c.qk_rope, "attention.value_length_mla": c.v_head, "rope.dimension_count": c.qk_rope,
          "expert_count": c.n_routed, "expert_used_count": c.top_k, "expert_shared_count": c.n_shared, "expert_feed_forward_length": c.moe_inter,
          "feed_forward_length": c.dense_inter, "leading_dense_block_count": c.first_k_dense, "vocab_size": c.vocab, "context_length": c.max_position,
          "expert_gating_func": 2 if c.scoring == "sigmoid" else 1, "expert_group_count": c.n_group, "expert_group_used_count": c.topk_group}
    for k, v in kv.items():
        gw.meta(f"{arch}.{k}", int(v))
    gw.meta(f"{arch}.rope.freq_base", float(c.rope_theta))
    gw.meta(f"{arch}.expert_weights_scale", float(c.routed_scale))
    gw.meta(f"{arch}.attention.layer_norm_rms_epsilon", float(c.rms_eps))


@pytest.mark.parametrize("make", [tiny_mla_moe, deepseek_v3_2])
def test_shape_from_gguf_metadata(tmp_path, make):
    c = make()
    gw = GgufWriter()
    _gguf_meta(gw, c)
    gw.add("token_embd.weight", np.zeros((4, 8), np.float32))
    gw.add("blk.1.ffn_gate_exps.weight", np.zeros((2, 32, 32), np.float32), ggml_type=8)
    p = str(tmp_path / "m.gguf")
    gw.write(p)
    r = GgufReader(p)
    s = shape_from_gguf(r)
    r.close()
    for f in ("hidden", "n_layers", "vocab", "n_heads", "q_lora", "kv_lora", "qk_nope", "qk_rope", "v_head", "n_routed", "top_k", "n_shared", "moe_inter",
              "dense_inter", "first_k_dense", "scoring", "n_group", "topk_group", "max_position"):
        assert getattr(s, f) == getattr(c, f), f
    assert abs(s.routed_scale - c.routed_scale) < 1e-6 and abs(s.rope_theta - c.rope_theta) < 1e-3
    pr = probe(p)
    assert pr.kind == "gguf" and pr.shards == 1 and pr.shape.hidden == c.hidden and pr.quant["experts"] == "Q8_0"
    assert set(pr.quant["bytes_by_type"]) == {"F32", "Q8_0"} and pr.bytes_on_disk > 0 and not pr.has_tokenizer
    cfg, ck = open_checkpoint(p)                                 # no config.json beside the file
    assert cfg.n_routed == c.n_routed and "embed.weight" in ck


def test_gguf_without_shape_metadata_is_reported(tmp_path):
    gw = GgufWriter()
    gw.meta("general.architecture", "deepseek2")
    gw.add("token_embd.weight", np.zeros((4, 8), np.float32))
    p = str(tmp_path / "bare.gguf")
    gw.write(p)
    pr = probe(p)
    assert pr.shape is None and "lacks deepseek2.block_count" in pr.notes[0]
    with pytest.raises(ValueError):
        open_checkpoint(p)


def test_probe_hf_dir_prepacked_dir_and_preset(tmp_path):
    c = tiny_mla_moe()
    hf = tmp_path / "hf"
    hf.mkdir()
    raw = hf_config_dict(c)
    raw["quantization_config"] = {"quant_method": "fp8", "weight_block_size": [128, 128]}
    (hf / "config.json").write_text(json.dumps(raw))
    (hf / "tokenizer.json").write_text("{}")
    (hf / "model-00001-of-00002.safetensors").write_bytes(b"x" * 100)
    (hf / "model-00002-of-00002.safetensors").write_bytes(b"x" * 50)
    pr = probe(str(hf))
    assert pr.kind == "hf" and pr.shards == 2 and pr.bytes_on_disk == 150 and pr.has_tokenizer
    assert pr.quant == {"method": "fp8", "block": [128, 128]} and pr.shape.n_routed == c.n_routed
    assert probe(str(hf / "model-00001-of-00002.safetensors")).kind == "hf"
    (hf / "hf_quant_config.json").write_text(json.dumps({"quantization": {"quant_algo": "NVFP4", "kv_cache_quant_algo": "FP8"}}))
    assert probe(str(hf)).quant == {"method": "modelopt", "algo": "NVFP4", "kv": "FP8"}
    pp = tmp_path / "packed"
    (pp / "L003").mkdir(parents=True)
    (pp / "manifest.json").write_text(json.dumps({"version": "lsb200-prepack-1", "quant": "nvfp4", "hidden": 64, "moe_inter": 32, "stride": 4096}))
    (pp / "L003" / "expert_0001.bin").write_bytes(b"y" * 4096)
    pk = probe(str(pp))
    assert pk.kind == "prepacked" and pk.shards == 1 and pk.bytes_on_disk == 4096 and pk.quant["quant"] == "nvfp4" and pk.shape is None
    ps = probe("glm-5.3-flash") if "glm-5.3-flash" in __import__("layerstorm_b200.models.config", fromlist=["PRESETS"]).PRESETS else probe("tiny-mla-moe")
    assert ps.kind == "preset" and ps.shape is not None and json.dumps(ps.to_dict())
    with pytest.raises(FileNotFoundError):
        probe(str(tmp_path / "nope"))
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(ValueError):
        probe(str(empty))
