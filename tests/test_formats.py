"""Checkpoint container and codec tests (CPU)."""
import numpy as np
import pytest
import torch

from layerstorm_b200 import build as _build

_build.build_all(only="runtime")

from layerstorm_b200.formats import gguf, quant, safetensors as st


@pytest.mark.parametrize("tname,tol", [("F32", 0.0), ("F16", 1e-3), ("BF16", 8e-3), ("Q8_0", 1e-2), ("Q6_K", 3e-2), ("Q4_K", 0.12)])
def test_ggml_quant_roundtrip(tname, tol):
    t = gguf.GGML_TYPES[tname]
    x = np.random.default_rng(0).standard_normal(4 * 256).astype(np.float32)
    raw = gguf.quantize(t, x)
    assert raw.size == gguf.nbytes_for(t, x.size)
    y = gguf.dequantize(t, raw, x.size)
    assert np.max(np.abs(x - y)) <= tol * np.max(np.abs(x)) + 1e-7


def test_block_sizes_match_spec():
    spec = {"Q2_K": (256, 84), "Q3_K": (256, 110), "Q4_K": (256, 144), "Q5_K": (256, 176), "Q6_K": (256, 210), "Q8_0": (32, 34), "MXFP4": (32, 17)}
    for k, (e, b) in spec.items():
        assert gguf.block_elems(gguf.GGML_TYPES[k]) == e and gguf.block_bytes(gguf.GGML_TYPES[k]) == b


def test_hand_built_blocks_decode():
    # Q5_K: d=1, dmin=0, all sub-scales 1, nibble 3 with the high bit set in the second half of each 64
    blk = np.zeros(176, dtype=np.uint8)
    blk[0:2] = np.frombuffer(np.float16(1.0).tobytes(), dtype=np.uint8)
    blk[4:8] = 1          # scales for sub-blocks 0..3 (6-bit), mins stay 0
    blk[12:16] = 1        # scales for sub-blocks 4..7 live in the low nibbles of bytes 8..11 of the 12-byte field
    blk[48:176] = 0x33
    blk[16:48] = 0xAA     # high bits: odd sub-blocks (u2) set
    y = gguf.dequantize(gguf.GGML_TYPES["Q5_K"], blk, 256)
    assert np.all(y[:32] == 3) and np.all(y[32:64] == 19)
    # MXFP4: scale byte 128 -> 2^1, nibbles (1, 2) -> 0.5*2, 1.0*2
    m = np.zeros(17, dtype=np.uint8); m[0] = 128; m[1:] = 0x21
    y = gguf.dequantize(gguf.GGML_TYPES["MXFP4"], m, 32)
    assert np.all(y[:16] == 1.0) and np.all(y[16:] == 2.0)
    # Q2_K / Q3_K decode without error and stay finite
    for name in ("Q2_K", "Q3_K"):
        raw = np.random.default_rng(1).integers(0, 255, gguf.block_bytes(gguf.GGML_TYPES[name]), dtype=np.uint8)
        raw[-2:] = np.frombuffer(np.float16(0.5).tobytes(), dtype=np.uint8)
        if name == "Q2_K":
            raw[-4:-2] = np.frombuffer(np.float16(0.25).tobytes(), dtype=np.uint8)
        assert np.all(np.isfinite(gguf.dequantize(gguf.GGML_TYPES[name], raw, 256)))


def test_gguf_container_roundtrip(tmp_path):
    w = gguf.GgufWriter()
    w.meta("general.architecture", "glm5_next")
    w.meta("glm5_next.block_count", 45)
    w.meta("glm5_next.attention.layer_norm_rms_epsilon", 1e-5)
    a = np.random.default_rng(2).standard_normal((8, 512)).astype(np.float32)
    b = np.random.default_rng(3).standard_normal((16,)).astype(np.float32)
    w.add("blk.0.ffn_gate_exps.weight", a, gguf.GGML_TYPES["Q4_K"])
    w.add("blk.0.attn_norm.weight", b, gguf.GGML_TYPES["F32"])
    p = str(tmp_path / "m.gguf")
    w.write(p)
    r = gguf.GgufReader(p)
    assert r.version == 3 and r.meta("general.architecture") == "glm5_next" and r.meta("glm5_next.block_count") == 45
    assert abs(r.meta("glm5_next.attention.layer_norm_rms_epsilon") - 1e-5) < 1e-9
    assert r.tensors["blk.0.ffn_gate_exps.weight"]["shape"] == (8, 512)
    assert np.array_equal(r.get("blk.0.attn_norm.weight"), b)
    assert np.max(np.abs(r.get("blk.0.ffn_gate_exps.weight") - a)) < 0.15 * np.max(np.abs(a))
    with pytest.raises(Exception):
        (tmp_path / "bad.gguf").write_bytes(b"NOPE" + b"\0" * 64)
        gguf.GgufReader(str(tmp_path / "bad.gguf"))


def test_safetensors_roundtrip_incl_nvfp4_quartet(tmp_path):
    w = torch.randn(128, 64)
    packed, atoms, gs = quant.quantize_nvfp4(w)
    q8, sc = quant.quantize_fp8_block(w)
    tensors = {"e.weight": packed, "e.weight_scale": atoms, "e.weight_scale_2": torch.tensor([gs]), "e.input_scale": torch.tensor([1.0]),
               "a.weight": q8.view(torch.float8_e4m3fn), "a.weight_scale_inv": sc, "n.weight": torch.randn(7).to(torch.bfloat16)}
    p = str(tmp_path / "m.safetensors")
    st.write_safetensors(p, tensors, {"format": "pt"})
    r = st.SafetensorsReader(p)
    assert set(r.keys()) == set(tensors) and r.metadata["format"] == "pt"
    for k, v in tensors.items():
        got = r.get(k)
        assert got.dtype == v.dtype and got.shape == v.shape and torch.equal(got.view(torch.uint8), v.view(torch.uint8))
    d = quant.dequantize_nvfp4(r.get("e.weight"), r.get("e.weight_scale"), float(r.get("e.weight_scale_2")), 128, 64)
    assert (d - w).abs().max() < 0.3 * w.abs().max()
    assert (quant.dequantize_fp8_block(r.get("a.weight").view(torch.uint8), r.get("a.weight_scale_inv")) - w).abs().max() < 0.07 * w.abs().max()
    r.close()


def test_prepacked_store_roundtrip_resume_and_verify(tmp_path):
    import os
    import torch
    from layerstorm_b200.formats.prepacked import PrepackedSource, PrepackWriter, load_experts, prepack_model
    from layerstorm_b200.models.checkpoint import export_hf
    from layerstorm_b200.models.config import get_preset
    from layerstorm_b200.models.device_model import ExpertArena, QLinear, expert_layout
    from layerstorm_b200.models.weights import init_weights, round_weights_bf16
    cfg = get_preset("tiny-mla-moe")
    w = round_weights_bf16(init_weights(cfg, 4))
    d = str(tmp_path / "store")
    wr = prepack_model(cfg, w, d, "nvfp4")
    n_exp = cfg.n_moe_layers() * (cfg.n_routed + cfg.n_shared)
    assert wr.written == n_exp and wr.skipped == 0
    wr2 = prepack_model(cfg, w, d, "nvfp4")                     # resume: nothing to do
    assert wr2.written == 0 and wr2.skipped == n_exp
    src = PrepackedSource(d, mode="pread")
    src.check_shape(cfg, "nvfp4")
    assert src.verify_all() == (n_exp, 0)
    # the image is byte-identical to what the arena writer produces
    ef = expert_layout("nvfp4", cfg.hidden, cfg.moe_inter)
    ar = ExpertArena(ef, 1, 1, "cpu")
    ar.data.zero_()
    nm = "layers.2.moe.experts.5."
    ar.write_expert(0, *(QLinear.from_float(w[nm + t], "nvfp4", "cpu") for t in ("gate", "up", "down")))
    buf = torch.empty(src.stride, dtype=torch.uint8)
    for mode in ("mmap", "pread", "direct"):
        PrepackedSource(d, mode=mode).read_into(2, 5, buf, verify=True)
        assert torch.equal(buf, ar.data[0])
    # corruption is detected
    p = src.path(1, 0)
    raw = bytearray(open(p, "rb").read())
    raw[100] ^= 0xFF
    open(p, "wb").write(raw)
    assert PrepackedSource(d).verify_all() == (n_exp, 1)
    # CLI on an exported checkpoint
    from layerstorm_b200.cli import prepack
    hf = str(tmp_path / "hf")
    export_hf(cfg, w, hf)
    assert prepack.main(["--model", hf, "--out", str(tmp_path / "s2"), "--quant", "fp8_e4m3", "--verify"]) == 0
    assert os.path.exists(tmp_path / "s2" / "manifest.json")


def test_gguf_device_layouts_hold_the_file_blocks_unchanged():
    """Q6_K blocks padded to 224 bytes and Q8_0 rows split into a quant plane and a scale plane give back the file's bytes."""
    import numpy as np
    from layerstorm_b200.formats import gguf as g
    rng = np.random.default_rng(0)
    x = rng.standard_normal((6, 512)).astype(np.float32)
    for t in (g.GGML_TYPES["Q4_K"], g.GGML_TYPES["Q6_K"], g.GGML_TYPES["Q8_0"]):
        raw = g.quantize(t, x)
        d = g.to_device_layout(t, raw, 6, 512)
        assert d.shape == (6, g.device_row_bytes(t, 512))
        assert np.array_equal(g.from_device_layout(t, d, 6, 512), raw)
    assert g.device_row_bytes(g.GGML_TYPES["Q5_K"], 512) == 2 * 176


def test_tokenizer_directory_minted_from_a_gguf_vocabulary(tmp_path):
    """A GGUF that carries its vocabulary, merges, token types, special ids and chat template -> tokenizer.json / tokenizer_config.json
    that the serving tokenizer wrapper loads: same ids as the tokenizer the vocabulary came from, specials by id, texts round-trip."""
    import json
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers
    from layerstorm_b200.formats.gguf import GgufWriter
    from layerstorm_b200.serving.tokenizer import TokenizerWrapper, resolve_tokenizer_dir
    from layerstorm_b200.utils import mint_gguf_tokenizer as mint
    # a small byte-level BPE trained here stands in for a model's vocabulary
    src = Tokenizer(models.BPE())
    src.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
    src.decoder = decoders.ByteLevel()
    corpus = ["the quick brown fox jumps over the lazy dog " * 5, "hello world, hello tokens; numbers 12345 and 678", "def f(x):\n    return x + 1\n"] * 20
    tr = trainers.BpeTrainer(vocab_size=400, initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), special_tokens=[])
    src.train_from_iterator(corpus, tr)
    vocab = src.get_vocab()
    tokens = [t for t, _ in sorted(vocab.items(), key=lambda kv: kv[1])]
    merges = [" ".join(m) for m in json.loads(src.to_str())["model"]["merges"]]
    specials = ["<|bos|>", "<|eos|>", "<think>", "</think>"]
    types = [1] * len(tokens) + [3, 3, 4, 3]
    tokens += specials
    gw = GgufWriter()
    gw.meta("general.architecture", "deepseek2")
    gw.meta("tokenizer.ggml.model", "gpt2")
    gw.meta("tokenizer.ggml.pre", "default")
    gw.meta("tokenizer.ggml.tokens", tokens)
    gw.meta("tokenizer.ggml.merges", merges)
    gw.meta("tokenizer.ggml.token_type", types)
    gw.meta("tokenizer.ggml.bos_token_id", len(tokens) - 4)
    gw.meta("tokenizer.ggml.eos_token_id", len(tokens) - 3)
    gw.meta("tokenizer.chat_template", "{% for m in messages %}{{ m.content }}{% endfor %}")
    gw.add("token_embd.weight", np.zeros((4, 8), np.float32))
    path = str(tmp_path / "m.gguf")
    gw.write(path)
    rep = mint.mint(path)
    assert rep["problems"] == [] and rep["tokens"] == len(tokens) and rep["added_tokens"] == 4 and rep["chat_template"]
    assert resolve_tokenizer_dir("auto", path) == str(tmp_path)
    tw = TokenizerWrapper(str(tmp_path))
    assert tw.special == {"<|bos|>": len(tokens) - 4, "<|eos|>": len(tokens) - 3, "</think>": len(tokens) - 1}      # control tokens; <think> is user-defined
    assert tw.eos_token_ids == [len(tokens) - 3] and tw.chat_template.startswith("{% for")
    for text in ["hello world 12345", "the lazy dog\n\treturn x", "unseen: Ünïcödé 🙂"]:
        ids = tw.encode(text)
        assert tw.decode(ids, skip_special_tokens=False) == text
    # plain words tokenise as in the tokenizer the vocabulary came from (same merges, same byte-level alphabet)
    assert tw.encode("hello world") == src.encode("hello world").ids
    assert tw.encode("a<think>b</think>") [1] == len(tokens) - 2
    # the command line: exit code 0 and a JSON report
    assert mint.main(["--gguf", path, "--out", str(tmp_path / "o")]) == 0 and (tmp_path / "o" / "tokenizer.json").exists()


def test_fp8_block_scales_are_powers_of_two_and_become_scale_atoms():
    """The FP8 block quantiser writes power-of-two scales by default (UE8M0 convention), which the block-scaled tensor-core path
    turns into one 512-byte atom per 128 x 128 block; a scale with a mantissa has no such form."""
    from layerstorm_b200.models.device_model import fp8_scale_atoms
    g = torch.Generator().manual_seed(0)
    w = torch.randn(256, 384, generator=g) * torch.rand(256, 1, generator=g) * 3
    q8, s = quant.quantize_fp8_block(w)
    assert s.shape == (2, 3)
    m, e = torch.frexp(s)
    assert torch.all(m == 0.5)                                              # exact powers of two
    back = quant.dequantize_fp8_block(q8, s)
    assert float((back - w).norm() / w.norm()) < 0.04                       # E4M3 relative precision, whatever the scale's rounding
    assert float(back.abs().max()) <= float(w.abs().max()) * 1.07
    atoms = fp8_scale_atoms(s)
    assert atoms.shape == (6, 512) and atoms.dtype == torch.uint8
    want = (torch.log2(s).round().to(torch.int32) + 127).to(torch.uint8).reshape(-1)
    assert torch.equal(atoms[:, 0], want) and bool((atoms == atoms[:, :1]).all())
    # stacked (per expert slot) scales keep their leading dimensions
    assert fp8_scale_atoms(torch.stack([s, s * 2])).shape == (2, 6, 512)
    q8b, sb = quant.quantize_fp8_block(w, pow2=False)
    assert fp8_scale_atoms(sb) is None and fp8_scale_atoms(torch.zeros(1, 1)) is None
    assert float((quant.dequantize_fp8_block(q8b, sb) - w).norm() / w.norm()) < 0.04
