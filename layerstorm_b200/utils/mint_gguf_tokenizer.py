"""Mint a HuggingFace tokenizer directory from the vocabulary embedded in a GGUF file.

    python -m layerstorm_b200.utils.mint_gguf_tokenizer --gguf model.gguf [--out DIR] [--base HF_TOKENIZER_DIR] [--skip-validate]

Some checkpoints ship as a GGUF only: vocabulary, merges, token types, special ids and chat template sit in the file's metadata
(``tokenizer.ggml.*``, ``tokenizer.chat_template``), but the serving stack wants ``tokenizer.json`` + ``tokenizer_config.json``.  This
tool writes them (default: next to the GGUF, where ``serve --tokenizer-path auto`` looks):
  * model: byte-level BPE over the file's own tokens and merges (nothing is taken from elsewhere);
  * pipeline (normaliser / pre-tokeniser / decoder): copied from ``--base`` when a tokenizer of the same family is at hand (its
    vocabulary is ignored), else chosen by the file's ``tokenizer.ggml.pre`` name - the DeepSeek-V3 family's digit / CJK / word
    splitting regexes for ``deepseek-v3`` / ``deepseek3-llm`` / ``joyai-llm`` / ``glm4``, the GPT-2 regex otherwise - followed by the
    byte-level mapping;
  * control and user-defined tokens (token types 3 and 4) become added tokens, control ones flagged ``special``;
  * ``tokenizer_config.json``: bos / eos / pad tokens from the ids in the file, the chat template, the added-token table.
Validation (unless ``--skip-validate``): the minted tokenizer is loaded back; every special token must encode to its own id, and
a battery of texts (ASCII, digits, CJK, emoji, whitespace runs) must survive encode -> decode unchanged.
Reference: tools/mint_v4_hf_tokenizer.py (V4 tokenizer minted from the GGUF header with the V3.2 pipeline, parity battery).
"""
from __future__ import annotations

import argparse
import json
import os
from typing import Dict, List, Optional

# pre-tokeniser regex sets by the GGUF's ``tokenizer.ggml.pre`` name
_DEEPSEEK3 = [r"\p{N}{1,3}", r"[一-龥぀-ゟ゠-ヿ]+",
              r"[!\"#$%&'()*+,\-./:;<=>?@\[\\\]^_`{|}~][A-Za-z]+|[^\r\n\p{L}\p{P}\p{S}]?[\p{L}\p{M}]+| ?[\p{P}\p{S}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"]
_GPT2 = [r"'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"]
PRE_REGEX = {"deepseek-v3": _DEEPSEEK3, "deepseek3-llm": _DEEPSEEK3, "joyai-llm": _DEEPSEEK3, "glm4": _DEEPSEEK3, "default": _GPT2, "gpt-2": _GPT2}

TOKEN_NORMAL, TOKEN_UNKNOWN, TOKEN_CONTROL, TOKEN_USER, TOKEN_UNUSED, TOKEN_BYTE = 1, 2, 3, 4, 5, 6

BATTERY = ["Hello, world!", "  leading and   inner   spaces ", "1234567 + 89 = 1234656", "def f(x):\n\treturn x ** 2\n\n", "naïve café — “quotes”",
           "数学と日本語のテキスト", "emoji 🙂🚀 mix", "tabs\tand\r\nnewlines\n\n\nend", ""]


def read_gguf_vocab(path: str) -> dict:
    from ..formats.gguf import GgufReader
    r = GgufReader(path)
    model = r.meta("tokenizer.ggml.model", "gpt2")
    tokens = r.meta("tokenizer.ggml.tokens")
    if not tokens:
        raise ValueError(f"{path}: no tokenizer.ggml.tokens in the file's metadata")
    if model not in ("gpt2", "bpe"):
        raise ValueError(f"{path}: tokenizer model {model!r} is not byte-level BPE")
    out = {"tokens": [str(t) for t in tokens], "merges": [str(m) for m in (r.meta("tokenizer.ggml.merges") or [])],
           "types": [int(t) for t in (r.meta("tokenizer.ggml.token_type") or [])], "pre": r.meta("tokenizer.ggml.pre", "default"),
           "chat_template": r.meta("tokenizer.chat_template"), "arch": r.meta("general.architecture", "")}
    for k in ("bos_token_id", "eos_token_id", "padding_token_id", "unknown_token_id", "eot_token_id"):
        v = r.meta("tokenizer.ggml." + k)
        out[k] = int(v) if v is not None else None
    out["add_bos"] = bool(r.meta("tokenizer.ggml.add_bos_token", 0))
    r.close()
    return out


def build_tokenizer_json(v: dict, base: Optional[dict] = None) -> dict:
    tokens, types = v["tokens"], v["types"] or [TOKEN_NORMAL] * len(v["tokens"])
    vocab = {t: i for i, t in enumerate(tokens)}
    if len(vocab) != len(tokens):
        # duplicate surface forms (unused slots): keep the first id, later ids stay reachable as added tokens only if special
        vocab = {}
        for i, t in enumerate(tokens):
            vocab.setdefault(t, i)
    added = [{"id": i, "content": tokens[i], "single_word": False, "lstrip": False, "rstrip": False, "normalized": False,
              "special": types[i] == TOKEN_CONTROL} for i in range(len(tokens)) if types[i] in (TOKEN_CONTROL, TOKEN_USER)]
    if base is not None:
        normalizer, pre, decoder, post = base.get("normalizer"), base.get("pre_tokenizer"), base.get("decoder"), base.get("post_processor")
    else:
        regs = PRE_REGEX.get(v["pre"], _GPT2)
        pre = {"type": "Sequence", "pretokenizers": [{"type": "Split", "pattern": {"Regex": rx}, "behavior": "Isolated", "invert": False} for rx in regs]
               + [{"type": "ByteLevel", "add_prefix_space": False, "trim_offsets": True, "use_regex": False}]}
        normalizer, post = None, {"type": "ByteLevel", "add_prefix_space": True, "trim_offsets": False, "use_regex": True}
        decoder = {"type": "ByteLevel", "add_prefix_space": True, "trim_offsets": True, "use_regex": True}
    merges = [m.split(" ", 1) for m in v["merges"]]
    return {"version": "1.0", "truncation": None, "padding": None, "added_tokens": added, "normalizer": normalizer, "pre_tokenizer": pre,
            "post_processor": post, "decoder": decoder,
            "model": {"type": "BPE", "dropout": None, "unk_token": None, "continuing_subword_prefix": None, "end_of_word_suffix": None,
                      "fuse_unk": False, "byte_fallback": False, "ignore_merges": False, "vocab": vocab, "merges": merges}}


def build_tokenizer_config(v: dict, tj: dict) -> dict:
    tok = v["tokens"]
    name = lambda i: tok[i] if i is not None and 0 <= i < len(tok) else None
    cfg = {"add_bos_token": v["add_bos"], "add_eos_token": False, "clean_up_tokenization_spaces": False, "model_max_length": 1 << 20,
           "tokenizer_class": "PreTrainedTokenizerFast", "bos_token": name(v["bos_token_id"]), "eos_token": name(v["eos_token_id"]),
           "pad_token": name(v["padding_token_id"]) or name(v["eos_token_id"]), "unk_token": name(v["unknown_token_id"]),
           "added_tokens_decoder": {str(a["id"]): {k: a[k] for k in ("content", "lstrip", "normalized", "rstrip", "single_word", "special")}
                                    for a in tj["added_tokens"]}}
    if v["chat_template"]:
        cfg["chat_template"] = v["chat_template"]
    return cfg


def validate(out_dir: str, v: dict) -> List[str]:
    """Problems found when the minted tokenizer is loaded back (empty = fine)."""
    from tokenizers import Tokenizer
    t = Tokenizer.from_file(os.path.join(out_dir, "tokenizer.json"))
    bad = []
    types = v["types"] or []
    for i, ty in enumerate(types):
        if ty == TOKEN_CONTROL:
            ids = t.encode(v["tokens"][i], add_special_tokens=False).ids
            if ids != [i]:
                bad.append(f"special token {v['tokens'][i]!r} encodes to {ids}, not [{i}]")
    for text in BATTERY:
        ids = t.encode(text, add_special_tokens=False).ids
        back = t.decode(ids, skip_special_tokens=False)
        if back != text:
            bad.append(f"round trip changed {text!r} -> {back!r}")
    if t.get_vocab_size(with_added_tokens=True) < len(set(v["tokens"])):
        bad.append("vocabulary smaller than the file's token list")
    return bad


def mint(gguf: str, out_dir: Optional[str] = None, base_dir: Optional[str] = None, skip_validate: bool = False) -> Dict:
    v = read_gguf_vocab(gguf)
    out_dir = out_dir or os.path.dirname(os.path.abspath(gguf))
    os.makedirs(out_dir, exist_ok=True)
    base = json.load(open(os.path.join(base_dir, "tokenizer.json"))) if base_dir else None
    tj = build_tokenizer_json(v, base)
    json.dump(tj, open(os.path.join(out_dir, "tokenizer.json"), "w"), ensure_ascii=False)
    json.dump(build_tokenizer_config(v, tj), open(os.path.join(out_dir, "tokenizer_config.json"), "w"), ensure_ascii=False, indent=1)
    eos = [i for i in (v["eos_token_id"], v["eot_token_id"]) if i is not None]
    if eos:
        json.dump({"eos_token_id": sorted(set(eos)), "bos_token_id": v["bos_token_id"]}, open(os.path.join(out_dir, "generation_config.json"), "w"))
    rep = {"out": out_dir, "tokens": len(v["tokens"]), "merges": len(v["merges"]), "added_tokens": len(tj["added_tokens"]), "pre": v["pre"],
           "pipeline": "base tokenizer" if base else f"regex set {v['pre'] if v['pre'] in PRE_REGEX else 'gpt-2 (unknown pre name)'}",
           "chat_template": bool(v["chat_template"]), "problems": [] if skip_validate else validate(out_dir, v)}
    return rep


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gguf", required=True)
    ap.add_argument("--out", default=None, help="output directory (default: the GGUF's directory)")
    ap.add_argument("--base", default=None, help="HuggingFace tokenizer directory of the same family: its normaliser / pre-tokeniser / decoder are reused")
    ap.add_argument("--skip-validate", action="store_true")
    a = ap.parse_args(argv)
    rep = mint(a.gguf, a.out, a.base, a.skip_validate)
    print(json.dumps(rep, ensure_ascii=False))
    return 1 if rep["problems"] else 0


if __name__ == "__main__":
    raise SystemExit(main())
