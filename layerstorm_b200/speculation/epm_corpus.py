"""Corpus recorder for expert-routing prediction: what the block draft knew, against what the target then routed.

A model that predicts, from the DRAFT's hidden states, which experts the TARGET will route the drafted positions to could fetch
those experts while the draft is still being verified.  Training it needs pairs of (draft features, target routing); this module
writes them during ordinary serving and reads them back:

  ``blocks.bin``    one record per block pass: sequence, block number, anchor position and token, the proposed ids, the confidence
                    head's per-row probabilities when it ran, and the draft's residual stream after EVERY draft layer for the
                    predicting rows ([gamma, L, H], bf16 bits) - the feature side;
  ``routing.bin``   one record per (sequence, token position) the target ran: for every routed layer the router's logits over all
                    experts (fp16) and the chosen experts with their weights - the label side;
  ``manifest.jsonl`` one line per verified block: how many proposed tokens the target accepted and which tokens were committed; and one
                    line per drafted block with the tokens the sequence gained since its last block, so that the sequences can be
                    re-run offline (:func:`label_with_oracle` writes the label side that way when it was not recorded live).
Records are little-endian, length-prefixed (a reader can skip a record type or version it does not know), appended - several runs
accumulate into one directory - and joined on (sequence, position) by :func:`join_examples`.  Writing never takes serving down: an
I/O error switches the writer off and is logged once.

Layout of a record: ``u32 magic, u32 version, u32 payload_bytes`` + payload.
  block payload  : u64 seq, u32 block, u32 anchor_pos, u32 anchor_token, u32 gamma, u32 layers, u32 hidden, u32 has_conf,
                   i32 ids[gamma], f32 conf[gamma] (if has_conf), u16 hiddens[gamma * layers * hidden]
  routing payload: u64 seq, u32 pos, u32 rows, u32 experts, u32 topk, rows x { u32 layer, f16 logits[experts], i32 ids[topk], f32 w[topk] }
Switch: ``speculation.dspark.epm_dump_dir``; the environment variable ``LS_EPM_DUMP`` overrides it (``0`` = off).
Reference: src/speculation/epm_dump.h (the two record streams and their fail-soft writers), python/orchestrator/epm_manifest.py.
"""
from __future__ import annotations

import json
import logging
import os
import struct
from typing import Dict, Iterator, List, Optional, Sequence, Tuple

import numpy as np
import torch

log = logging.getLogger("layerstorm_b200.epm")

BLOCK_MAGIC = 0x4B4C4245          # "EBLK"
ROUTE_MAGIC = 0x54524545          # "EERT"
VERSION = 1
_HEAD = struct.Struct("<III")
_BLOCK = struct.Struct("<QIIIIIII")
_ROUTE = struct.Struct("<QIIII")


def effective_dump_dir(configured: str = "", env: Optional[dict] = None) -> str:
    """The directory in effect: ``LS_EPM_DUMP`` wins when set (``0`` switches dumping off), else the configured one; "" = off."""
    e = (os.environ if env is None else env).get("LS_EPM_DUMP")
    if e is not None and e != "":
        return "" if e == "0" else e
    return configured or ""


class CorpusWriter:
    def __init__(self, directory: str):
        self.dir = directory
        self.ok = True
        self._files: Dict[str, object] = {}
        self.blocks = self.routes = self.manifest_lines = 0
        try:
            os.makedirs(directory, exist_ok=True)
            for name, mode in (("blocks.bin", "ab"), ("routing.bin", "ab"), ("manifest.jsonl", "a")):
                self._files[name] = open(os.path.join(directory, name), mode)
        except OSError as e:
            self._fail(e)

    def _fail(self, e: Exception):
        if self.ok:
            log.error("expert-routing corpus dump switched off: %s", e)
        self.ok = False
        self.close()

    def close(self):
        for f in self._files.values():
            try:
                f.close()
            except OSError:
                pass
        self._files = {}

    def _append(self, name: str, data):
        if not self.ok:
            return False
        try:
            f = self._files[name]
            f.write(data)
            f.flush()
            return True
        except (OSError, KeyError, ValueError) as e:
            self._fail(e)
            return False

    def write_block(self, seq: int, block: int, anchor_pos: int, anchor_token: int, ids: Sequence[int], conf: Optional[Sequence[float]],
                    hiddens: torch.Tensor):
        """``hiddens`` [gamma, layers, hidden]: the draft's residual stream after each layer for the predicting rows."""
        g, L, H = hiddens.shape
        if g != len(ids):
            raise ValueError(f"{len(ids)} proposed ids against {g} rows of hidden states")
        has_conf = conf is not None and len(conf) >= g
        bits = hiddens.detach().to(torch.bfloat16).contiguous().cpu().view(torch.int16).numpy().astype("<i2", copy=False)
        body = _BLOCK.pack(int(seq), int(block), int(anchor_pos), int(anchor_token), g, L, H, 1 if has_conf else 0)
        body += np.asarray(list(ids), "<i4").tobytes()
        if has_conf:
            body += np.asarray(list(conf)[:g], "<f4").tobytes()
        body += bits.tobytes()
        if self._append("blocks.bin", _HEAD.pack(BLOCK_MAGIC, VERSION, len(body)) + body):
            self.blocks += 1

    def write_routing(self, seq: int, pos: int, rows: Sequence[Tuple[int, Sequence[float], Sequence[int], Sequence[float]]]):
        """``rows``: (layer, router logits over all experts, chosen expert ids, their weights) for every routed layer of one position."""
        if not rows:
            return
        E, K = len(rows[0][1]), len(rows[0][2])
        body = _ROUTE.pack(int(seq), int(pos), len(rows), E, K)
        for layer, logits, ids, w in rows:
            if len(logits) != E or len(ids) != K or len(w) != K:
                raise ValueError("routing rows of one position must share the expert count and top-k")
            body += struct.pack("<I", int(layer)) + np.asarray(logits, "<f2").tobytes() + np.asarray(ids, "<i4").tobytes() + np.asarray(w, "<f4").tobytes()
        if self._append("routing.bin", _HEAD.pack(ROUTE_MAGIC, VERSION, len(body)) + body):
            self.routes += 1

    def write_manifest(self, seq: int, block: int, anchor_pos: int, proposed: int, accepted: int, committed: Sequence[int], conf: Optional[Sequence[float]] = None):
        line = {"seq": int(seq), "block": int(block), "anchor_pos": int(anchor_pos), "proposed": int(proposed), "accepted": int(accepted),
                "committed": [int(t) for t in committed]}
        if conf:
            line["conf"] = [round(float(c), 6) for c in conf]
        if self._append("manifest.jsonl", json.dumps(line) + "\n"):
            self.manifest_lines += 1


    def write_context(self, seq: int, block: int, start: int, tokens: Sequence[int]):
        """The tokens at positions ``start ..`` that the sequence held when block ``block`` was drafted (the anchor is the last one)."""
        self._append("manifest.jsonl", json.dumps({"seq": int(seq), "block": int(block), "context_from": int(start), "tokens": [int(t) for t in tokens]}) + "\n")


def _records(path: str, magic: int) -> Iterator[bytes]:
    if not os.path.exists(path):
        return
    with open(path, "rb") as f:
        while True:
            head = f.read(_HEAD.size)
            if len(head) < _HEAD.size:
                return
            m, ver, n = _HEAD.unpack(head)
            body = f.read(n)
            if len(body) < n:
                return                                   # a record cut off by a crash: everything before it stands
            if m == magic and ver == VERSION:
                yield body


def read_blocks(directory: str) -> List[dict]:
    out = []
    for body in _records(os.path.join(directory, "blocks.bin"), BLOCK_MAGIC):
        seq, block, apos, atok, g, L, H, has_conf = _BLOCK.unpack_from(body)
        o = _BLOCK.size
        ids = np.frombuffer(body, "<i4", g, o)
        o += 4 * g
        conf = None
        if has_conf:
            conf = np.frombuffer(body, "<f4", g, o)
            o += 4 * g
        bits = np.frombuffer(body, "<i2", g * L * H, o).copy()
        hid = torch.from_numpy(bits).view(torch.bfloat16).view(g, L, H)
        out.append({"seq": seq, "block": block, "anchor_pos": apos, "anchor_token": atok, "ids": ids.tolist(), "conf": None if conf is None else conf.tolist(),
                    "hiddens": hid})
    return out


def read_routing(directory: str) -> List[dict]:
    out = []
    for body in _records(os.path.join(directory, "routing.bin"), ROUTE_MAGIC):
        seq, pos, n, E, K = _ROUTE.unpack_from(body)
        o = _ROUTE.size
        rows = []
        for _ in range(n):
            (layer,) = struct.unpack_from("<I", body, o)
            o += 4
            logits = np.frombuffer(body, "<f2", E, o).astype(np.float32)
            o += 2 * E
            ids = np.frombuffer(body, "<i4", K, o)
            o += 4 * K
            w = np.frombuffer(body, "<f4", K, o)
            o += 4 * K
            rows.append({"layer": layer, "logits": logits, "ids": ids.tolist(), "weights": w.tolist()})
        out.append({"seq": seq, "pos": pos, "rows": rows})
    return out


def read_manifest(directory: str, contexts: bool = False) -> List[dict]:
    """The verdict lines of the manifest (``contexts``: the context lines instead)."""
    p = os.path.join(directory, "manifest.jsonl")
    if not os.path.exists(p):
        return []
    out = []
    for line in open(p):
        line = line.strip()
        if line:
            try:
                rec = json.loads(line)
            except ValueError:
                break                                    # a line cut off by a crash
            if ("context_from" in rec) == contexts:
                out.append(rec)
    return out


def sequences_of(directory: str) -> Dict[int, List[int]]:
    """Every recorded sequence's tokens as far as the corpus knows them: the contexts written at each block, plus the tokens the last
    block's verdict committed."""
    toks: Dict[int, List[int]] = {}
    for c in read_manifest(directory, contexts=True):
        t = toks.setdefault(c["seq"], [])
        if c["block"] == 0:
            del t[:]
        if c["context_from"] <= len(t):
            del t[c["context_from"]:]
            t.extend(c["tokens"])
    last: Dict[int, dict] = {}
    for m in read_manifest(directory):
        if m["seq"] not in last or m["block"] >= last[m["seq"]]["block"]:
            last[m["seq"]] = m
    for seq, m in last.items():
        t = toks.get(seq)
        if t is not None and len(t) == m["anchor_pos"] + 1:
            t.extend(m["committed"])
    return toks


def label_with_oracle(directory: str, oracle) -> int:
    """Write the routing records of a corpus whose label side is missing (recorded beside the GPU engine) by re-running the recorded
    sequences through the fp32 reference model: exact, and as slow as that model - a tool for small targets.  Returns the number of
    positions labelled."""
    firsts: Dict[int, int] = {}
    for b in read_blocks(directory):
        firsts[b["seq"]] = min(firsts.get(b["seq"], b["anchor_pos"]), b["anchor_pos"])
    wr = CorpusWriter(directory)
    n = 0
    try:
        for seq, tokens in sorted(sequences_of(directory).items()):
            if seq in firsts and tokens:
                first = max(0, firsts[seq] - 1)
                record_oracle_routing(wr, oracle, seq, tokens, first)
                n += len(tokens) - first
    finally:
        wr.close()
    return n


def join_examples(directory: str, accepted_only: bool = True) -> List[dict]:
    """Training examples: for block row k (the draft's guess for position anchor_pos + 1 + k) the draft features of that row and the
    target's routing AT that position.  ``accepted_only``: keep the rows whose guess the target accepted - only there did the target
    run the position with the token the draft had in mind; the first rejected row is kept too (its position was run with the target's
    own token: a harder, still valid example) and marked ``accepted = False``."""
    routing = {(r["seq"], r["pos"]): r["rows"] for r in read_routing(directory)}          # a later record of a position replaces an earlier one
    verdict = {(m["seq"], m["block"]): m for m in read_manifest(directory)}
    out = []
    for b in read_blocks(directory):
        m = verdict.get((b["seq"], b["block"]))
        if m is None:
            continue
        for k in range(len(b["ids"])):
            acc = k < m["accepted"]
            if accepted_only and k > m["accepted"]:
                break
            rows = routing.get((b["seq"], b["anchor_pos"] + 1 + k))
            if rows is None:
                continue
            out.append({"seq": b["seq"], "pos": b["anchor_pos"] + 1 + k, "row": k, "accepted": acc, "draft_token": b["ids"][k], "features": b["hiddens"][k],
                        "labels": {r["layer"]: r["ids"] for r in rows}, "logits": {r["layer"]: r["logits"] for r in rows}})
    return out


def previous_position_coverage(directory: str) -> Dict[str, float]:
    """The zero-training bar a predictor has to beat: which share of a position's routed experts were also routed, in the same layer, at
    the position before it (per sequence), overall and per layer."""
    by_seq: Dict[int, Dict[int, list]] = {}
    for r in read_routing(directory):
        by_seq.setdefault(r["seq"], {})[r["pos"]] = r["rows"]
    hit = tot = 0
    per_layer: Dict[int, List[int]] = {}
    for poss in by_seq.values():
        for pos, rows in poss.items():
            prev = poss.get(pos - 1)
            if prev is None:
                continue
            before = {r["layer"]: set(r["ids"]) for r in prev}
            for r in rows:
                if r["layer"] not in before:
                    continue
                h = len(set(r["ids"]) & before[r["layer"]])
                hit += h
                tot += len(r["ids"])
                c = per_layer.setdefault(r["layer"], [0, 0])
                c[0] += h
                c[1] += len(r["ids"])
    return {"coverage": hit / tot if tot else 0.0, "pairs": tot, **{f"layer_{l}": c[0] / c[1] for l, c in sorted(per_layer.items()) if c[1]}}


def record_oracle_routing(writer: CorpusWriter, oracle, seq: int, tokens: Sequence[int], first: int = 0):
    """The label side from the fp32 reference model (the CPU engine's model): one routing record per position ``first ..`` of ``tokens``
    with every routed layer's logits, experts and weights."""
    oracle.route_log = {}
    try:
        oracle.forward(torch.tensor([int(t) for t in tokens]))
        log_ = oracle.route_log
    finally:
        oracle.route_log = None
    for pos in range(first, len(tokens)):
        writer.write_routing(seq, pos, [(layer, lg[pos].tolist(), ids[pos].tolist(), w[pos].tolist()) for layer, (lg, ids, w) in sorted(log_.items())])
