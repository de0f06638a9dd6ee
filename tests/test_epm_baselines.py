"""Baselines over an expert-routing prediction corpus (utils/epm_baselines.py) on a synthetic corpus with a known structure."""
import json

import numpy as np
import pytest
import torch

from layerstorm_b200.speculation import epm_corpus as ec
from layerstorm_b200.utils import epm_baselines as eb

E, K, H, TAPS, LAYERS = 16, 2, 8, 2, (1, 3)


def _corpus(directory, n_seq=8, blocks=5, gamma=3, seed=0):
    """Layer 1 routes every position to the same two experts (pure locality); layer 3's router logits are a fixed linear map of the
    draft's hidden row after its SECOND layer (so a probe through the target's router reads them off tap 1, and nothing off tap 0)."""
    g = np.random.default_rng(seed)
    W = {l: g.standard_normal((E, H)).astype(np.float32) for l in LAYERS}
    wr = ec.CorpusWriter(directory)
    for s in range(1, n_seq + 1):
        pos = 10
        wr.write_routing(s, pos - 1, _rows(g.standard_normal((TAPS, H)).astype(np.float32), W))       # the position before the first anchor
        carry = None
        for b in range(blocks):
            feats = g.standard_normal((gamma, TAPS, H)).astype(np.float32)
            feats = torch.from_numpy(feats).to(torch.bfloat16).float().numpy()                          # what the corpus can hold exactly
            accepted = int(g.integers(0, gamma + 1))
            wr.write_block(s, b, pos, 5, [7] * gamma, [0.5] * gamma, torch.from_numpy(feats))
            wr.write_manifest(s, b, pos, gamma, accepted, [7] * accepted)
            # the anchor's position is the one the previous block's first rejected row sat at: the target ran it with its own token
            wr.write_routing(s, pos, _rows(carry if carry is not None else g.standard_normal((TAPS, H)).astype(np.float32), W))
            for k in range(accepted):
                wr.write_routing(s, pos + 1 + k, _rows(feats[k], W))
            carry = feats[accepted] if accepted < gamma else None
            pos += accepted + 1
        if carry is not None:
            wr.write_routing(s, pos, _rows(carry, W))
    wr.close()
    return W


def _rows(feat, W):
    rows = []
    for l in LAYERS:
        logits = feat[1] @ W[l].T
        ids = [2, 9] if l == 1 else np.argsort(-logits)[:K].tolist()
        rows.append((l, logits.tolist(), ids, [0.6, 0.4]))
    return rows


def test_baselines_find_the_structure_that_was_put_into_the_corpus(tmp_path, capsys):
    d = str(tmp_path / "corpus")
    W = _corpus(d)
    weights = {f"layers.{l}.moe.router": torch.from_numpy(W[l]) for l in LAYERS}
    rep = eb.evaluate(d, weights, holdout=0.25, lam=1e-3, widths=(2, 4), sigmoid_scores=False)
    assert rep["sequences"] == 8 and rep["top_k"] == 2 and not rep["in_sample"] and rep["train_examples"] > rep["heldout_examples"] > 0
    # locality: layer 1 never changes its experts, layer 3 follows fresh features (chance level: 2 of 16)
    lp = rep["locality_prev"]["recall@2"]["by_layer"]
    assert lp["1"]["recall"] == 1.0 and lp["3"]["recall"] < 0.5 and rep["locality_block_start"]["recall@2"]["by_layer"]["1"]["recall"] == 1.0
    assert rep["locality_prev"]["missing_predictions"] == 0
    # the router probe reads layer 3 off the draft's second layer exactly; layer 1's constant experts are not a function of the features
    rp = rep["router_probe"]
    assert rp["best_draft_layer"]["3"] == 1 and rp["recall@2"]["by_layer"]["3"]["recall"] > 0.97
    sweep = rp["train_recall_by_layer_and_draft_layer"]["3"]
    assert sweep["1"] > 0.97 and sweep["0"] < 0.5
    # the ridge probe recovers the same map from the data alone (bf16 features, fp16 logits)
    rg = rep["ridge_probe"]
    assert rg["recall@2"]["by_layer"]["3"]["recall"] > 0.95 and rg["recall@4"]["by_layer"]["3"]["recall"] >= rg["recall@2"]["by_layer"]["3"]["recall"]
    # cells thin out with the depth of the row; union coverage counts blocks
    by_row = rep["ridge_probe"]["recall@2"]["by_row"]
    assert by_row["0"]["n"] >= by_row["1"]["n"] >= by_row["2"]["n"] > 0
    assert rep["router_probe"]["union_coverage"]["by_layer"]["3"] > 0.97 and rep["router_probe"]["union_coverage"]["blocks"] > 0
    # sequences are never split
    ex = ec.join_examples(d)
    tr, he = eb.split_by_sequence(ex, 0.25)
    assert not ({e["seq"] for e in tr} & {e["seq"] for e in he}) and len(tr) + len(he) == len(ex)
    # command line: without weights the router probe is left out; an empty directory is an error
    out = str(tmp_path / "rep.json")
    assert eb.main([d, "--widths", "2,4", "--ridge", "0.001", "--out", out]) == 0
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert "router_probe" not in line and line["ridge_probe"]["recall@2"][0] > 0.5 and "ridge_probe" in json.load(open(out))
    assert eb.main([str(tmp_path / "nothing")]) == 2


def test_a_single_sequence_is_scored_in_sample_and_says_so(tmp_path):
    d = str(tmp_path / "one")
    _corpus(d, n_seq=1, blocks=8)
    rep = eb.evaluate(d, None, widths=(2,))
    assert rep["in_sample"] and rep["sequences"] == 1 and rep["ridge_probe"]["recall@2"]["n"] > 0
