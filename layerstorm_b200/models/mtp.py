"""Multi-token-prediction (MTP) blocks on the fp32 reference model.

Block k (layer id ``n_layers + k``) takes, for every position i, the stream of the previous depth at i and the embedding of the token
``depth`` places ahead, and predicts the token one further:
    x_i   = eh_proj [ RMSNorm_e(Emb(t_{i+depth})) ; RMSNorm_h(h_i^{depth-1}) ]
    h_i^d = decoder_block_k(x)_i                      (MLA attention over positions 0..i, dense, + the block's FFN / MoE)
    P(t_{i+depth+1}) = softmax(head(RMSNorm_f(h_i^d)))    (embedding and output head shared with the main model)
with h^0 = the main model's stream before its output norm.  Depth d uses block (d - 1) mod n_mtp, so a model with one block can draft
several tokens by feeding the block its own output stream.
Reference counterparts: python/orchestrator/mtp_draft.py (cyclic block index, dynamic depth) and the engine's MtpSpeculationMethod
(src/speculation/); architecture: DeepSeek-V3 technical report, section 2.2.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch

from .reference import Oracle, rmsnorm


def mtp_block(oracle: Oracle, k: int, hidden_prev: torch.Tensor, tokens_ahead: Sequence[int]) -> Tuple[torch.Tensor, torch.Tensor]:
    """One MTP block over a whole sequence.  ``hidden_prev`` [T, H]: stream of the previous depth; ``tokens_ahead`` [T]: the token
    ``depth`` places ahead of each position.  Returns (logits [T, vocab], stream [T, H])."""
    cfg, w = oracle.cfg, oracle.w
    L = cfg.n_layers + k
    p = f"layers.{L}."
    T = hidden_prev.shape[0]
    pos = torch.arange(T)
    e = rmsnorm(w["embed.weight"][torch.as_tensor(list(tokens_ahead), dtype=torch.long)], w[p + "mtp.enorm"], cfg.rms_eps)
    h = rmsnorm(hidden_prev, w[p + "mtp.hnorm"], cfg.rms_eps)
    resid = torch.cat([e, h], -1) @ w[p + "mtp.eh_proj"].T
    dense = [list(range(t + 1)) for t in range(T)]                       # the block attends densely (no indexer of its own)
    x = rmsnorm(resid, w[p + "attn_norm.weight"], cfg.rms_eps)
    resid = resid + oracle.mla(L, x, pos, dense)
    x = rmsnorm(resid, w[p + "ffn_norm.weight"], cfg.rms_eps)
    resid = resid + oracle.ffn(L, x)
    logits = rmsnorm(resid, w[p + "mtp.final_norm"], cfg.rms_eps) @ w["head.weight"].T
    return logits, resid


def mtp_draft_tokens(oracle: Oracle, context: Sequence[int], depth: int, stop=None) -> Tuple[List[int], List[float]]:
    """Greedy MTP draft after ``context`` (whose last token has not been fed to the main model yet).  Returns the drafted tokens and the
    probability the block gave each.  ``stop(step, confidence)``: return True to end the draft after that step."""
    cfg = oracle.cfg
    if cfg.n_mtp <= 0 or len(context) < 2:
        return [], []
    ext = [int(t) for t in context]
    n = len(ext) - 1
    _, hidden = oracle.forward(torch.tensor(ext[:n]), return_hidden=True)
    out, conf = [], []
    for d in range(1, depth + 1):
        logits, hidden = mtp_block(oracle, (d - 1) % cfg.n_mtp, hidden, ext[d: d + n])
        pr = torch.softmax(logits[-1], -1)
        tok = int(torch.argmax(pr))
        out.append(tok)
        conf.append(float(pr[tok]))
        ext.append(tok)
        if stop is not None and stop(d - 1, conf[-1]):
            break
    return out, conf
