"""fp32 CPU oracle: a plain PyTorch forward pass of every supported architecture over a
whole token sequence.  It is the correctness anchor for the CUDA engine (tests compare the
engine's prefill / decode / verify logits with this forward on the same prefix) and the
timed CPU baseline of the tiny "CPU plumbing" configuration.

Math sources: MLA absorbed layer src/daemon/attention/arch_mla.cpp:47-312,1824-1994;
gating tests/unit/topk_gating_test.cpp:31-125; expert FFN + combine src/core/expert_device.h:31-52;
glm5_next (mHC, KDA, NoPE MLA, MoE) tools/glm53_numpy_ref.py:128-232,430-499;
IndexPool tests/unit/kpool_reference.h.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from .config import ModelConfig


def rmsnorm(x, w, eps):
    x = x.float()
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def rope_interleaved(x, pos, inv_freq):
    """x [..., T, d] with d even, rotate adjacent pairs by pos * inv_freq."""
    if x.shape[-1] == 0:
        return x
    ang = pos.float()[:, None] * torch.tensor(inv_freq, dtype=torch.float32)[None, :]   # [T, d/2]
    c, s = torch.cos(ang), torch.sin(ang)
    xe, xo = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = xe * c - xo * s
    out[..., 1::2] = xe * s + xo * c
    return out


def swiglu(g, u, limit):
    if limit and limit > 0:
        g = g.clamp(max=limit)
        u = u.clamp(-limit, limit)
    return torch.nn.functional.silu(g) * u


def hadamard(x):
    d = x.shape[-1]
    h = 1
    y = x.clone()
    while h < d:
        y = y.view(*x.shape[:-1], d // (2 * h), 2, h)
        a, b = y[..., 0, :], y[..., 1, :]
        y = torch.stack((a + b, a - b), dim=-2).reshape(*x.shape)
        h *= 2
    return y * (d ** -0.5)


def route(cfg: ModelConfig, logits, bias):
    """Returns (ids [T,k], weights [T,k]); ties to the lower index."""
    if cfg.scoring == "sigmoid":
        score = torch.sigmoid(logits)
    elif cfg.scoring == "softmax":
        score = torch.softmax(logits, -1)
    else:
        score = torch.sqrt(torch.nn.functional.softplus(logits))
    sel = score + (bias if bias is not None else 0.0)
    T, E = sel.shape
    if cfg.n_group > 1:
        gs = E // cfg.n_group
        g = sel.view(T, cfg.n_group, gs)
        gscore = g.topk(2, -1).values.sum(-1)
        order = torch.argsort(-gscore, dim=-1, stable=True)[:, :cfg.topk_group]
        mask = torch.zeros(T, cfg.n_group, dtype=torch.bool)
        mask.scatter_(1, order, True)
        sel = torch.where(mask[:, :, None].expand(T, cfg.n_group, gs).reshape(T, E), sel, torch.tensor(-float("inf")))
    ids = torch.argsort(-sel, dim=-1, stable=True)[:, :cfg.top_k]
    w = torch.gather(score, 1, ids)
    if cfg.norm_topk_prob:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return ids, w * cfg.routed_scale


def route_hash(cfg: ModelConfig, logits, tid2eid, token_ids):
    """Hash-layer routing (DeepSeek-V4): the experts of a row are the table row of its token id (table order), the
    weights the scores of those experts without selection bias.  Entries outside the table or the expert range give
    id -1 / weight 0.  Reference semantics: src/compute/kernels/moe/hash_gating.h:1-16."""
    if cfg.scoring == "sigmoid":
        score = torch.sigmoid(logits)
    elif cfg.scoring == "softmax":
        score = torch.softmax(logits, -1)
    else:
        score = torch.sqrt(torch.nn.functional.softplus(logits))
    T, E = score.shape
    tok = token_ids.long()
    ok_tok = (tok >= 0) & (tok < tid2eid.shape[0])
    ids = tid2eid[tok.clamp(0, tid2eid.shape[0] - 1)].long()
    ok = ok_tok[:, None] & (ids >= 0) & (ids < E)
    w = torch.where(ok, torch.gather(score, 1, ids.clamp(0, E - 1)), torch.zeros(()))
    if cfg.norm_topk_prob:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return torch.where(ok, ids, torch.full_like(ids, -1)), w * cfg.routed_scale


class Oracle:
    def __init__(self, cfg: ModelConfig, weights: Dict[str, torch.Tensor]):
        self.cfg = cfg
        self.w = {k: v.float() for k, v in weights.items() if not k.endswith(".tid2eid")}
        self.tables = {k: v.long() for k, v in weights.items() if k.endswith(".tid2eid")}       # integer tables stay integers
        self._tok = None
        self.sel_log: Dict[int, List] = {}

    # ---------------- sublayers ----------------
    def ffn(self, i, x):
        cfg, w = self.cfg, self.w
        p = f"layers.{i}."
        if not cfg.is_moe_layer(i):
            return swiglu(x @ w[p + "mlp.gate"].T, x @ w[p + "mlp.up"].T, cfg.swiglu_limit) @ w[p + "mlp.down"].T
        m = p + "moe."
        logits = x @ w[m + "router"].T
        if cfg.is_hash_layer(i) and (m + "tid2eid") in self.tables:
            # hash layer: the experts are the table row of the token id, the weights their unbiased scores; -1 = dropped
            if self._tok is None or self._tok.shape[0] != x.shape[0]:
                raise RuntimeError("a hash layer needs the token ids of the rows (Oracle.forward sets them)")
            ids, wt = route_hash(cfg, logits, self.tables[m + "tid2eid"], self._tok)
        else:
            ids, wt = route(cfg, logits, w.get(m + "router_bias"))
        self.last_route = (ids, wt)
        if getattr(self, "route_log", None) is not None:
            self.route_log[i] = (logits, ids, wt)                 # per row: router logits, chosen experts, their weights
        out = torch.zeros_like(x)
        for t in range(x.shape[0]):
            for k in range(cfg.top_k):
                e = int(ids[t, k])
                if e < 0:
                    continue                                      # a dropped slot of a hash layer
                h = swiglu(x[t] @ w[m + f"experts.{e}.gate"].T, x[t] @ w[m + f"experts.{e}.up"].T, cfg.swiglu_limit)
                out[t] += wt[t, k] * (h @ w[m + f"experts.{e}.down"].T)
        for s in range(cfg.n_shared):
            h = swiglu(x @ w[m + f"shared.{s}.gate"].T, x @ w[m + f"shared.{s}.up"].T, cfg.swiglu_limit)
            out = out + h @ w[m + f"shared.{s}.down"].T
        return out

    def indexer_select(self, i, x, q_c, pos):
        """Per query row the sorted list of selected token positions (or None = dense)."""
        cfg, w = self.cfg, self.w
        src = cfg.index_source_layer(i)
        if src != i:
            return self.sel_log[src]
        p = f"layers.{i}.indexer."
        T = x.shape[0]
        IH, ID, P = cfg.index_n_heads, cfg.index_head_dim, cfg.index_kpool
        inv = cfg.rope_inv_freq(cfg.index_rope_dim) if cfg.index_rope_dim else []
        k = torch.nn.functional.layer_norm(x @ w[p + "wk"].T, (ID,), w[p + "k_norm.weight"], w[p + "k_norm.bias"], 1e-6)
        q = (q_c @ w[p + "wq_b"].T).view(T, IH, ID)
        if cfg.index_rope_dim:
            dr = cfg.index_rope_dim
            k = torch.cat([rope_interleaved(k[:, :dr], pos, inv), k[:, dr:]], -1)
            q = torch.cat([rope_interleaved(q[..., :dr].transpose(0, 1), pos, inv).transpose(0, 1), q[..., dr:]], -1)
        q = hadamard(q)
        wts = (x @ w[p + "weights_proj"].T) * (IH ** -0.5) * (ID ** -0.5)
        if P > 1:
            gate = x @ w[p + "gate"].T
            npool = T // P
            kk = k[: npool * P].view(npool, P, ID)
            s = gate[: npool * P].view(npool, P, ID) + w[p + "ape"][None]
            pw = torch.softmax(s, dim=1)
            ent = hadamard((pw * kk).sum(1))
        else:
            ent = hadamard(k)
        sels = []
        budget = cfg.index_topk // P
        for t in range(T):
            ln = int(pos[t]) + 1
            ne = ln // P
            if ne <= budget:
                chosen = list(range(ne))
            else:
                sc = (torch.relu(torch.einsum("hd,nd->hn", q[t], ent[:ne])) * wts[t][:, None]).sum(0)
                order = torch.argsort(-sc, stable=True)[:budget]
                chosen = sorted(int(o) for o in order)
            toks = [c * P + j for c in chosen for j in range(P)] + list(range(ne * P, ln))
            sels.append(toks)
        self.sel_log[i] = sels
        return sels

    def mla(self, i, x, pos, sel_override=None):
        cfg, w = self.cfg, self.w
        p = f"layers.{i}.attn."
        T, Hh = x.shape[0], cfg.n_heads
        inv = cfg.rope_inv_freq()
        q_c = rmsnorm(x @ w[p + "q_a"].T, w[p + "q_a_norm"], cfg.rms_eps)
        q = (q_c @ w[p + "q_b"].T).view(T, Hh, cfg.qk_head)
        q_nope, q_pe = q[..., : cfg.qk_nope], q[..., cfg.qk_nope:]
        kv = x @ w[p + "kv_a"].T
        c = rmsnorm(kv[:, : cfg.kv_lora], w[p + "kv_a_norm"], cfg.rms_eps)
        k_pe = rope_interleaved(kv[:, cfg.kv_lora:], pos, inv)
        q_pe = rope_interleaved(q_pe.transpose(0, 1), pos, inv).transpose(0, 1)
        q_lat = torch.einsum("thp,hlp->thl", q_nope, w[p + "k_b"])
        scores = (torch.einsum("thl,sl->hts", q_lat, c) + torch.einsum("thr,sr->hts", q_pe, k_pe)) * cfg.softmax_scale
        mask = pos[None, :] > pos[:, None]          # [t, s] True = not visible
        if sel_override is not None:
            sels = sel_override
        elif cfg.has_indexer:
            sels = self.indexer_select(i, x, q_c, pos)
        else:
            sels = None
        if sels is not None:
            allow = torch.zeros(T, T, dtype=torch.bool)
            for t, s in enumerate(sels):
                allow[t, torch.tensor(s, dtype=torch.long)] = True
            mask = mask | ~allow
        scores = scores.masked_fill(mask[None], -float("inf"))
        pr = torch.softmax(scores, -1)
        o_lat = torch.einsum("hts,sl->thl", pr, c)
        o = torch.einsum("thl,hvl->thv", o_lat, w[p + "v_b"]).reshape(T, Hh * cfg.v_head)
        return o @ w[p + "o"].T

    def kda(self, i, x):
        cfg, w = self.cfg, self.w
        p = f"layers.{i}.kda."
        T, Hk, D = x.shape[0], cfg.kda_heads, cfg.kda_head_dim

        def conv_silu(raw, cw):
            hist = torch.cat([torch.zeros(cfg.kda_conv - 1, raw.shape[1]), raw], 0)
            acc = torch.zeros_like(raw)
            for j in range(cfg.kda_conv):
                acc = acc + hist[j: j + T] * cw[:, j][None]
            return torch.nn.functional.silu(acc)

        q = conv_silu(x @ w[p + "q"].T, w[p + "conv_q"]).view(T, Hk, D)
        k = conv_silu(x @ w[p + "k"].T, w[p + "conv_k"]).view(T, Hk, D)
        v = conv_silu(x @ w[p + "v"].T, w[p + "conv_v"]).view(T, Hk, D)
        beta = torch.sigmoid(x @ w[p + "beta"].T)
        raw_g = ((x @ w[p + "f_a"].T) @ w[p + "f_b"].T).view(T, Hk, D)
        g2 = ((x @ w[p + "g_a"].T) @ w[p + "g_b"].T).view(T, Hk, D)
        a_exp = torch.exp(w[p + "a_log"])
        decay = torch.exp(cfg.kda_lower_bound * torch.sigmoid(a_exp[None, :, None] * (raw_g + w[p + "dt_bias"][None])))
        qn = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * (D ** -0.5)
        kn = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        if getattr(self, "kda_chunk", 0):
            # chunk-parallel form (models/kda_chunked.py): same result, the algorithm of a tensor-core prefill kernel
            from .kda_chunked import kda_chunked
            core, _ = kda_chunked(qn, kn, v, beta, decay, None, chunk=self.kda_chunk, blockwise=True)
        else:
            S = torch.zeros(Hk, D, D)
            core = torch.empty(T, Hk, D)
            for t in range(T):
                S = S * decay[t][:, None, :]
                err = (v[t] - (S * kn[t][:, None, :]).sum(-1)) * beta[t][:, None]
                S = S + err[:, :, None] * kn[t][:, None, :]
                core[t] = (S * qn[t][:, None, :]).sum(-1)
        on = core * torch.rsqrt(core.pow(2).mean(-1, keepdim=True) + cfg.rms_eps) * w[p + "o_norm"][None, None] * torch.sigmoid(g2)
        return on.reshape(T, Hk * D) @ w[p + "o"].T

    # ---------------- mHC ----------------
    def mhc_pre(self, residual, fn, scale, base, norm_w):
        cfg = self.cfg
        T, n, H = residual.shape
        xf = residual.reshape(T, n * H)
        mixes = (xf @ fn.T) * torch.rsqrt((xf * xf).sum(-1, keepdim=True) / (n * H) + cfg.rms_eps)
        pre = torch.sigmoid(mixes[:, :n] * scale[0] + base[:n]) + cfg.hc_eps
        post = torch.sigmoid(mixes[:, n:2 * n] * scale[1] + base[n:2 * n]) * cfg.hc_post_mult
        comb = torch.softmax(mixes[:, 2 * n:].view(T, n, n) * scale[2] + base[2 * n:].view(1, n, n), -1) + cfg.hc_eps
        comb = comb / (comb.sum(-2, keepdim=True) + cfg.hc_eps)
        for _ in range(cfg.hc_sinkhorn_iters - 1):
            comb = comb / (comb.sum(-1, keepdim=True) + cfg.hc_eps)
            comb = comb / (comb.sum(-2, keepdim=True) + cfg.hc_eps)
        x = rmsnorm((pre[:, :, None] * residual).sum(1), norm_w, cfg.rms_eps)
        return post, comb, x

    @staticmethod
    def mhc_post(x, residual, post, comb):
        return torch.einsum("tij,tih->tjh", comb, residual) + post[:, :, None] * x[:, None, :]

    # ---------------- full forward ----------------
    def forward(self, ids: torch.Tensor, pos: Optional[torch.Tensor] = None, sel_override: Optional[dict] = None,
                trace: Optional[list] = None, return_hidden: bool = False, aux: Optional[dict] = None):
        """``aux``: a dict whose keys are layer numbers; each gets the stream that ENTERS that layer ([T, hidden]; hyper-connection
        models: the mean over the residual streams), key ``n_layers`` the stream that leaves the last layer - the features a block
        draft model is conditioned on (``speculation/dspark.py``)."""
        cfg, w = self.cfg, self.w
        ids = torch.as_tensor(ids, dtype=torch.long)
        T = ids.shape[0]
        self._tok = ids                                           # hash layers route by token id
        pos = torch.arange(T) if pos is None else torch.as_tensor(pos)
        self.sel_log = {}
        h = w["embed.weight"][ids]
        if cfg.mhc:
            residual = h[:, None, :].repeat(1, cfg.hc_mult, 1)
            post = comb = None
            x_out = None
            for i in range(cfg.n_layers):
                p = f"layers.{i}."
                if post is not None:
                    residual = self.mhc_post(x_out, residual, post, comb)
                if aux is not None and i in aux:
                    aux[i] = residual.mean(1)
                post, comb, x = self.mhc_pre(residual, w[p + "hc_attn.fn"], w[p + "hc_attn.scale"], w[p + "hc_attn.base"], w[p + "attn_norm.weight"])
                a = self.kda(i, x) if cfg.is_kda_layer(i) else self.mla(i, x, pos, (sel_override or {}).get(i))
                residual = self.mhc_post(a, residual, post, comb)
                post, comb, x = self.mhc_pre(residual, w[p + "hc_ffn.fn"], w[p + "hc_ffn.scale"], w[p + "hc_ffn.base"], w[p + "ffn_norm.weight"])
                x_out = self.ffn(i, x)
                if trace is not None:
                    trace.append(x_out.clone())
            final = self.mhc_post(x_out, residual, post, comb).mean(1)
        else:
            resid = h
            for i in range(cfg.n_layers):
                p = f"layers.{i}."
                if aux is not None and i in aux:
                    aux[i] = resid.clone()
                x = rmsnorm(resid, w[p + "attn_norm.weight"], cfg.rms_eps)
                a = self.kda(i, x) if cfg.is_kda_layer(i) else self.mla(i, x, pos, (sel_override or {}).get(i))
                resid = resid + a
                x = rmsnorm(resid, w[p + "ffn_norm.weight"], cfg.rms_eps)
                resid = resid + self.ffn(i, x)
                if trace is not None:
                    trace.append(resid.clone())
            final = resid
        if aux is not None and cfg.n_layers in aux:
            aux[cfg.n_layers] = final.clone()
        logits = rmsnorm(final, w["final_norm.weight"], cfg.rms_eps) @ w["head.weight"].T
        return (logits, final) if return_hidden else logits        # ``final``: the stream before the output norm (input of the MTP blocks)

    def greedy(self, prompt, n_new: int) -> List[int]:
        """Greedy decode by re-running the full forward (O(T^2); fine for the tiny model)."""
        ids = list(int(t) for t in prompt)
        out = []
        for _ in range(n_new):
            logits = self.forward(torch.tensor(ids))
            nxt = int(torch.argmax(logits[-1]))
            out.append(nxt)
            ids.append(nxt)
        return out
