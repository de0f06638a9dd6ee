"""Chunk-parallel form of the KDA (gated delta rule with per-channel decay) recurrence: the algorithm the tensor-core prefill kernel
implements, as plain PyTorch, checked against the token-by-token recurrence.

Per head, with state S [Dv, Dk], key-channel decay d_t in (0, 1]^Dk, write strength beta_t:
    S <- S diag(d_t);   u_t = beta_t (v_t - S k_t);   S <- S + u_t k_t^T;   o_t = S q_t
Within a chunk of C tokens let G_t = sum_{s<=t} log d_s (cumulative log-decay from the chunk start, per channel).  Then
    A[t, s] = sum_c k_t[c] k_s[c] exp(G_t[c] - G_s[c])          (s <  t)      how much of write s is seen by read t
    B[t, s] = sum_c q_t[c] k_s[c] exp(G_t[c] - G_s[c])          (s <= t)
    (I + diag(beta) tril(A, -1)) U = diag(beta) (V - (K * exp(G)) S0^T)       forward substitution, U [C, Dv]
    O = (Q * exp(G)) S0^T + tril(B) U
    S_C = S0 diag(exp(G_C)) + U^T (K * exp(G_C - G))
Every exponent is <= 0, so nothing overflows however strong the decay (the naive "divide the keys by the cumulative decay" form
overflows fp32 after a few dozen tokens at the model's lower bound).

A and B are not plain matrix products because the decay ratio depends on the channel.  ``blockwise=True`` builds them the way a
tensor-core kernel can: the chunk is cut into sub-chunks of ``sub`` tokens; for a read sub-chunk i and an earlier write sub-chunk j
the ratio factorises through the start b_i of sub-chunk i,  exp(G_t - G_s) = exp(G_t - G_{b_i}) * exp(G_{b_i} - G_s),  both factors
<= 1, so the block is one matrix product of two rescaled operand tiles; diagonal blocks (sub x sub) are evaluated element-wise.
``operand_dtype=torch.bfloat16`` rounds the matrix-product operands as the kernel would and keeps fp32 accumulation.
Reference counterpart: src/compute/kernels/sm120/attention/kda_linear.cu (``launch_kda_chunked_scan``, the reference's chunked scan
for prefill); ``csrc/kernels/kda.cu`` ``kda_recur`` of this framework still walks the tokens one by one.  The derivation here follows the
public gated-delta-rule / Kimi Delta Attention formulation, not the reference's code.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch


def kda_sequential(q, k, v, beta, decay, S0=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """q, k [T, H, Dk]; v [T, H, Dv]; beta [T, H]; decay [T, H, Dk].  Returns (o [T, H, Dv], S [H, Dv, Dk])."""
    T, H, Dk = k.shape
    Dv = v.shape[-1]
    S = torch.zeros(H, Dv, Dk, dtype=q.dtype) if S0 is None else S0.clone()
    out = torch.empty(T, H, Dv, dtype=q.dtype)
    for t in range(T):
        S = S * decay[t][:, None, :]
        u = (v[t] - (S * k[t][:, None, :]).sum(-1)) * beta[t][:, None]
        S = S + u[:, :, None] * k[t][:, None, :]
        out[t] = (S * q[t][:, None, :]).sum(-1)
    return out, S


def _mm(a, b, operand_dtype):
    if operand_dtype is None:
        return a @ b
    return (a.to(operand_dtype).to(a.dtype)) @ (b.to(operand_dtype).to(b.dtype))


def _pair_matrices(qc, kc, G, blockwise: bool, sub: int, operand_dtype):
    """A[t, s] and B[t, s] for one head and chunk (rows t, columns s), full [C, C] (the caller masks)."""
    C = kc.shape[0]
    if not blockwise:
        ratio = torch.exp((G[:, None, :] - G[None, :, :]).clamp(max=0.0))          # [t, s, c]; entries with s > t are masked later
        return torch.einsum("tc,sc,tsc->ts", kc, kc, ratio), torch.einsum("tc,sc,tsc->ts", qc, kc, ratio)
    A = torch.zeros(C, C, dtype=kc.dtype)
    B = torch.zeros(C, C, dtype=kc.dtype)
    for i0 in range(0, C, sub):
        i1 = min(i0 + sub, C)
        Gb = G[i0 - 1] if i0 > 0 else torch.zeros_like(G[0])                       # cumulative log-decay just before the sub-chunk
        up = torch.exp(G[i0:i1] - Gb)                                               # exp(G_t - G_b) <= 1
        kt, qt = kc[i0:i1] * up, qc[i0:i1] * up
        if i0 > 0:
            ks = kc[:i0] * torch.exp(Gb - G[:i0])                                   # exp(G_b - G_s) <= 1 for s before the sub-chunk
            A[i0:i1, :i0] = _mm(kt, ks.T, operand_dtype)
            B[i0:i1, :i0] = _mm(qt, ks.T, operand_dtype)
        r = torch.exp((G[i0:i1, None, :] - G[None, i0:i1, :]).clamp(max=0.0))      # diagonal block, element-wise
        A[i0:i1, i0:i1] = torch.einsum("tc,sc,tsc->ts", kc[i0:i1], kc[i0:i1], r)
        B[i0:i1, i0:i1] = torch.einsum("tc,sc,tsc->ts", qc[i0:i1], kc[i0:i1], r)
    return A, B


def kda_chunk_prepare(q, k, beta, decay, chunk: int = 64, blockwise: bool = True, sub: int = 16, operand_dtype: Optional[torch.dtype] = None):
    """Phase 1, independent of the state and therefore parallel over (chunk, head): for every chunk
        W  = (I + diag(beta) tril(A, -1))^-1 diag(beta)      [C, C]   (so that U = W (V - Kp S0^T))
        Bm = tril(B)                                          [C, C]
        Qp = Q * exp(G), Kp = K * exp(G)                      [C, Dk]  read keys / queries seen from the chunk start
        Km = K * exp(G_C - G)                                 [C, Dk]  write keys seen from the chunk end
        gC = exp(G_C)                                         [Dk]     decay of the carried state over the whole chunk
    Returns a list over chunks of dicts of tensors with a leading head dimension."""
    T, H, Dk = k.shape
    logd = torch.log(decay)
    out = []
    for c0 in range(0, T, chunk):
        c1 = min(c0 + chunk, T)
        C = c1 - c0
        G = torch.cumsum(logd[c0:c1], 0)
        eye = torch.eye(C, dtype=q.dtype)
        W, Bm = torch.empty(H, C, C, dtype=q.dtype), torch.empty(H, C, C, dtype=q.dtype)
        for h in range(H):
            A, B = _pair_matrices(q[c0:c1, h], k[c0:c1, h], G[:, h], blockwise, sub, operand_dtype)
            bc = beta[c0:c1, h]
            W[h] = torch.linalg.solve_triangular(eye + bc[:, None] * torch.tril(A, -1), torch.diag(bc), upper=False)
            Bm[h] = torch.tril(B)
        eg = torch.exp(G).transpose(0, 1)                                               # [H, C, Dk]
        kh, qh = k[c0:c1].transpose(0, 1), q[c0:c1].transpose(0, 1)
        out.append({"rows": (c0, c1), "W": W, "B": Bm, "Qp": qh * eg, "Kp": kh * eg,
                    "Km": kh * torch.exp(G[-1][None] - G).transpose(0, 1), "gC": torch.exp(G[-1])})
    return out


def kda_chunk_scan(prep, v, S0=None, operand_dtype: Optional[torch.dtype] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Phase 2, sequential over chunks, independent per (head, value channel): four small matrix products per chunk."""
    T, H, Dv = v.shape
    Dk = prep[0]["Kp"].shape[-1]
    S = torch.zeros(H, Dv, Dk, dtype=v.dtype) if S0 is None else S0.clone()
    out = torch.empty(T, H, Dv, dtype=v.dtype)
    mm = lambda a, b: _mm(a, b, operand_dtype)
    for p in prep:
        c0, c1 = p["rows"]
        St = S.transpose(1, 2)                                                          # [H, Dk, Dv]
        U = mm(p["W"], v[c0:c1].transpose(0, 1) - mm(p["Kp"], St))                       # [H, C, Dv]
        out[c0:c1] = (mm(p["Qp"], St) + mm(p["B"], U)).transpose(0, 1)
        S = S * p["gC"][:, None, :] + mm(U.transpose(1, 2), p["Km"])
    return out, S


def kda_chunked(q, k, v, beta, decay, S0=None, chunk: int = 64, blockwise: bool = False, sub: int = 16,
                operand_dtype: Optional[torch.dtype] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    T, H, Dk = k.shape
    Dv = v.shape[-1]
    S = torch.zeros(H, Dv, Dk, dtype=q.dtype) if S0 is None else S0.clone()
    out = torch.empty(T, H, Dv, dtype=q.dtype)
    logd = torch.log(decay)
    for c0 in range(0, T, chunk):
        c1 = min(c0 + chunk, T)
        C = c1 - c0
        G = torch.cumsum(logd[c0:c1], 0)                                            # [C, H, Dk]
        eye = torch.eye(C, dtype=q.dtype)
        for h in range(H):
            qc, kc, vc, bc, Gh = q[c0:c1, h], k[c0:c1, h], v[c0:c1, h], beta[c0:c1, h], G[:, h]
            A, B = _pair_matrices(qc, kc, Gh, blockwise, sub, operand_dtype)
            eg = torch.exp(Gh)
            rhs = bc[:, None] * (vc - _mm(kc * eg, S[h].T, operand_dtype))          # [C, Dv]
            Tm = eye + bc[:, None] * torch.tril(A, -1)
            U = torch.linalg.solve_triangular(Tm, rhs, upper=False)
            out[c0:c1, h] = _mm(qc * eg, S[h].T, operand_dtype) + _mm(torch.tril(B), U, operand_dtype)
            S[h] = S[h] * eg[-1][None, :] + _mm(U.T, kc * torch.exp(Gh[-1][None, :] - Gh), operand_dtype)
    return out, S
