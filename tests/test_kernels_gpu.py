"""Numerics of the decode-path CUDA kernels against plain PyTorch fp32 references."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from layerstorm_b200.formats import quant
from layerstorm_b200.models import reference as ref
from layerstorm_b200.models.config import ModelConfig, get_preset
from layerstorm_b200.ops import _native as nat

DEV = "cuda"


def rnd(*shape, s=1.0, dtype=torch.float32, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * s).to(dtype).to(DEV)


def close(a, b, rtol, atol, what=""):
    a, b = a.float().cpu(), b.float().cpu()
    err = (a - b).abs()
    lim = atol + rtol * b.abs()
    bad = err > lim
    assert not bad.any(), f"{what}: {int(bad.sum())}/{a.numel()} off, max err {float(err.max()):.4g} (ref max {float(b.abs().max()):.4g})"


@pytest.mark.parametrize("M", [1, 2, 3, 7])
@pytest.mark.parametrize("fmt", ["bf16", "f32", "fp8", "nvfp4"])
def test_gemv_formats(M, fmt):
    N, K = 200, 512
    x = rnd(M, K, dtype=torch.bfloat16)
    w = rnd(N, K, s=0.05, seed=1)
    out = torch.zeros(M, N, device=DEV)
    if fmt == "bf16":
        wq = w.to(torch.bfloat16)
        nat.call("lsb_gemv_bf16", out, x, wq, None, M, N, K, K, K, N, 1.0, 0, None)
        wd = wq.float()
    elif fmt == "f32":
        nat.call("lsb_gemv_f32w", out, x, w, None, M, N, K, K, K, N, 1.0, 0)
        wd = w
    elif fmt == "fp8":
        q, s = quant.quantize_fp8_block(w)
        nat.call("lsb_gemv_fp8b", out, x, q, s, None, M, N, K, K, N, 1.0, 0, None)
        wd = quant.dequantize_fp8_block(q, s)
    else:
        q, a, gs = quant.quantize_nvfp4(w)
        nat.call("lsb_gemv_nvfp4", out, x, q, a, None, M, N, K, K, N, gs, 0, None)
        wd = quant.dequantize_nvfp4(q, a, gs, N, K)
        assert (wd - w).abs().max() < 0.3 * w.abs().max()
    torch.cuda.synchronize()
    close(out, x.float() @ wd.T, 1e-3, 1e-3, f"gemv {fmt} M={M}")


def test_gemv_bf16_out_and_bias():
    M, N, K = 2, 64, 256
    x = rnd(M, K, dtype=torch.bfloat16)
    w = rnd(N, K, s=0.05, dtype=torch.bfloat16)
    b = rnd(N)
    out = torch.zeros(M, N, device=DEV, dtype=torch.bfloat16)
    nat.call("lsb_gemv_bf16", out, x, w, b, M, N, K, K, K, N, 1.0, 1, None)
    torch.cuda.synchronize()
    close(out, x.float() @ w.float().T + b, 1e-2, 1e-2, "gemv bf16 out")


def test_rmsnorm_and_add():
    R, D = 5, 768
    x = rnd(R, D)
    w = rnd(D) * 0.1 + 1
    out = torch.zeros(R, D, device=DEV, dtype=torch.bfloat16)
    nat.call("lsb_rmsnorm", out, x, w, R, D, D, D, 1e-6, 1, None)
    torch.cuda.synchronize()
    close(out, ref.rmsnorm(x.cpu(), w.cpu(), 1e-6), 1e-2, 1e-2, "rmsnorm")
    resid = rnd(R, D, seed=3)
    r0 = resid.clone()
    nat.call("lsb_add_rmsnorm", out, resid, x, w, R, D, 1e-6, None)
    torch.cuda.synchronize()
    close(resid, r0 + x, 1e-6, 1e-6, "resid add")
    close(out, ref.rmsnorm((r0 + x).cpu(), w.cpu(), 1e-6), 1e-2, 1e-2, "add_rmsnorm")


@pytest.mark.parametrize("fused,R", [(False, 3), (True, 3), (False, 70)])     # 70 rows: the wide many-row partial kernel
def test_mhc_post_pre_and_contract(fused, R):
    cfg = get_preset("tiny-glm5-next")
    H, n = cfg.hidden, cfg.hc_mult
    o = ref.Oracle(cfg, {})
    fn, sc, base, nw = rnd(24, n * H, s=0.05), torch.tensor([0.7, 1.1, 1.3], device=DEV), rnd(24, s=0.5), rnd(H) * 0.1 + 1
    emb = rnd(R, H)
    resid = torch.zeros(R, n, H, device=DEV)
    post = torch.zeros(R, n, device=DEV); comb = torch.zeros(R, n, n, device=DEV)
    part = torch.zeros(R, H // 32, 36, device=DEV)
    # fused = the few-row path (last block finalises, RMS from the Gram matrix); otherwise partial + per-row finalize
    done = torch.zeros(R, dtype=torch.int32, device=DEV) if fused else None
    prex = torch.zeros(R, 8, device=DEV) if fused else None
    x = torch.zeros(R, H, device=DEV, dtype=torch.bfloat16)
    args = (cfg.hc_sinkhorn_iters, cfg.hc_eps, cfg.rms_eps, cfg.hc_post_mult)
    nat.call("lsb_mhc_post_pre", x, resid, emb, post, comb, fn, sc, base, nw, part, R, H, n, 0, *args, done, prex, None)
    torch.cuda.synchronize()
    r_ref = emb.cpu()[:, None, :].repeat(1, n, 1)
    p_ref, c_ref, x_ref = o.mhc_pre(r_ref, fn.cpu(), sc.cpu(), base.cpu(), nw.cpu())
    close(resid, r_ref, 1e-6, 1e-6, "expand")
    close(post, p_ref, 1e-4, 1e-5, "post")
    close(comb, c_ref, 1e-4, 1e-5, "comb")
    close(x, x_ref, 1e-2, 1e-2, "x")
    sub = rnd(R, H, seed=5)
    nat.call("lsb_mhc_post_pre", x, resid, sub, post, comb, fn, sc, base, nw, part, R, H, n, 1, *args, done, prex, None)
    torch.cuda.synchronize()
    r2 = o.mhc_post(sub.cpu(), r_ref, p_ref, c_ref)
    p2, c2, x2 = o.mhc_pre(r2, fn.cpu(), sc.cpu(), base.cpu(), nw.cpu())
    close(resid, r2, 1e-4, 1e-5, "post residual")
    close(comb, c2, 1e-4, 1e-5, "comb2")
    close(x, x2, 1e-2, 1e-2, "x2")
    sub2 = rnd(R, H, seed=6)
    nat.call("lsb_mhc_contract_norm", x, resid, sub2, post, comb, nw, R, H, n, cfg.rms_eps, None)
    torch.cuda.synchronize()
    fin = ref.rmsnorm(o.mhc_post(sub2.cpu(), r2, p2, c2).mean(1), nw.cpu(), cfg.rms_eps)
    close(x, fin, 1e-2, 1e-2, "contract")


@pytest.mark.parametrize("H,E,k,R", [(256, 16, 4, 3), (4096, 288, 8, 1), (4096, 288, 8, 5), (2048, 64, 6, 2)])
def test_mhc_cluster_kernel_with_folded_combine_and_router(H, E, k, R):
    """The one-launch cluster form of the hyper-connection pass: plain, with the MoE combine folded in front, and with the router
    projection + top-k folded behind, against the oracle and the stand-alone router / combine arithmetic."""
    import dataclasses
    cfg = dataclasses.replace(get_preset("tiny-glm5-next"), hidden=H, n_routed=E, top_k=k, hc_sinkhorn_iters=20)
    n = cfg.hc_mult
    if nat.call("lsb_mhc_cluster_width", H, n) <= 0:
        pytest.skip("no cluster shape for this hidden size on this device")
    o = ref.Oracle(cfg, {})
    fn, sc, base, nw = rnd(24, n * H, s=0.05), torch.tensor([0.7, 1.1, 1.3], device=DEV), rnd(24, s=0.5), rnd(H) * 0.1 + 1
    S = k + 1
    rw, rb = rnd(E, H, s=0.1, seed=9), rnd(E, s=0.05, seed=10)
    resid = torch.zeros(R, n, H, device=DEV)
    post = torch.zeros(R, n, device=DEV); comb = torch.zeros(R, n, n, device=DEV)
    x = torch.zeros(R, H, device=DEV, dtype=torch.bfloat16)
    ids = torch.zeros(R, S, dtype=torch.int32, device=DEV); wts = torch.zeros(R, S, device=DEV)
    logits = torch.zeros(R, E, device=DEV)
    hc = (cfg.hc_sinkhorn_iters, cfg.hc_eps, cfg.rms_eps, cfg.hc_post_mult)
    rt = (E, k, 1, 1, 0, 1, 2.5, 1)

    def run(sub, mode, y=None, cw=None, ci=None, so=None, route=False):
        nat.call("lsb_mhc_cluster", x, resid, sub, post, comb, fn, sc, base, nw, R, H, n, mode, *hc, y, cw, ci, so, S,
                 rw if route else None, rb if route else None, logits if route else None, ids if route else None, wts if route else None, *rt, None)
        torch.cuda.synchronize()

    emb = rnd(R, H)
    run(emb, 0)
    r_ref = emb.cpu()[:, None, :].repeat(1, n, 1)
    p_ref, c_ref, x_ref = o.mhc_pre(r_ref, fn.cpu(), sc.cpu(), base.cpu(), nw.cpu())
    close(resid, r_ref, 1e-6, 1e-6, "expand")
    close(post, p_ref, 1e-4, 1e-5, "post"); close(comb, c_ref, 1e-4, 1e-5, "comb"); close(x, x_ref, 1e-2, 1e-2, "x")
    # post of a plain sublayer output, router folded behind
    sub = rnd(R, H, seed=5)
    run(sub, 1, route=True)
    r2 = o.mhc_post(sub.cpu(), r_ref, p_ref, c_ref)
    p2, c2, x2 = o.mhc_pre(r2, fn.cpu(), sc.cpu(), base.cpu(), nw.cpu())
    close(resid, r2, 1e-4, 1e-5, "post residual"); close(comb, c2, 1e-4, 1e-5, "comb2"); close(x, x2, 1e-2, 1e-2, "x2")
    lg_ref = x.float().cpu() @ rw.cpu().T                      # the router consumes the bf16-rounded activations
    close(logits, lg_ref, 1e-4, 1e-4, "router logits")
    ids2 = torch.zeros_like(ids); wts2 = torch.zeros_like(wts)
    nat.call("lsb_router_topk", logits, rb, ids2, wts2, R, E, k, 1, 1, 0, 1, 2.5, 1, E)
    torch.cuda.synchronize()
    assert torch.equal(ids, ids2) and torch.equal(wts, wts2), "folded router differs from the stand-alone top-k on the same logits"
    rid, rwt = ref.route(dataclasses.replace(cfg, routed_scale=2.5), logits.cpu(), rb.cpu())
    assert torch.equal(ids[:, :k].cpu().long(), rid)
    # post with the MoE combine folded in front: one expert marked non-resident
    y = rnd(R * S, H, seed=6)
    so = torch.arange(E + 1, dtype=torch.int32, device=DEV)
    so[int(ids[0, 1])] = -1
    want = torch.zeros(R, H, device=DEV)
    nat.call("lsb_moe_combine", want, y, wts, ids, so, R, S, H, 0, None)
    torch.cuda.synchronize()
    run(None, 1, y=y, cw=wts, ci=ids, so=so)
    r3 = o.mhc_post(want.cpu(), r2, p2, c2)
    p3, c3, x3 = o.mhc_pre(r3, fn.cpu(), sc.cpu(), base.cpu(), nw.cpu())
    close(resid, r3, 1e-4, 1e-5, "post residual after combine"); close(post, p3, 1e-4, 1e-5, "post3"); close(x, x3, 1e-2, 1e-2, "x3")


@pytest.mark.parametrize("scoring,n_group,topk_group", [("sigmoid", 1, 1), ("softmax", 1, 1), ("sigmoid", 4, 2), ("sqrtsoftplus", 1, 1)])
def test_router_topk(scoring, n_group, topk_group):
    E, k, R = 32, 4, 9
    cfg = ModelConfig(n_routed=E, top_k=k, scoring=scoring, n_group=n_group, topk_group=topk_group, routed_scale=2.5)
    logits = rnd(R, E)
    logits[0, 3] = logits[0, 7]           # exact tie -> lower index
    bias = rnd(E, s=0.1)
    ids = torch.zeros(R, k + 1, dtype=torch.int32, device=DEV)
    wts = torch.zeros(R, k + 1, device=DEV)
    nat.call("lsb_router_topk", logits, bias, ids, wts, R, E, k, n_group, topk_group,
             {"sigmoid": 0, "softmax": 1, "sqrtsoftplus": 2}[scoring], 1, 2.5, 1, E)
    torch.cuda.synchronize()
    rid, rw = ref.route(cfg, logits.cpu(), bias.cpu())
    assert torch.equal(ids[:, :k].cpu().long(), rid), (ids.cpu(), rid)
    close(wts[:, :k], rw, 1e-4, 1e-6, "router weights")
    assert (ids[:, k] == E).all() and (wts[:, k] == 1).all()


@pytest.mark.parametrize("E,k,n_group,topk_group,R", [(288, 8, 1, 1, 1), (256, 8, 8, 4, 3), (48, 6, 1, 1, 8)])
def test_router_fused_projection_and_topk(E, k, n_group, topk_group, R):
    """Router projection + rank-based top-k in one launch against the fp32 reference routing; the two-launch form must give the
    same bits on the same logits."""
    H = 512
    cfg = ModelConfig(n_routed=E, top_k=k, scoring="sigmoid", n_group=n_group, topk_group=topk_group, routed_scale=2.5)
    w = rnd(E, H, s=0.1, seed=3)
    x = rnd(R, H, dtype=torch.bfloat16, seed=4)
    bias = rnd(E, s=0.1)
    ids = torch.zeros(R, k + 1, dtype=torch.int32, device=DEV); wts = torch.zeros(R, k + 1, device=DEV)
    logits = torch.zeros(R, E, device=DEV)
    done = torch.zeros(1, dtype=torch.int32, device=DEV)
    nat.call("lsb_router_fused", w, x, logits, bias, ids, wts, done, R, H, E, k, n_group, topk_group, 0, 1, 2.5, 1)
    torch.cuda.synchronize()
    close(logits, x.float().cpu() @ w.cpu().T, 1e-4, 1e-4, "router logits")
    rid, rw = ref.route(cfg, logits.cpu(), bias.cpu())
    assert torch.equal(ids[:, :k].cpu().long(), rid), (ids.cpu(), rid)
    close(wts[:, :k], rw, 1e-4, 1e-6, "router weights")
    assert (ids[:, k] == E).all() and (wts[:, k] == 1).all() and int(done[0]) == 0
    ids2 = torch.zeros_like(ids); wts2 = torch.zeros_like(wts)
    nat.call("lsb_router_topk", logits, bias, ids2, wts2, R, E, k, n_group, topk_group, 0, 1, 2.5, 1, E)
    torch.cuda.synchronize()
    assert torch.equal(ids, ids2) and torch.equal(wts, wts2)


def test_moe_pair_kernels_give_the_same_bits_for_every_block_shape():
    """Pair-mode NVFP4 expert kernels: the rows of an expert can be cut into blocks of 32 / 16 / 8 (gate, up) and 64 / 32 / 16 (down)
    rows; the per-row arithmetic does not depend on the cut, so all shapes give identical bits, and they match fp32 math."""
    import ctypes
    from layerstorm_b200.models.device_model import ExpertArena, QLinear, expert_layout
    H, F, E, k, R = 512, 768, 6, 3, 2
    S = k + 1
    g = torch.Generator().manual_seed(7)
    arena = ExpertArena(expert_layout("nvfp4", H, F), E + 1, E + 1, DEV)
    mats = []
    for e in range(E + 1):
        gate, up, down = (QLinear.from_float(torch.randn(n_, k_, generator=g) * 0.05, "nvfp4", DEV) for n_, k_ in ((F, H), (F, H), (H, F)))
        arena.write_expert(e, gate, up, down)
        arena.slot_of[e] = e
        mats.append((gate.dequant().cpu(), up.dequant().cpu(), down.dequant().cpu()))
    efp = ctypes.addressof(arena.ef)
    x = rnd(R, H, dtype=torch.bfloat16, seed=8)
    ids = torch.stack([torch.cat([torch.randperm(E, generator=g)[:k], torch.tensor([E])]) for _ in range(R)]).int().to(DEV)
    outs = []
    for run_gu, run_dn in ((8, 16), (4, 8), (2, 4)):
        act = torch.zeros(R * S, F, dtype=torch.bfloat16, device=DEV)
        y = torch.zeros(R * S, H, device=DEV)
        nat.call("lsb_moe_gateup", x, arena.data, arena.slot_of, efp, ids, None, None, None, act, S, R * S, 10.0, None, run_gu)
        nat.call("lsb_moe_down", act, arena.data, arena.slot_of, efp, ids, None, None, None, y, R * S, run_dn)
        torch.cuda.synchronize()
        outs.append((act.clone(), y.clone()))
    for a, y in outs[1:]:
        assert torch.equal(a, outs[0][0]) and torch.equal(y, outs[0][1])
    xf = x.float().cpu()
    for r in range(R):
        for s_ in range(S):
            gm, um, dm = mats[int(ids[r, s_])]
            gv, uv = (xf[r] @ gm.T).clamp(max=10.0), (xf[r] @ um.T).clamp(-10.0, 10.0)
            want = (torch.nn.functional.silu(gv) * uv).to(torch.bfloat16).float() @ dm.T
            close(outs[0][1][r * S + s_], want, 2e-2, 2e-2 * float(want.abs().max()), "expert output")


@pytest.mark.parametrize("scoring", ["sigmoid", "softmax", "sqrtsoftplus"])
def test_router_hash(scoring):
    E, k, R, V = 48, 6, 7, 100
    cfg = ModelConfig(n_routed=E, top_k=k, scoring=scoring, routed_scale=1.5)
    logits = rnd(R, E)
    g = torch.Generator().manual_seed(3)
    table = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(V)]).int()
    table[5, 2] = E + 3                     # entry outside the expert range -> dropped slot
    toks = torch.tensor([0, 5, 17, 99, 100, 42, 5], dtype=torch.int32)    # 100 is outside the table
    ids = torch.zeros(R, k + 1, dtype=torch.int32, device=DEV)
    wts = torch.zeros(R, k + 1, device=DEV)
    nat.call("lsb_router_hash", logits, table.to(DEV), toks.to(DEV), ids, wts, R, E, k, V,
             {"sigmoid": 0, "softmax": 1, "sqrtsoftplus": 2}[scoring], 1, 1.5, 1, E)
    torch.cuda.synchronize()
    rid, rw = ref.route_hash(cfg, logits.cpu(), table, toks)
    assert torch.equal(ids[:, :k].cpu().long(), rid), (ids.cpu(), rid)
    close(wts[:, :k], rw, 1e-4, 1e-6, "hash router weights")
    assert (ids[4, :k] == -1).all() and (wts[4, :k] == 0).all() and int(ids[1, 2]) == -1
    assert (ids[:, k] == E).all() and (wts[:, k] == 1).all()


@pytest.mark.parametrize("R,sparse,H", [(4, False, 24), (20, False, 24), (20, True, 24), (33, True, 24), (18, True, 12), (20, True, 72)])
def test_mla_decode_attention(R, sparse, H):
    """Absorbed MLA attention over a paged bf16 cache against an fp32 reference; R >= 16 takes the tensor-core
    (mma) variant, smaller R the CUDA-core one; sparse = per-row selected positions (the indexer's output)."""
    dl, dr, page, NS = 128, 16, 16, 2           # 12 heads: one 16-head group; 24: two share a K tile; 72: four + a partial block
    D = dl + dr
    n_seq, max_pages, ctx = 2, 8, 100
    g = torch.Generator().manual_seed(11)
    cache = (torch.randn(n_seq * max_pages * page, D, generator=g) * 0.5).to(torch.bfloat16)
    bt = torch.arange(n_seq * max_pages, dtype=torch.int32).view(n_seq, max_pages).flip(1).contiguous()   # pages out of order
    q = (torch.randn(R, H, D, generator=g) * 0.5).to(torch.bfloat16)
    row_seq = torch.tensor([i % n_seq for i in range(R)], dtype=torch.int32)
    row_len = torch.tensor([1 + (7 * i) % ctx for i in range(R)], dtype=torch.int32)
    sel_ld = 48
    sel_idx = torch.full((R, sel_ld), -1, dtype=torch.int32)
    sel_cnt = torch.zeros(R, dtype=torch.int32)
    if sparse:
        for i in range(R):
            n = int(row_len[i])
            pick = torch.randperm(n, generator=g)[: min(n, 5 + (3 * i) % 40)]
            sel_idx[i, : len(pick)] = pick.int()
            sel_cnt[i] = len(pick)
    out = torch.zeros(R, H, dl, dtype=torch.bfloat16, device=DEV)
    o_part = torch.zeros(R, H, NS, dl, device=DEV)
    ml_part = torch.zeros(R, H, NS, 2, device=DEV)
    scale = D ** -0.5
    nat.call("lsb_mla_decode", q.to(DEV), cache.to(DEV).view(torch.uint8), bt.to(DEV), max_pages, row_seq.to(DEV), row_len.to(DEV),
             sel_idx.to(DEV) if sparse else None, sel_cnt.to(DEV) if sparse else None, sel_ld if sparse else 0, out, None, o_part, ml_part,
             R, H, dl, dr, page, 0, NS, scale, None)
    torch.cuda.synchronize()
    cf, qf = cache.float(), q.float()
    for i in range(R):
        pos = sel_idx[i, : int(sel_cnt[i])].long() if sparse else torch.arange(int(row_len[i]))
        rows = bt[int(row_seq[i])].long()[pos // page] * page + pos % page
        k = cf[rows]
        pr = torch.softmax(qf[i] @ k.T * scale, -1)
        close(out[i], pr @ k[:, :dl], 2e-2, 2e-2, f"mla attention row {i}")


def test_sampling_kernels():
    R, V = 4, 5000
    logits = rnd(R, V, s=3.0)
    part = torch.zeros(R, 64, dtype=torch.int64, device=DEV)
    ids = torch.zeros(R, dtype=torch.int32, device=DEV)
    val = torch.zeros(R, device=DEV)
    logits[1, 17] = logits[1, 4000] = 50.0
    nat.call("lsb_argmax", logits, V, R, V, part, ids, val, 0, None)
    torch.cuda.synchronize()
    assert ids.cpu().tolist() == [int(t) for t in logits.cpu().argmax(-1)[:1]] + [17] + [int(t) for t in logits.cpu().argmax(-1)[2:]]
    close(val, logits.max(-1).values, 0, 0, "argmax value")
    top1 = torch.zeros(R, device=DEV); ent = torch.zeros(R, device=DEV)
    nat.call("lsb_confidence", logits, V, R, V, top1, ent)
    p = torch.softmax(logits.cpu(), -1)
    torch.cuda.synchronize()
    close(top1, p.max(-1).values, 1e-3, 1e-6, "top1")
    close(ent, -(p * torch.log(p.clamp_min(1e-30))).sum(-1) / math.log(V), 1e-3, 1e-5, "entropy")
    # top-k=1 sampling is argmax; the same seed repeats; top-p keeps the draw inside the nucleus
    out = torch.zeros(R, dtype=torch.int32, device=DEV)
    logits[1, 4000] = 49.0               # exact ties at the k-th value are all kept, so break the tie
    nat.call("lsb_sample", logits, V, R, V, 1.0, 1, 1.0, 123, None, out)
    torch.cuda.synchronize()
    assert out.cpu().tolist() == ids.cpu().tolist()
    a = torch.zeros(R, dtype=torch.int32, device=DEV); b = torch.zeros(R, dtype=torch.int32, device=DEV)
    nat.call("lsb_sample", logits, V, R, V, 0.8, 50, 0.9, 7, None, a)
    nat.call("lsb_sample", logits, V, R, V, 0.8, 50, 0.9, 7, None, b)
    torch.cuda.synchronize()
    assert torch.equal(a, b)
    top50 = logits.cpu().topk(50, -1).indices
    for r in range(R):
        assert int(a[r]) in top50[r].tolist()
    # distribution check on a small vocabulary
    lg = torch.tensor([[0.0, 1.0, 2.0, 3.0]], device=DEV).repeat(2000, 1).contiguous()
    offs = torch.arange(2000, dtype=torch.int64, device=DEV)
    o = torch.zeros(2000, dtype=torch.int32, device=DEV)
    nat.call("lsb_sample", lg, 4, 2000, 4, 1.0, 0, 1.0, 99, offs, o)
    torch.cuda.synchronize()
    freq = torch.bincount(o.cpu().long(), minlength=4).float() / 2000
    close(freq, torch.softmax(lg[0].cpu(), -1), 0.0, 0.04, "sample distribution")
    # verify
    d = torch.tensor([5, 6, 7, 8], dtype=torch.int32, device=DEV)
    t = torch.tensor([5, 6, 9, 8, 1], dtype=torch.int32, device=DEV)
    res = torch.zeros(2, dtype=torch.int32, device=DEV)
    nat.call("lsb_spec_verify", d, t, 4, res)
    torch.cuda.synchronize()
    assert res.cpu().tolist() == [2, 9]


@pytest.mark.parametrize("M", [1, 4, 40])
def test_q4k_linear_gemv_and_tensor_core(M):
    """GGUF Q4_K weights: decode GEMV (M <= 4) and the tensor-core path (M >= 16) against the container codec's dequantisation."""
    from layerstorm_b200.models.device_model import QLinear
    g = torch.Generator().manual_seed(21)
    N, K = 256, 512
    lin = QLinear.from_float(torch.randn(N, K, generator=g) * 0.05, "gguf_q4_k", "cuda")
    assert lin.w.shape == (N, K // 256 * 144)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    ref = x.float() @ lin.dequant().float().T
    out = torch.zeros(M, N, device="cuda")
    lin(out, x, M)
    torch.cuda.synchronize()
    assert float((out - ref).abs().max() / ref.abs().max()) < 3e-3
    rnd = QLinear.random(N, K, "gguf_q4_k", "cuda")
    wd = rnd.dequant()
    assert torch.isfinite(wd).all() and 0.005 < float(wd.std()) < 0.08


def test_mhc_many_row_pass_is_reproducible_run_to_run():
    """The many-row hyper-connection pass updates the residual streams in place while all four warps of a block read them: the same
    inputs must give the same bits every time (a missing block barrier showed up as a handful of differing rows per 2048-row chunk)."""
    cfg = get_preset("tiny-glm5-next")
    H, n, R = 1024, cfg.hc_mult, 1024
    fn, sc, base, nw = rnd(24, n * H, s=0.05), torch.tensor([0.7, 1.1, 1.3], device=DEV), rnd(24, s=0.5), rnd(H) * 0.1 + 1
    sub = rnd(R, H)
    resid0, post0, comb0 = rnd(R, n, H), torch.rand(R, n, device=DEV), torch.rand(R, n, n, device=DEV)
    part = torch.zeros(R, H // 32, 36, device=DEV)
    args = (cfg.hc_sinkhorn_iters, cfg.hc_eps, cfg.rms_eps, cfg.hc_post_mult)
    outs = []
    for _ in range(12):
        resid, post, comb = resid0.clone(), post0.clone(), comb0.clone()
        x = torch.zeros(R, H, device=DEV, dtype=torch.bfloat16)
        nat.call("lsb_mhc_post_pre", x, resid, sub, post, comb, fn, sc, base, nw, part, R, H, n, 1, *args, None, None, None)
        torch.cuda.synchronize()
        outs.append((x.clone(), resid, post, comb))
    for o_ in outs[1:]:
        for a, b in zip(outs[0], o_):
            assert torch.equal(a, b)


def test_many_row_fp32_matrix_runs_as_split_bf16_tensor_core_gemm():
    """The router projection of a prefill chunk: fp32 weights split into bf16 hi + lo halves, one tcgen05 GEMM over the stacked halves.
    Must agree with the fp32 product far below the spacing of router logits (the few-row path reads the fp32 weights directly)."""
    from layerstorm_b200.models.device_model import QLinear
    N, K, M = 288, 1024, 300
    W = QLinear("f32", N, K, rnd(N, K, s=0.1))
    x = rnd(M, K).to(torch.bfloat16)
    out = torch.zeros(M, N, device=DEV)
    W(out, x, M)
    torch.cuda.synchronize()
    assert getattr(W, "_hilo", None) is not None and tuple(W._hilo.shape) == (2 * N, K)       # the tensor-core path ran
    ref = x.double() @ W.w.double().t()
    assert (out.double() - ref).abs().max().item() < 2e-5 * ref.abs().max().item()
    few = torch.zeros(4, N, device=DEV)
    W(few, x[:4].contiguous(), 4)
    torch.cuda.synchronize()
    assert (few - out[:4]).abs().max().item() < 2e-5 * ref.abs().max().item()


@pytest.mark.parametrize("R,IH,pos0", [(200, 32, 2000), (130, 4, 37), (70, 64, 900), (2048, 32, 6144), (1, 32, 5000), (3, 64, 777)])
def test_indexer_scores_on_tensor_cores_match_the_cuda_core_kernel(R, IH, pos0):
    """A single-sequence prefill chunk: the tcgen05 scoring (keys gathered to bf16, one GEMM, ReLU / head weights / head sum in the
    epilogue) against the one-thread-per-(row, entry) kernel on the same paged FP8 index cache, for every causal (row, entry)."""
    from layerstorm_b200.models.device_model import TcScratch
    P, page_e = 4, 16                                        # 4 tokens per pooled entry, 16 entries per page
    g = torch.Generator(device=DEV).manual_seed(R + IH)
    ne = torch.tensor([(pos0 + r + 1) // P for r in range(R)], dtype=torch.int32, device=DEV)
    ne_max = int(ne[-1])
    n_pages = (ne_max + page_e - 1) // page_e + 2
    cache = torch.zeros(n_pages, page_e, 144, dtype=torch.uint8, device=DEV)
    cache[:, :, :128] = torch.randint(0, 256, (n_pages, page_e, 128), device=DEV, generator=g, dtype=torch.uint8) & 0x77   # finite e4m3
    cache[:, :, 128:132] = (torch.rand(n_pages, page_e, 1, device=DEV, generator=g) * 0.05 + 0.01).view(torch.uint8)
    perm = torch.randperm(n_pages, device=DEV, generator=g).int()
    bt = perm.view(1, n_pages).contiguous()                  # one sequence, scattered pages
    q = rnd(R, IH, 128).to(torch.bfloat16)
    w = rnd(R, IH)
    row_seq = torch.zeros(R, dtype=torch.int32, device=DEV)
    ld = (ne_max + 127) // 128 * 128 + 64
    ref = torch.full((R, ld), -7.0, device=DEV)
    out = torch.full((R, ld), -7.0, device=DEV)
    nat.call("lsb_indexer_score", q, w, IH, cache, bt, n_pages, page_e, row_seq, ne, ref, ld, R, ld)
    kbf_rows = (ld + 127) // 128 * 128
    kbf = torch.zeros(kbf_rows, 128, dtype=torch.bfloat16, device=DEV)
    ksc = torch.zeros(kbf_rows, device=DEV)
    err = TcScratch.get(DEV).err
    err.zero_()
    nat.call("lsb_indexer_score_tc", q, w, IH, cache, bt, n_pages, page_e, row_seq, ne, out, ld, R, ne_max, kbf, kbf_rows, ksc, err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    mask = torch.arange(ld, device=DEV)[None, :] < ne[:, None]
    assert torch.equal(out[~mask], ref[~mask])              # nothing written beyond a row's causal frontier
    d = (out[mask] - ref[mask]).abs().max().item()
    assert d < 2e-4 * ref[mask].abs().max().item() + 1e-6, d
    if R <= 4:
        # a decode step under a CUDA graph sizes the grids for the row's CAPACITY, not its fill: same scores, nothing beyond the fill
        out2 = torch.full((R, ld), -7.0, device=DEV)
        nat.call("lsb_indexer_score_tc", q, w, IH, cache, bt, n_pages, page_e, row_seq, ne, out2, ld, R, min(ld, kbf_rows), kbf, kbf_rows, ksc, err)
        torch.cuda.synchronize()
        assert int(err.item()) == 0 and torch.equal(out2, out)


@pytest.mark.parametrize("P,budget,kind", [(4, 512, "normal"), (1, 2048, "normal"), (4, 512, "relu"), (4, 512, "const")])
def test_split_top_k_selection_equals_the_single_block_kernel(P, budget, kind):
    """Long index rows: the selection spread over many blocks (three histogram launches, count, emit) gives the single-block
    kernel's output entry for entry - ascending order, ties to the lower index, tail tokens, count - also for rows shorter than
    the budget, unused rows, rows full of equal scores, and on a second call over the scratch the first one left behind."""
    g = torch.Generator(device=DEV).manual_seed(11)
    ne_list = [70001, budget - 3, 262144, 9000, 0, 2048 * 3]
    R = len(ne_list)
    ld = 262144 + 8
    sc = torch.randn(R, ld, device=DEV, generator=g)
    if kind == "relu":
        sc = (sc - 2.2).clamp_min(0)                          # most scores are exactly zero, as after the indexer's ReLU
    elif kind == "const":
        sc.fill_(0.25)
    ne = torch.tensor(ne_list, dtype=torch.int32, device=DEV)
    row_len = (ne * P + torch.tensor([1, 0, 3, 2, 0, 0], device=DEV).clamp_max(P - 1)).int()
    row_seq = torch.tensor([0, 1, 2, 3, -1, 4], dtype=torch.int32, device=DEV)
    sel_ld = budget * P + P
    ref_idx = torch.full((R, sel_ld), -1, dtype=torch.int32, device=DEV)
    ref_cnt = torch.full((R,), -1, dtype=torch.int32, device=DEV)
    nat.call("lsb_indexer_topk", sc, ld, ne, row_len, row_seq, budget, P, ref_idx, ref_cnt, sel_ld, R)
    scratch = torch.zeros((int(nat.call("lsb_indexer_topk_split_scratch", R, ld)) + 3) // 4, dtype=torch.int32, device=DEV)
    for _ in range(2):
        idx = torch.full((R, sel_ld), -1, dtype=torch.int32, device=DEV)
        cnt = torch.full((R,), -1, dtype=torch.int32, device=DEV)
        nat.call("lsb_indexer_topk_split", sc, ld, ne, row_len, row_seq, budget, P, idx, cnt, sel_ld, R, ld, scratch)
        torch.cuda.synchronize()
        assert torch.equal(cnt, ref_cnt), (cnt.tolist(), ref_cnt.tolist())
        assert torch.equal(idx, ref_idx)
    # and against a sort: the budget best entries of the longest row
    r = 2
    order = torch.sort(sc[r, :ne_list[r]], descending=True, stable=True).indices[:budget].sort().values
    got = ref_idx[r, : budget * P].view(budget, P)[:, 0] // P
    assert torch.equal(got.long(), order)


@pytest.mark.parametrize("R,IH,page_e,ne_list", [(1, 32, 16, [5000]), (3, 64, 16, [777, 4100, 129]), (2, 32, 64, [3000, 2]), (1, 4, 8, [1000])])
def test_fp8_indexer_scores_over_the_cached_keys_match_the_cuda_core_kernel(R, IH, page_e, ne_list):
    """Few-row steps over long index rows: keys by TMA straight from the paged FP8 cache, query heads quantised to E4M3 per head,
    tcgen05.mma kind::f8f6f4, scale / ReLU / head weights / head sum in the epilogue - against the CUDA-core kernel (bf16 queries)
    over the same cache: within the query's FP8 rounding, nothing written beyond a row's fill, the same top entries."""
    from layerstorm_b200.models.device_model import TcScratch
    g = torch.Generator(device=DEV).manual_seed(R * 100 + IH)
    ne = torch.tensor(ne_list, dtype=torch.int32, device=DEV)
    ne_max = max(ne_list)
    pages_per_seq = (ne_max + page_e - 1) // page_e + 1
    n_pages = R * pages_per_seq + 3
    cache = torch.zeros(n_pages, page_e, 144, dtype=torch.uint8, device=DEV)
    cache[:, :, :128] = torch.randint(0, 256, (n_pages, page_e, 128), device=DEV, generator=g, dtype=torch.uint8) & 0x77   # finite e4m3
    cache[:, :, 128:132] = (torch.rand(n_pages, page_e, 1, device=DEV, generator=g) * 0.05 + 0.01).view(torch.uint8)
    bt = torch.randperm(n_pages, device=DEV, generator=g)[: R * pages_per_seq].int().view(R, pages_per_seq).contiguous()   # every sequence its own scattered pages
    q = rnd(R, IH, 128).to(torch.bfloat16)
    w = rnd(R, IH)
    row_seq = torch.arange(R, dtype=torch.int32, device=DEV)
    ld = (ne_max + 127) // 128 * 128 + 64
    ref = torch.full((R, ld), -7.0, device=DEV)
    out = torch.full((R, ld), -7.0, device=DEV)
    nat.call("lsb_indexer_score", q, w, IH, cache, bt, pages_per_seq, page_e, row_seq, ne, ref, ld, R, ld)
    err = TcScratch.get(DEV).err
    err.zero_()
    nat.call("lsb_indexer_score_f8", q, w, IH, cache, n_pages, bt, pages_per_seq, page_e, row_seq, ne, out, ld, R, ld, err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    mask = torch.arange(ld, device=DEV)[None, :] < ne[:, None]
    assert torch.equal(out[~mask], ref[~mask])              # nothing written beyond a row's fill
    for r in range(R):
        a, b = out[r, : ne_list[r]], ref[r, : ne_list[r]]
        assert torch.isfinite(a).all()
        # the query heads are rounded to E4M3 (3 mantissa bits): a few percent in RMS (signed head weights cancel signal, not error)
        assert float((a - b).norm() / (b.norm() + 1e-9)) < 0.06, (r, float((a - b).norm() / b.norm()))
        assert (a - b).abs().max().item() < 0.1 * b.abs().max().item() + 1e-6, (r, (a - b).abs().max().item(), b.abs().max().item())
        if ne_list[r] >= 512:
            k = 64
            ta, tb = set(a.topk(k).indices.tolist()), set(b.topk(k).indices.tolist())
            assert len(ta & tb) >= 0.8 * k, len(ta & tb)
