"""Block-scaled FP8 x FP8 tensor-core path (tcgen05.mma kind::mxf8f6f4, E4M3 values, one UE8M0 scale per 32 reduction elements):
activation quantisation, dense GEMM over FP8 weights with power-of-two 128 x 128 block scales, grouped expert FFN, a model prefill.

As for the NVFP4 path the GEMM is checked against a plain fp64 matmul of the SAME de-quantised operands (the products are exact in
fp32; only the summation order differs), the quantiser against its own definition.
"""
import ctypes
import dataclasses

import pytest
import torch

pytestmark = pytest.mark.gpu


def _dequant_tiles(q, sf, K, BN, ntiles):
    """[ntiles * BN, K] fp32 from the tile-order FP8 operand (scale atoms: tile t owns atom row t for BN <= 128)."""
    dev = q.device
    rows = ntiles * BN
    vals = q[:rows].view(torch.float8_e4m3fn).float()
    G = K // 32
    gt = (G + 3) // 4
    r = torch.arange(rows, device=dev)
    t, j = r // BN, r % BN
    g = torch.arange(G, device=dev)
    off = (t[:, None] * gt + g[None, :] // 4) * 512 + (j[:, None] % 32) * 16 + (j[:, None] // 32) * 4 + g[None, :] % 4
    s = torch.exp2(sf[off.reshape(-1)].float() - 127.0).view(rows, G)
    return (vals.view(rows, G, 32) * s[:, :, None]).view(rows, K)


def _dense_tiles(M, BN, dev):
    n = (M + BN - 1) // BN
    r0 = torch.arange(n, dtype=torch.int32, device=dev) * BN
    tn = torch.clamp(M - r0, max=BN).int()
    cnt = torch.tensor([n, M], dtype=torch.int32, device=dev)
    return n, r0, tn, cnt


@pytest.mark.parametrize("M,K,BN", [(200, 512, 128), (70, 256, 64), (40, 4096, 32), (130, 7168, 64)])
def test_fp8_activation_quantiser(M, K, BN):
    from layerstorm_b200.ops import _native as nat
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(3)
    x = (torch.randn(M, K, device=dev, generator=g) * torch.rand(M, 1, device=dev, generator=g) * 3).to(torch.bfloat16)
    x[1] = 0                                                        # an all-zero row stays zero and finite
    x[2, :32] = 448.0 * 4                                           # a group whose largest value sits exactly on a power of two times 448
    n, r0, tn, cnt = _dense_tiles(M, BN, dev)
    q = torch.zeros(n * BN, K, dtype=torch.uint8, device=dev)
    sf = torch.full((n * (K // 128) * 512,), 77, dtype=torch.uint8, device=dev)
    al = torch.zeros(n * BN, device=dev)
    nat.call("lsb_quant_fp8_tiles", x, 2, None, r0, tn, cnt, 1, K, BN, n, q, sf, al)
    torch.cuda.synchronize()
    d = _dequant_tiles(q, sf, K, BN, n)
    rows = (torch.arange(M, device=dev) // BN) * BN + torch.arange(M, device=dev) % BN
    d = d[rows]
    xf = x.float()
    assert torch.isfinite(d).all() and torch.equal(al[rows], torch.ones(M, device=dev))
    assert torch.equal(d[1], torch.zeros_like(d[1]))
    assert torch.equal(d[2, :32], xf[2, :32])                       # 448 * 2^2: scale 2^2, value 448, exact
    # E4M3 with a power-of-two scale that puts the group's largest value in (224, 448]: 3 mantissa bits -> relative error <= 2^-4
    # per element (values far below the group's maximum lose more: compare against the group maximum too)
    err = (d - xf).abs()
    gmax = xf.view(M, K // 32, 32).abs().amax(dim=2, keepdim=True)
    assert (err.view(M, K // 32, 32) <= xf.view(M, K // 32, 32).abs() * 0.0626 + gmax * 2.0 ** -9 + 1e-12).all()
    assert (d - xf).norm() / xf.norm() < 0.045


@pytest.mark.parametrize("M,N,K,BN", [(200, 256, 512, 128), (70, 128, 256, 64), (40, 384, 1024, 32), (300, 512, 7168, 128)])
def test_dense_fp8_block_scaled_gemm_matches_fp64_of_same_operands(M, N, K, BN):
    from layerstorm_b200.models.device_model import QLinear, TcScratch
    from layerstorm_b200.ops import _native as nat
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(5)
    W = QLinear.random(N, K, "fp8_e4m3", dev, gen=g)
    # every 128 x 128 block its own power-of-two scale
    W.scales.copy_(torch.exp2(torch.randint(-8, -2, W.scales.shape, device=dev, generator=g).float()))
    atoms = W.bs_scale_atoms()
    assert atoms is not None and atoms.shape == ((N // 128) * (K // 128), 512)
    Wf = W.dequant()
    x = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
    n, r0, tn, cnt = _dense_tiles(M, BN, dev)
    q = torch.zeros(n * BN, K, dtype=torch.uint8, device=dev)
    sf = torch.zeros(n * (K // 128) * 512, dtype=torch.uint8, device=dev)
    al = torch.zeros(n * BN, device=dev)
    nat.call("lsb_quant_fp8_tiles", x, 2, None, r0, tn, cnt, 1, K, BN, n, q, sf, al)
    out = torch.zeros(M, N, device=dev)
    err = TcScratch.get(dev).err
    err.zero_()
    nat.call("lsb_gemm_fp8_bs", out, q, sf, al, W.w, atoms, N, K, N, 0, r0, tn, cnt, BN, n, err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    xd = _dequant_tiles(q, sf, K, BN, n)
    rows = (torch.arange(M, device=dev) // BN) * BN + torch.arange(M, device=dev) % BN
    ref = xd[rows].double() @ Wf.double().t()
    tol = 1e-4 * ref.abs().max().item() + 1e-6
    assert (out.double() - ref).abs().max().item() < tol, ((out.double() - ref).abs().max().item(), tol)
    full = x.float() @ Wf.t()
    assert (out - full).norm() / full.norm() < 0.045
    # a scale that is not a power of two has no UE8M0 form: the matrix stays on the other paths
    W2 = QLinear.random(128, 256, "fp8_e4m3", dev, gen=g)
    W2.scales.fill_(0.03)
    assert W2.bs_scale_atoms() is None


@pytest.mark.parametrize("R,BN", [(64, 32), (256, 64), (700, 128)])
def test_grouped_fp8_block_scaled_expert_ffn(R, BN):
    from layerstorm_b200.models.device_model import ExpertArena, TcScratch, expert_layout
    from layerstorm_b200.ops import _native as nat
    dev = torch.device("cuda", 0)
    H, F, E, S = 512, 256, 12, 3
    g = torch.Generator(device=dev).manual_seed(7)
    ef = expert_layout("fp8_e4m3", H, F)
    arena = ExpertArena(ef, E, E, dev)
    arena.data.zero_()
    arena.data[:, : ef.off_sg].random_(0, 256, generator=g)
    arena.data[:, : ef.off_sg] &= 0xBF
    sc = arena.data[:, ef.off_sg: ef.off_tail].view(torch.float32)
    sc.copy_(torch.exp2(torch.randint(-7, -3, sc.shape, device=dev, generator=g).float()))
    slot_of = torch.arange(E, dtype=torch.int32, device=dev)
    slot_of[5] = -1                                                  # one expert is not resident: its pairs are skipped
    arena.slot_of.copy_(slot_of)
    wsf, og, ou, od = arena.bs_scale_atoms()
    x = torch.randn(R, H, device=dev, generator=g).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(E, device=dev, generator=g)[:S] for _ in range(R)]).int().contiguous()
    P = R * S
    tiles = P // BN + E + 1
    i32 = dict(dtype=torch.int32, device=dev)
    sorted_pair, te, tr, tn, cnt = (torch.zeros(P, **i32), torch.zeros(tiles, **i32), torch.zeros(tiles, **i32), torch.zeros(tiles, **i32),
                                    torch.zeros(2, **i32))
    nat.call("lsb_moe_tc_sort", ids, P, E, BN, sorted_pair, te, tr, tn, cnt)
    u8 = torch.uint8
    xq, xsf, xa = torch.zeros(tiles * BN, H, dtype=u8, device=dev), torch.zeros(tiles * (H // 128) * 512, dtype=u8, device=dev), torch.zeros(tiles * BN, device=dev)
    act = torch.zeros(tiles * BN, F, dtype=torch.float16, device=dev)
    aq, asf, aa = torch.zeros(tiles * BN, F, dtype=u8, device=dev), torch.zeros(tiles * (F // 128) * 512, dtype=u8, device=dev), torch.zeros(tiles * BN, device=dev)
    y = torch.zeros(P, H, device=dev)
    err = TcScratch.get(dev).err
    err.zero_()
    miss = torch.zeros(1, **i32)
    efp = ctypes.addressof(arena.ef)
    a = (arena.data, arena.slot_of, efp, wsf, wsf.shape[1], og, ou, od, te, tr, tn, cnt, sorted_pair)
    limit = 7.0
    nat.call("lsb_quant_fp8_tiles", x, 0, sorted_pair, tr, tn, cnt, S, H, BN, tiles, xq, xsf, xa)
    nat.call("lsb_moe_bs_ffn_fp8", 1, xq, xsf, xa, *a, act, BN, tiles, limit, miss, err)
    nat.call("lsb_quant_fp8_tiles", act, 1, None, tr, tn, cnt, S, F, BN, tiles, aq, asf, aa)
    nat.call("lsb_moe_bs_ffn_fp8", 0, aq, asf, aa, *a, y, BN, tiles, 0.0, None, err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    assert int(miss.item()) == 6                                    # expert 5 (+1) reported missing
    nt = int(cnt[0].item())
    xd = _dequant_tiles(xq, xsf, H, BN, nt)
    ad = _dequant_tiles(aq, asf, F, BN, nt)
    te_h, tr_h, tn_h, sp_h = te.tolist(), tr.tolist(), tn.tolist(), sorted_pair.tolist()
    checked = 0
    for t in range(nt):
        e = te_h[t]
        if e == 5:
            continue
        gate, up, down = arena.read_expert(e, "fp8_e4m3")
        rows = slice(t * BN, t * BN + tn_h[t])
        src = torch.tensor([sp_h[tr_h[t] + j] // S for j in range(tn_h[t])], device=dev)
        assert (xd[rows] - x[src].float()).norm() / x[src].float().norm() < 0.045
        gv = torch.clamp(xd[rows].double() @ gate.double().t(), max=limit)
        uv = torch.clamp(xd[rows].double() @ up.double().t(), min=-limit, max=limit)
        ref_act = torch.nn.functional.silu(gv) * uv
        assert (act[rows].double() - ref_act).abs().max().item() < 2e-3 * ref_act.abs().max().item() + 1e-4
        ref_y = ad[rows].double() @ down.double().t()
        pairs = torch.tensor([sp_h[tr_h[t] + j] for j in range(tn_h[t])], device=dev)
        assert (y[pairs].double() - ref_y).abs().max().item() < 1e-4 * ref_y.abs().max().item() + 1e-6
        checked += tn_h[t]
    assert checked > 0


def test_model_prefill_with_fp8_block_scaled_experts_and_dense_layers(monkeypatch):
    """An FP8 model (experts and dense matrices, power-of-two block scales) prefills a prompt with the fp16-operand path and with
    the block-scaled path: the logits differ by the FP8 activation quantisation only, and the block-scaled path was the one in use."""
    from layerstorm_b200.models import device_model as dm
    from layerstorm_b200.models.config import get_preset
    from layerstorm_b200.models.weights import init_weights
    from layerstorm_b200.runtime.engine import Engine
    cfg = dataclasses.replace(get_preset("tiny-deepseek-v32"), moe_inter=256)
    w = init_weights(cfg, 0)
    m = dm.DeviceModel.from_state_dict(cfg, w, "cuda", kv_fmt="bf16", page=16, expert_quant="fp8_e4m3", dense_quant="fp8_e4m3")
    assert all(L["arena"].bs_scale_atoms() is not None for L in m.layers if "arena" in L)       # the quantiser writes power-of-two scales
    ids = torch.randint(0, cfg.vocab, (48,), generator=torch.Generator().manual_seed(11)).tolist()
    out = {}
    for flag in (False, True):
        monkeypatch.setattr(dm, "MOE_BLOCK_SCALED", flag)
        eng = Engine(m, max_seqs=1, max_ctx=128, prefill_chunk=32, max_batch=1, use_graph=False)
        sid = eng.create_sequence()
        _, lg = eng.prefill(sid, ids, want_logits=True)
        assert eng.ws_prefill.bs_ok == flag and (not flag or eng.ws_prefill.bs_fp8)
        out[flag] = lg.float().cpu()
        eng.free_sequence(sid)
    assert torch.isfinite(out[True]).all()
    rel = float((out[True] - out[False]).norm() / out[False].norm())
    assert 0 < rel < 0.08, rel
