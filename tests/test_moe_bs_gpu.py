"""Block-scaled NVFP4 x NVFP4 tensor-core path (tcgen05.mma kind::mxf4nvf4): activation quantisation and the grouped / dense GEMM.

The GEMM is checked against a plain fp32 matmul of the SAME de-quantised operands (products of two 4-bit values with their
scales are exact in fp32, so only the summation order differs); the quantiser against its own definition.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

from layerstorm_b200.formats import quant  # noqa: E402


def _need_gpu():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")


def _dequant_tiles(q, sf, alpha, K, BN, ntiles):
    """[ntiles * BN, K] fp32 from the tile-order NVFP4 operand (scale atoms: tile t owns atom row t for BN <= 128)."""
    dev = q.device
    rows = ntiles * BN
    lut = torch.tensor([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6], device=dev)
    lo, hi = (q[:rows] & 0xF).long(), (q[:rows] >> 4).long()
    vals = torch.stack([lut[lo], lut[hi]], dim=-1).reshape(rows, K)
    G = K // 16
    gt = (G + 3) // 4
    r = torch.arange(rows, device=dev)
    t, j = r // BN, r % BN
    g = torch.arange(G, device=dev)
    off = (t[:, None] * gt + g[None, :] // 4) * 512 + (j[:, None] % 32) * 16 + (j[:, None] // 32) * 4 + g[None, :] % 4
    s = sf[off.reshape(-1)].view(torch.float8_e4m3fn).float().view(rows, G)
    return (vals.view(rows, G, 16) * s[:, :, None]).view(rows, K) * alpha[:rows, None]


def _dense_tiles(M, BN, dev):
    n = (M + BN - 1) // BN
    r0 = torch.arange(n, dtype=torch.int32, device=dev) * BN
    tn = torch.clamp(M - r0, max=BN).int()
    cnt = torch.tensor([n, M], dtype=torch.int32, device=dev)
    return n, r0, tn, cnt


@pytest.mark.parametrize("M,K,BN", [(200, 512, 128), (70, 256, 64), (40, 4096, 32), (130, 2048, 64)])
def test_activation_quantiser(M, K, BN):
    _need_gpu()
    from layerstorm_b200.ops import _native as nat
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(3)
    x = (torch.randn(M, K, device=dev, generator=g) * torch.rand(M, 1, device=dev, generator=g) * 3).to(torch.bfloat16)
    x[1] = 0                                                        # an all-zero row stays zero and finite
    n, r0, tn, cnt = _dense_tiles(M, BN, dev)
    q = torch.zeros(n * BN, K // 2, dtype=torch.uint8, device=dev)
    sf = torch.zeros(n * (K // 64) * 512, dtype=torch.uint8, device=dev)
    al = torch.zeros(n * BN, device=dev)
    nat.call("lsb_quant_nvfp4_tiles", x, 2, None, r0, tn, cnt, 1, K, BN, n, q, sf, al)
    torch.cuda.synchronize()
    d = _dequant_tiles(q, sf, al, K, BN, n)
    rows = (torch.arange(M, device=dev) // BN) * BN + torch.arange(M, device=dev) % BN
    d = d[rows]
    xf = x.float()
    assert torch.isfinite(d).all()
    assert torch.equal(d[1], torch.zeros_like(d[1]))
    # per-row scale: the row's largest magnitude over (6 * 448)
    assert torch.allclose(al[rows][2:], xf[2:].abs().amax(dim=1) / (6 * 448), rtol=1e-6)
    # E2M1 with a per-16 scale: a few percent of the group's largest value per element, about a tenth in relative RMS
    rel = (d - xf).norm() / xf.norm()
    assert rel < 0.15, rel
    gmax = xf.view(M, K // 16, 16).abs().amax(dim=2, keepdim=True)
    assert ((d - xf).view(M, K // 16, 16).abs() <= gmax * 0.27 + 1e-6).all()


@pytest.mark.parametrize("M,N,K,BN", [(200, 256, 512, 128), (70, 128, 256, 64), (40, 384, 1024, 32), (300, 512, 4096, 128)])
def test_dense_block_scaled_gemm_matches_fp32_of_same_operands(M, N, K, BN):
    _need_gpu()
    from layerstorm_b200.models.device_model import QLinear, TcScratch
    from layerstorm_b200.ops import _native as nat
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(5)
    W = QLinear.random(N, K, "nvfp4", dev, gen=g)
    Wf = W.dequant()
    x = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
    n, r0, tn, cnt = _dense_tiles(M, BN, dev)
    q = torch.zeros(n * BN, K // 2, dtype=torch.uint8, device=dev)
    sf = torch.zeros(n * (K // 64) * 512, dtype=torch.uint8, device=dev)
    al = torch.zeros(n * BN, device=dev)
    nat.call("lsb_quant_nvfp4_tiles", x, 2, None, r0, tn, cnt, 1, K, BN, n, q, sf, al)
    out = torch.zeros(M, N, device=dev)
    err = TcScratch.get(dev).err
    err.zero_()
    nat.call("lsb_gemm_nvfp4_bs", out, q, sf, al, W.w, W.scales, W.alpha, N, K, N, 0, r0, tn, cnt, BN, n, err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    xd = _dequant_tiles(q, sf, al, K, BN, n)
    rows = (torch.arange(M, device=dev) // BN) * BN + torch.arange(M, device=dev) % BN
    ref = xd[rows].double() @ Wf.double().t()
    tol = 1e-4 * ref.abs().max().item() + 1e-6
    assert (out.double() - ref).abs().max().item() < tol, ((out.double() - ref).abs().max().item(), tol)
    # and the lossy part: against the bf16 activations the result is within the 4-bit quantisation noise
    full = x.float() @ Wf.t()
    assert (out - full).norm() / full.norm() < 0.15


@pytest.mark.parametrize("R,BN", [(64, 32), (256, 64), (700, 128)])
def test_grouped_block_scaled_expert_ffn(R, BN):
    _need_gpu()
    from layerstorm_b200.models.device_model import ExpertArena, TcScratch, expert_layout
    from layerstorm_b200.ops import _native as nat
    dev = torch.device("cuda", 0)
    H, F, E, S = 512, 256, 12, 3
    g = torch.Generator(device=dev).manual_seed(7)
    ef = expert_layout("nvfp4", H, F)
    arena = ExpertArena(ef, E, E, dev)
    arena.data.zero_()
    for e in range(E):
        v = arena.data[e]
        wq = v[: ef.off_sg]
        wq.random_(0, 256, generator=g)
        v[ef.off_sg: ef.off_tail].random_(0x30, 0x40, generator=g)
        v[ef.off_tail: ef.off_tail + 12].view(torch.float32).copy_(torch.tensor([0.011, 0.013, 0.009]) * (1 + 0.1 * e))
    slot_of = torch.arange(E, dtype=torch.int32, device=dev)
    slot_of[5] = -1                                                  # one expert is not resident: its pairs are skipped
    arena.slot_of.copy_(slot_of)
    x = torch.randn(R, H, device=dev, generator=g).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(E, device=dev, generator=g)[:S] for _ in range(R)]).int().contiguous()
    P = R * S
    tiles = P // BN + E + 1
    i32 = dict(dtype=torch.int32, device=dev)
    sorted_pair, te, tr, tn, cnt = (torch.zeros(P, **i32), torch.zeros(tiles, **i32), torch.zeros(tiles, **i32), torch.zeros(tiles, **i32),
                                    torch.zeros(2, **i32))
    nat.call("lsb_moe_tc_sort", ids, P, E, BN, sorted_pair, te, tr, tn, cnt)
    u8 = torch.uint8
    xq, xsf, xa = torch.zeros(tiles * BN, H // 2, dtype=u8, device=dev), torch.zeros(tiles * (H // 64) * 512, dtype=u8, device=dev), torch.zeros(tiles * BN, device=dev)
    act = torch.zeros(tiles * BN, F, dtype=torch.float16, device=dev)
    aq, asf, aa = torch.zeros(tiles * BN, F // 2, dtype=u8, device=dev), torch.zeros(tiles * (F // 64) * 512, dtype=u8, device=dev), torch.zeros(tiles * BN, device=dev)
    y = torch.zeros(P, H, device=dev)
    err = TcScratch.get(dev).err
    err.zero_()
    miss = torch.zeros(1, **i32)
    efp = ctypes.addressof(arena.ef)
    a = (arena.data, arena.slot_of, efp, te, tr, tn, cnt, sorted_pair)
    limit = 7.0
    nat.call("lsb_quant_nvfp4_tiles", x, 0, sorted_pair, tr, tn, cnt, S, H, BN, tiles, xq, xsf, xa)
    nat.call("lsb_moe_bs_ffn", 1, xq, xsf, xa, *a, act, BN, tiles, limit, miss, err)
    nat.call("lsb_quant_nvfp4_tiles", act, 1, None, tr, tn, cnt, S, F, BN, tiles, aq, asf, aa)
    nat.call("lsb_moe_bs_ffn", 0, aq, asf, aa, *a, y, BN, tiles, 0.0, None, err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    assert int(miss.item()) == 6                                    # expert 5 (+1) reported missing
    nt = int(cnt[0].item())
    xd = _dequant_tiles(xq, xsf, xa, H, BN, nt)
    ad = _dequant_tiles(aq, asf, aa, F, BN, nt)
    te_h, tr_h, tn_h, sp_h = te.tolist(), tr.tolist(), tn.tolist(), sorted_pair.tolist()
    checked = 0
    for t in range(nt):
        e = te_h[t]
        if e == 5:
            continue
        gate, up, down = arena.read_expert(e, "nvfp4")
        rows = slice(t * BN, t * BN + tn_h[t])
        # the quantised rows of the tile are the gathered token rows
        src = torch.tensor([sp_h[tr_h[t] + j] // S for j in range(tn_h[t])], device=dev)
        assert (xd[rows] - x[src].float()).norm() / x[src].float().norm() < 0.15
        gv = torch.clamp(xd[rows].double() @ gate.double().t(), max=limit)
        uv = torch.clamp(xd[rows].double() @ up.double().t(), min=-limit, max=limit)
        ref_act = torch.nn.functional.silu(gv) * uv
        assert (act[rows].double() - ref_act).abs().max().item() < 2e-3 * ref_act.abs().max().item() + 1e-4
        ref_y = ad[rows].double() @ down.double().t()
        pairs = torch.tensor([sp_h[tr_h[t] + j] for j in range(tn_h[t])], device=dev)
        assert (y[pairs].double() - ref_y).abs().max().item() < 1e-4 * ref_y.abs().max().item() + 1e-6
        checked += tn_h[t]
    assert checked > 0


def test_model_prefill_with_block_scaled_experts_stays_within_quantisation_noise(monkeypatch):
    """The same NVFP4-expert model prefills a prompt with the fp16-operand path and with the block-scaled path: the logits differ
    by the activation quantisation only, and the block-scaled kernels really ran (launcher count)."""
    _need_gpu()
    import dataclasses

    from layerstorm_b200.models import device_model as dm
    from layerstorm_b200.models.config import get_preset
    from layerstorm_b200.models.weights import init_weights
    from layerstorm_b200.ops import _native as nat
    from layerstorm_b200.runtime.engine import Engine
    cfg = dataclasses.replace(get_preset("tiny-glm5-next"), moe_inter=256)
    w = init_weights(cfg, 0)
    m = dm.DeviceModel.from_state_dict(cfg, w, "cuda", kv_fmt="bf16", page=16, expert_quant="nvfp4")
    ids = torch.randint(0, cfg.vocab, (48,), generator=torch.Generator().manual_seed(11)).tolist()
    out = {}
    for flag in (False, True):
        monkeypatch.setattr(dm, "MOE_BLOCK_SCALED", flag)
        eng = Engine(m, max_seqs=1, max_ctx=128, prefill_chunk=32, max_batch=1, use_graph=False)
        sid = eng.create_sequence()
        _, lg = eng.prefill(sid, ids, want_logits=True)
        assert eng.ws_prefill.bs_ok == flag
        out[flag] = lg.float().cpu()
        eng.free_sequence(sid)
    assert torch.isfinite(out[True]).all()
    rel = float((out[True] - out[False]).norm() / out[False].norm())
    assert 0 < rel < 0.12, rel
