"""Tensor-core grouped expert FFN (sort -> gather -> gate/up+SwiGLU -> down) against an fp32
PyTorch reference built from the same (de-quantised) expert slots."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(fmt, H, F, E, n_missing, seed):
    from layerstorm_b200.models.device_model import ExpertArena, QLinear, expert_layout
    dev = torch.device("cuda")
    g = torch.Generator(device="cpu").manual_seed(seed)
    ef = expert_layout(fmt, H, F)
    arena = ExpertArena(ef, E - n_missing, E, dev)
    ref = {}
    slot = 0
    for e in range(E):
        if e < n_missing:
            continue                                   # experts 0..n_missing-1 are not resident
        mats = [torch.randn(F, H, generator=g) * 0.05, torch.randn(F, H, generator=g) * 0.05, torch.randn(H, F, generator=g) * 0.05]
        arena.write_expert(slot, *(QLinear.from_float(m.to(dev), fmt, dev) for m in mats))
        arena.slot_of[e] = slot
        ref[e] = [m.double().cpu() for m in arena.read_expert(slot, fmt)]
        slot += 1
    return arena, ref


@pytest.mark.parametrize("fmt", ["nvfp4", "fp8_e4m3", "bf16", "gguf_q4_k"])
@pytest.mark.parametrize("BN,R", [(32, 40), (64, 150), (128, 300)])
def test_grouped_ffn_matches_reference(fmt, BN, R):
    from layerstorm_b200.ops import _native as nat
    dev = torch.device("cuda")
    H, F, E, S, limit = 256, (256 if fmt == "gguf_q4_k" else 128), 6, 3, 7.0
    arena, ref = _setup(fmt, H, F, E, n_missing=1, seed=1)
    g = torch.Generator(device="cpu").manual_seed(2)
    x = (torch.randn(R, H, generator=g) * 1.5).to(torch.bfloat16).to(dev)
    # skewed routing: expert E-1 gets every row (like a shared expert), the others are random; a few invalid ids
    ids = torch.stack([torch.randint(0, E - 1, (R,), generator=g), torch.randint(0, E - 1, (R,), generator=g), torch.full((R,), E - 1)], 1).int()
    ids[3, 0] = -1
    ids = ids.to(dev).contiguous()
    P = R * S
    i32 = dict(dtype=torch.int32, device=dev)
    tiles = P // BN + E + 1
    srt, te, tr, tn, cnt = (torch.zeros(P, **i32), torch.zeros(tiles, **i32), torch.zeros(tiles, **i32), torch.zeros(tiles, **i32), torch.zeros(2, **i32))
    xs = torch.zeros(P, H, dtype=torch.float16, device=dev)
    act = torch.zeros(P, F, dtype=torch.float16, device=dev)
    y = torch.full((P, H), float("nan"), device=dev)
    err, miss = torch.zeros(1, **i32), torch.zeros(1, **i32)
    efp = ctypes.addressof(arena.ef)
    for _ in range(2):                                  # twice: barriers, TMEM and scratch are reusable
        nat.call("lsb_moe_tc_sort", ids, P, E, BN, srt, te, tr, tn, cnt)
        nat.call("lsb_moe_tc_gather", x, srt, cnt, xs, P, S, H)
        nat.call("lsb_moe_tc_ffn", 1, xs, P, arena.data, arena.slot_of, efp, te, tr, tn, cnt, srt, act, BN, tiles, limit, miss, err, None)
        nat.call("lsb_moe_tc_ffn", 0, act, P, arena.data, arena.slot_of, efp, te, tr, tn, cnt, srt, y, BN, tiles, 0.0, None, err, None)
    torch.cuda.synchronize()
    assert int(err) == 0
    assert int(miss) == 1                               # expert 0 (+1) was routed to but is not resident
    n_valid = int((ids >= 0).sum())
    assert int(cnt[1]) == n_valid
    # the sort is a permutation of the valid pairs, grouped by expert
    sp = srt[:n_valid].cpu()
    assert sorted(sp.tolist()) == [i for i in range(P) if int(ids.view(-1)[i]) >= 0]
    es = ids.view(-1).cpu()[sp]
    assert torch.all(es[1:] >= es[:-1])
    # numerics
    xd = x.double().cpu()
    idc = ids.cpu()
    worst = 0.0
    for r in range(R):
        for s in range(S):
            e = int(idc[r, s])
            if e < 1:
                continue
            gate, up, down = ref[e]
            gv = torch.clamp(gate @ xd[r], max=limit)
            uv = torch.clamp(up @ xd[r], -limit, limit)
            want = down @ (torch.nn.functional.silu(gv) * uv)
            got = y[r * S + s].double().cpu()
            worst = max(worst, float((got - want).abs().max() / (want.abs().max() + 1e-6)))
    assert worst < 6e-3, worst


def test_engine_prefill_uses_grouped_path_and_matches_oracle():
    """Long enough chunks => the routed experts run on the tensor-core path; logits still match the fp32 oracle
    and the short-chunk (weight-streaming) path."""
    from layerstorm_b200.models.config import get_preset
    from layerstorm_b200.models.device_model import DeviceModel, TC_MOE_MIN_ROWS
    from layerstorm_b200.models.reference import Oracle
    from layerstorm_b200.models.weights import init_weights
    from layerstorm_b200.runtime.engine import Engine
    for name, eq in (("tiny-mla-moe", "bf16"), ("tiny-glm5-next", "nvfp4")):
        cfg = get_preset(name)
        m = DeviceModel.from_state_dict(cfg, init_weights(cfg, 5), "cuda", kv_fmt="bf16", page=16, expert_quant=eq)
        oracle = Oracle(cfg, m.effective_state_dict())
        g = torch.Generator().manual_seed(0)
        T = 30
        prompt = torch.randint(0, cfg.vocab, (T,), generator=g)
        want = oracle.forward(prompt)[T - 1]
        outs = []
        for chunk in (64, 8):                           # 64: one tensor-core chunk; 8: GEMV chunks
            assert (chunk >= TC_MOE_MIN_ROWS) == (chunk == 64)
            eng = Engine(m, max_seqs=2, max_ctx=256, prefill_chunk=chunk, use_graph=False)
            sid = eng.create_sequence()
            nxt, lg = eng.prefill(sid, prompt.tolist(), want_logits=True)
            assert nxt == int(want.argmax()), (name, chunk)
            assert float((lg - want).abs().max() / want.abs().max()) < 3e-2, (name, chunk)
            outs.append(lg)
            eng.free_sequence(sid)
        assert float((outs[0] - outs[1]).abs().max() / outs[1].abs().max()) < 2e-2
