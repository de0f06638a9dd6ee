"""Capped VRAM expert cache with pinned-host backing store: outputs are identical to the fully resident model,
experts move in waves when a step needs more of them than there are slots."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from layerstorm_b200.models.config import get_preset
from layerstorm_b200.models.device_model import DeviceModel
from layerstorm_b200.models.weights import init_weights
from layerstorm_b200.runtime.engine import Engine
from layerstorm_b200.runtime.streaming import ExpertStreamer


@pytest.mark.parametrize("name,eq", [("tiny-mla-moe", "bf16"), ("tiny-glm5-next", "nvfp4")])
def test_streamed_experts_match_resident_model(name, eq):
    cfg = get_preset(name)
    w = init_weights(cfg, 9)
    g = torch.Generator().manual_seed(4)
    prompt = torch.randint(0, cfg.vocab, (40,), generator=g).tolist()

    def run(streamed, chunk):
        m = DeviceModel.from_state_dict(cfg, w, "cuda", kv_fmt="bf16", page=16, expert_quant=eq)
        st = ExpertStreamer(m, slots_per_layer=cfg.top_k + cfg.n_shared + 1, prefetch=True) if streamed else None
        eng = Engine(m, max_seqs=1, max_ctx=128, prefill_chunk=chunk, max_batch=1, use_graph=False)
        sid = eng.create_sequence()
        nxt, lg = eng.prefill(sid, prompt, want_logits=True)
        toks = [nxt]
        for _ in range(6):
            toks.append(eng.decode([sid], [toks[-1]])[0])
        return toks, lg, st

    for chunk in (8, 32):                                  # 8: weight-streaming kernels; 32: tensor-core grouped path, several waves
        ref_t, ref_l, _ = run(False, chunk)
        got_t, got_l, st = run(True, chunk)
        assert got_t == ref_t, (chunk, got_t, ref_t)
        assert torch.equal(got_l, ref_l)                   # same kernels, same order of accumulation => same bits
        s = st.summary()
        assert s["misses"] > 0 and s["bytes_h2d"] > 0 and s["waves"] > cfg.n_moe_layers()
        for li, lst in st.layers.items():
            assert lst["arena"].n_slots == cfg.top_k + cfg.n_shared + 1
            assert lst["host"].is_pinned()


def test_fetch_deadline_finishes_the_step_degraded_and_recovers():
    """A copy whose completion is stalled (injected on the host: the completion query is made to answer 'not yet') misses the
    fetch deadline: the step finishes without that expert instead of waiting, the streamer counts it, and once the stall is
    lifted the late copy is published and the outputs equal the resident model's again."""
    cfg = get_preset("tiny-mla-moe")
    w = init_weights(cfg, 9)
    prompt = torch.randint(0, cfg.vocab, (24,), generator=torch.Generator().manual_seed(4)).tolist()

    def build(streamed):
        m = DeviceModel.from_state_dict(cfg, w, "cuda", kv_fmt="bf16", page=16, expert_quant="bf16")
        st = ExpertStreamer(m, slots_per_layer=cfg.top_k + cfg.n_shared + 1, fetch_deadline_ms=2.0) if streamed else None
        return Engine(m, max_seqs=1, max_ctx=128, prefill_chunk=8, max_batch=1, use_graph=False), st

    ref_eng, _ = build(False)
    sid = ref_eng.create_sequence()
    ref = [ref_eng.prefill(sid, prompt)]
    for _ in range(4):
        ref.append(ref_eng.decode([sid], [ref[-1]])[0])

    eng, st = build(True)
    sid = eng.create_sequence()
    got = [eng.prefill(sid, prompt)]
    assert got == ref[:1] and st.summary()["degraded_steps"] == 0 and st.summary()["host_waits"] > 0
    real = st._copy_done
    st._copy_done = lambda ev: False                       # every completion now looks stalled
    eng.decode([sid], [got[-1]])                           # must return (degraded), not hang
    s = st.summary()
    stalled = s["late_experts"]
    st._copy_done = real                                    # the stall is lifted: late copies are published on the next use
    eng.free_sequence(sid)
    sid = eng.create_sequence()
    again = [eng.prefill(sid, prompt)]
    for _ in range(4):
        again.append(eng.decode([sid], [again[-1]])[0])
    assert again == ref
    assert not st._late and (stalled == 0 or s["degraded_steps"] >= 1)


def test_layer_by_layer_loading_prewarm_and_fetch_trace(tmp_path, monkeypatch):
    """The streamer as the model's layer hook: every MoE layer's experts leave HBM as soon as the layer is built (a model larger
    than HBM loads this way), the steps give the resident model's tokens, a demand-fetch table pre-warms the cache, and the copy
    batches land in the fetch trace with device times the cost-model fit can read."""
    from layerstorm_b200.utils import loader_xray as lx
    cfg = get_preset("tiny-mla-moe")
    w = init_weights(cfg, 9)
    prompt = torch.randint(0, cfg.vocab, (40,), generator=torch.Generator().manual_seed(4)).tolist()
    m0 = DeviceModel.from_state_dict(cfg, w, "cuda", kv_fmt="bf16", page=16, expert_quant="bf16")
    e0 = Engine(m0, max_seqs=1, max_ctx=128, prefill_chunk=8, max_batch=1, use_graph=False)
    sid = e0.create_sequence()
    ref = [e0.prefill(sid, prompt)]
    for _ in range(5):
        ref.append(e0.decode([sid], [ref[-1]])[0])

    ftrace, rtrace = tmp_path / "fetch.txt", tmp_path / "routing.txt"
    monkeypatch.setenv("LS_FETCH_TRACE", str(ftrace))
    monkeypatch.setenv("LS_ROUTING_TRACE", str(rtrace))
    slots = cfg.top_k + cfg.n_shared + 2

    def run(place_freq=None):
        st = ExpertStreamer(None, slots_per_layer=slots, prefetch=False, cfg=cfg, device="cuda", place_freq=place_freq)
        built = []
        hook = lambda i, L: (built.append((i, L["arena"].n_slots if "arena" in L else 0)), st.add_layer(i, L))
        m = DeviceModel.from_state_dict(cfg, w, "cuda", kv_fmt="bf16", page=16, expert_quant="bf16", layer_hook=hook)
        # at hook time each MoE layer still had its full arena; afterwards only the capped one is left
        assert all(n in (0, cfg.n_routed + cfg.n_shared) for _, n in built) and len(built) == cfg.n_layers
        assert all(L["arena"].n_slots == slots for L in m.layers if "arena" in L)
        st.attach(m)
        eng = Engine(m, max_seqs=1, max_ctx=128, prefill_chunk=8, max_batch=1, use_graph=False)
        sid = eng.create_sequence()
        got = [eng.prefill(sid, prompt)]
        for _ in range(5):
            got.append(eng.decode([sid], [got[-1]])[0])
        return got, st

    got, st = run()
    assert got == ref
    s = st.summary()                                       # also flushes the fetch trace
    st.trace.close()
    assert s["misses"] > 0
    batches = lx.read_fetch_trace(str(ftrace))
    assert len(batches) > 3 and (batches[:, 1] > 0).all() and (batches[:, 2] > 0).all()
    assert int(batches[:, 1].sum()) == s["bytes_h2d"]
    table = str(tmp_path / "freq.csv")
    from layerstorm_b200.utils.cache_sim import read_trace
    lx.write_freq_table(table, lx.fetch_counts([read_trace(str(rtrace))], slots, skip_steps=0), "test")
    got2, st2 = run(place_freq=table)
    assert got2 == ref
    s2 = st2.summary()
    assert s2["bytes_h2d"] > 0 and sum(len(l["host_row"]) for l in st2.layers.values()) > 0
    # the pre-warmed run starts with the most-fetched experts resident: fewer demand misses than the cold run
    assert s2["misses"] <= s["misses"]


def test_missed_experts_can_run_on_the_host_kernels_instead_of_being_fetched():
    """CPU offload under a capped cache: with the host made to look fast, a decode step's missed experts are computed by the host
    kernels from the pinned slot images and added after the combine; with the host made to look slow nothing is offloaded.  The
    logits stay within the precision of the two expert implementations and the greedy tokens agree with the resident model."""
    cfg = get_preset("tiny-mla-moe")
    w = init_weights(cfg, 9)
    prompt = torch.randint(0, cfg.vocab, (24,), generator=torch.Generator().manual_seed(4)).tolist()

    def run(offload, cpu_ms=None):
        m = DeviceModel.from_state_dict(cfg, w, "cuda", kv_fmt="bf16", page=16, expert_quant="bf16")
        st = ExpertStreamer(m, slots_per_layer=cfg.top_k + cfg.n_shared + 1, cpu_offload=True) if offload else None
        if st is not None and cpu_ms is not None:
            st._cpu_ms = cpu_ms
        eng = Engine(m, max_seqs=1, max_ctx=128, prefill_chunk=8, max_batch=1, use_graph=False)
        sid = eng.create_sequence()
        toks, lgs = [eng.prefill(sid, prompt)], []
        for _ in range(6):
            out, lg = eng.decode([sid], [toks[-1]], return_logits=True)
            toks.append(out[0])
            lgs.append(lg[0].clone())
        return toks, torch.stack(lgs), st

    ref_t, ref_l, _ = run(False)
    fast_t, fast_l, st = run(True, cpu_ms=1e-6)             # the host looks free: every missed expert of a decode step goes to it
    s = st.summary()
    assert s["cpu_experts"] > 0 and st.cpu.threads >= 1
    rel = float((fast_l - ref_l).abs().max() / ref_l.abs().max())
    assert rel < 2e-2, rel
    assert fast_t == ref_t
    slow_t, slow_l, st2 = run(True, cpu_ms=1e6)             # the host looks hopeless: never-lose keeps everything on the copy engine
    assert st2.summary()["cpu_experts"] == 0 and slow_t == ref_t and torch.equal(slow_l, ref_l)
