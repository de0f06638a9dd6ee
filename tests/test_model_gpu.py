"""End-to-end engine vs the fp32 CPU oracle on shrunken versions of every architecture:
chunked prefill == teacher-forced decode == oracle (tolerance), greedy token identity."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from layerstorm_b200.models.config import get_preset
from layerstorm_b200.models.device_model import DeviceModel
from layerstorm_b200.models.reference import Oracle
from layerstorm_b200.models.weights import init_weights
from layerstorm_b200.runtime.engine import Engine


def build(name, eq="bf16", dq="bf16", kv="bf16", seed=0, **kw):
    cfg = get_preset(name)
    w = init_weights(cfg, seed)
    m = DeviceModel.from_state_dict(cfg, w, "cuda", kv_fmt=kv, page=16, expert_quant=eq, dense_quant=dq)
    oracle = Oracle(cfg, m.effective_state_dict())
    return cfg, m, oracle


def rel_err(a, b):
    return float((a - b).abs().max() / (b.abs().max() + 1e-9))


@pytest.mark.parametrize("name", ["tiny-mla-moe", "tiny-glm5-next", "tiny-deepseek-v32"])
def test_prefill_and_decode_match_oracle(name):
    cfg, m, oracle = build(name)
    eng = Engine(m, max_seqs=2, max_ctx=256, prefill_chunk=16, max_batch=2, use_graph=False)
    g = torch.Generator().manual_seed(5)
    T = 28          # below index_topk=32 -> dense selection on both sides
    ids = torch.randint(0, cfg.vocab, (T + 4,), generator=g)
    ref_logits = oracle.forward(ids)
    sid = eng.create_sequence()
    nxt, lg = eng.prefill(sid, ids[:T].tolist(), want_logits=True)
    assert rel_err(lg, ref_logits[T - 1]) < 3e-2, rel_err(lg, ref_logits[T - 1])
    assert nxt == int(ref_logits[T - 1].argmax())
    for j in range(4):
        out, lg = eng.decode([sid], [int(ids[T + j])], return_logits=True)
        e = rel_err(lg[0], ref_logits[T + j])
        assert e < 3e-2, (j, e)
        assert out[0] == int(ref_logits[T + j].argmax())


@pytest.mark.parametrize("name", ["tiny-glm5-next", "tiny-deepseek-v32"])
def test_sparse_selection_path(name):
    """Context beyond index_topk: the engine's own selection is fed to the oracle, so the test
    checks the sparse attention itself; the selection must be valid and mostly agree with the
    oracle's unquantised indexer."""
    cfg, m, oracle = build(name)
    eng = Engine(m, max_seqs=1, max_ctx=256, prefill_chunk=32, max_batch=1, use_graph=False)
    g = torch.Generator().manual_seed(6)
    T = 102          # two tokens in the open pool when IndexPool is on
    ids = torch.randint(0, cfg.vocab, (T,), generator=g)
    sid = eng.create_sequence()
    eng.prefill(sid, ids[:T - 1].tolist())
    out, lg = eng.decode([sid], [int(ids[T - 1])], return_logits=True)
    ws = eng.ws_decode[1]
    cnt = int(ws.sel_cnt[0])
    sel = ws.sel_idx[0, :cnt].cpu().tolist()
    P = cfg.index_kpool
    assert cnt == (cfg.index_topk // P) * P + (T % P if P > 1 else 0)
    assert sel == sorted(set(sel)) and all(0 <= t < T for t in sel)
    if P > 1:
        assert sel[-1] == T - 1          # the open pool's tokens are always selected
    ref_logits = oracle.forward(ids)                      # oracle's own selection
    src_layers = [i for i in cfg.mla_layers() if cfg.index_source_layer(i) == i]
    last = src_layers[-1]
    osel = oracle.sel_log[last][T - 1]
    overlap = len(set(sel) & set(osel)) / len(osel)
    assert overlap > 0.8, overlap


@pytest.mark.parametrize("eq,dq,kv", [("nvfp4", "bf16", "fp8"), ("fp8_e4m3", "fp8_e4m3", "fp8")])
def test_quantised_formats_match_oracle(eq, dq, kv):
    cfg, m, oracle = build("tiny-mla-moe", eq=eq, dq=dq, kv=kv)
    eng = Engine(m, max_seqs=1, max_ctx=128, prefill_chunk=8, max_batch=1, use_graph=False)
    ids = torch.randint(0, cfg.vocab, (24,), generator=torch.Generator().manual_seed(2))
    ref_logits = oracle.forward(ids)
    sid = eng.create_sequence()
    _, lg = eng.prefill(sid, ids.tolist(), want_logits=True)
    # weights are compared dequantised, so the only extra error is the fp8 KV cache
    assert rel_err(lg, ref_logits[-1]) < 6e-2, rel_err(lg, ref_logits[-1])


def test_gguf_q4k_experts_decode_and_prefill_match_oracle():
    """Q4_K expert slots: weight-streaming kernels (short chunks / decode) and the tensor-core grouped path (long chunk)."""
    import dataclasses
    cfg = dataclasses.replace(get_preset("tiny-mla-moe"), moe_inter=256, name="tiny-q4k")
    w = init_weights(cfg, 3)
    m = DeviceModel.from_state_dict(cfg, w, "cuda", kv_fmt="bf16", page=16, expert_quant="gguf_q4_k")
    assert m.layers[1]["arena"].ef.fmt == 3
    oracle = Oracle(cfg, m.effective_state_dict())
    ids = torch.randint(0, cfg.vocab, (26,), generator=torch.Generator().manual_seed(2))
    ref_logits = oracle.forward(ids)
    for chunk in (8, 32):
        eng = Engine(m, max_seqs=1, max_ctx=128, prefill_chunk=chunk, max_batch=1, use_graph=False)
        sid = eng.create_sequence()
        _, lg = eng.prefill(sid, ids[:24].tolist(), want_logits=True)
        assert rel_err(lg, ref_logits[23]) < 3e-2, (chunk, rel_err(lg, ref_logits[23]))
        out, lg = eng.decode([sid], [int(ids[24])], return_logits=True)
        assert rel_err(lg[0], ref_logits[24]) < 3e-2 and out[0] == int(ref_logits[24].argmax())
        eng.free_sequence(sid)


def test_graph_decode_equals_eager_and_batched():
    cfg, m, _ = build("tiny-glm5-next")
    prompt_a = torch.randint(0, cfg.vocab, (20,), generator=torch.Generator().manual_seed(3)).tolist()
    prompt_b = torch.randint(0, cfg.vocab, (13,), generator=torch.Generator().manual_seed(4)).tolist()
    eng = Engine(m, max_seqs=4, max_ctx=128, prefill_chunk=16, max_batch=2, use_graph=False)
    ref_a = eng.generate(prompt_a, 8)
    ref_b = eng.generate(prompt_b, 8)
    eng2 = Engine(m, max_seqs=4, max_ctx=128, prefill_chunk=16, max_batch=2, use_graph=True)
    assert eng2.generate(prompt_a, 8) == ref_a
    # two sequences decoded together must give what each gives alone
    sa, sb = eng2.create_sequence(), eng2.create_sequence()
    ta, tb = eng2.prefill(sa, prompt_a), eng2.prefill(sb, prompt_b)
    out_a, out_b = [ta], [tb]
    for _ in range(7):
        ta, tb = eng2.decode([sa, sb], [ta, tb])
        out_a.append(ta); out_b.append(tb)
    assert out_a == ref_a and out_b == ref_b


def test_chunking_invariance():
    cfg, m, _ = build("tiny-glm5-next")
    prompt = torch.randint(0, cfg.vocab, (37,), generator=torch.Generator().manual_seed(8)).tolist()
    outs = []
    for chunk in (37, 16, 5):
        eng = Engine(m, max_seqs=1, max_ctx=128, prefill_chunk=chunk, max_batch=1, use_graph=False)
        sid = eng.create_sequence()
        nxt, lg = eng.prefill(sid, prompt, want_logits=True)
        outs.append((nxt, lg))
    # token identity across execution shapes; logits agree to rounding (rows >= 8 run on the
    # tensor-core GEMM, smaller chunks on the GEMV, whose summation orders differ)
    assert outs[0][0] == outs[1][0] == outs[2][0]
    for o in outs[1:]:
        assert rel_err(o[1], outs[0][1]) < 2e-2


def test_run_to_run_determinism():
    cfg, m, _ = build("tiny-glm5-next", eq="nvfp4", kv="fp8")
    prompt = torch.randint(0, cfg.vocab, (41,), generator=torch.Generator().manual_seed(9)).tolist()
    res = []
    for _ in range(2):
        eng = Engine(m, max_seqs=1, max_ctx=128, prefill_chunk=16, max_batch=1, use_graph=False)
        sid = eng.create_sequence()
        res.append(eng.prefill(sid, prompt, want_logits=True))
    assert res[0][0] == res[1][0] and torch.equal(res[0][1], res[1][1])


def test_turboquant_kv_rows_match_reference_quantiser_and_oracle():
    """4-bit TurboQuant KV: the cached codes equal the PyTorch reference quantiser's, and the logits stay close to the fp32 oracle."""
    from layerstorm_b200.formats import turboquant as tq
    cfg, m, oracle = build("tiny-mla-moe", kv="tq4")
    assert m.kv_row_bytes == cfg.kv_lora // 2 + 16 + 2 * cfg.qk_rope
    eng = Engine(m, max_seqs=1, max_ctx=128, prefill_chunk=8, max_batch=1, use_graph=False)
    ids = torch.randint(0, cfg.vocab, (30,), generator=torch.Generator().manual_seed(8))
    ref_logits = oracle.forward(ids)
    sid = eng.create_sequence()
    _, lg = eng.prefill(sid, ids[:28].tolist(), want_logits=True)
    assert rel_err(lg, ref_logits[27]) < 0.25                      # 4-bit cache: coarse, but the same distribution
    out, lg2 = eng.decode([sid], [int(ids[28])], return_logits=True)
    assert rel_err(lg2[0], ref_logits[28]) < 0.25
    # codes in the cache reproduce: quantise(dequantise(row)) is a fixed point of the reference quantiser
    li = cfg.mla_layers()[0]
    dl = cfg.kv_lora
    page0 = m.kv_cache[li][int(m.block_table[eng.seqs[sid].slot, 0])].cpu()            # [page, row_bytes]
    codes_b = page0[:8, : dl // 2]
    codes = torch.stack([codes_b & 15, codes_b >> 4], -1).reshape(8, dl)
    scale = page0[:8, dl // 2: dl // 2 + 4].contiguous().view(torch.float32).reshape(8)
    levels, rot = tq.lloyd_max_gaussian(16), tq.rotation(dl, li)
    c_hat = tq.dequantise(codes, scale, rot, levels)
    codes2, scale2 = tq.quantise(c_hat, rot, levels)
    assert float((codes2 == codes).float().mean()) > 0.97          # re-quantising the reconstruction gives the same codes (up to bf16 rotation rounding)
    assert torch.all(scale > 0) and levels.numel() == 16 and torch.allclose(levels, -levels.flip(0), atol=1e-5)
    assert torch.allclose(rot @ rot.T, torch.eye(dl), atol=1e-4)


@pytest.mark.parametrize("name", ["tiny-glm5-next", "tiny-deepseek-v32"])
def test_hibernate_resume_is_bit_identical_and_frees_pages(name):
    """KV tiering at sequence granularity: pages move to pinned host memory and back; tokens and logits are unchanged and
    another sequence can use the freed HBM pages in between."""
    cfg, m, _ = build(name, kv="fp8")
    eng = Engine(m, max_seqs=3, max_ctx=128, prefill_chunk=16, max_batch=1, num_pages=12, use_graph=False)
    eng.enable_kv_tiering(cold_pages=16)
    g = torch.Generator().manual_seed(11)
    pa = torch.randint(0, cfg.vocab, (70,), generator=g).tolist()
    pb = torch.randint(0, cfg.vocab, (90,), generator=g).tolist()

    def run(hib):
        a = eng.create_sequence()
        ta = [eng.prefill(a, pa)]
        free0 = eng.free_page_count()
        if hib:
            assert eng.hibernate(a) == 5 and eng.free_page_count() == free0 + 5 and eng.hibernate(a) == 0
            b = eng.create_sequence()                      # needs 6 pages: only fits because a's pages were released
            eng.prefill(b, pb)
            eng.free_sequence(b)
        lgs = []
        for _ in range(4):                                 # the first decode resumes the sequence transparently
            out, lg = eng.decode([a], [ta[-1]], return_logits=True)
            ta.append(out[0]); lgs.append(lg[0].clone())
        eng.free_sequence(a)
        return ta, torch.stack(lgs)

    t0, l0 = run(False)
    t1, l1 = run(True)
    assert t0 == t1 and torch.equal(l0, l1)
    assert eng.d2h_bytes > 0 and not eng.hibernated


def test_kda_chunked_prefill_matches_token_recurrence(monkeypatch):
    """Single-sequence steps of >= 128 rows run kda_chunk_prep / kda_chunk_scan; shorter steps run the token-by-token kernel.
    Both must give the same next token, and logits as close to the fp32 oracle as the token recurrence gives - at the prompt's
    last position and, through the carried state, at the decode steps that follow."""
    from layerstorm_b200.models import device_model as dm
    monkeypatch.setattr(dm, "KDA_CHUNKED", True)
    cfg, m, oracle = build("tiny-glm5-next")
    prompt = torch.randint(0, cfg.vocab, (200,), generator=torch.Generator().manual_seed(11)).tolist()      # 3 full chunks + 8 tokens
    cont = [5, 9, 2]
    refs = [oracle.forward(torch.tensor(prompt + cont[:j]))[-1] for j in range(len(cont) + 1)]
    res = []
    for chunk in (200, 100):
        eng = Engine(m, max_seqs=1, max_ctx=256, prefill_chunk=chunk, max_batch=1, use_graph=False)
        assert (eng.ws_prefill is None)
        sid = eng.create_sequence()
        nxt, lg = eng.prefill(sid, prompt, want_logits=True)
        assert (eng.ws_prefill.kda_chunk_ws is not None) == (chunk >= 128)
        steps = [eng.decode([sid], [t], return_logits=True)[1][0].clone() for t in cont]
        res.append((nxt, [lg.clone()] + steps))
        eng.free_sequence(sid)
    assert res[0][0] == res[1][0] == int(refs[0].argmax())
    for j, ref in enumerate(refs):
        e_chunk, e_tok = rel_err(res[0][1][j], ref), rel_err(res[1][1][j], ref)
        print(f"position {j}: chunk-parallel {e_chunk:.4g}, token recurrence {e_tok:.4g} (relative to the oracle)")
        assert e_chunk < 3e-2 and e_chunk < 2.0 * e_tok + 5e-3, (j, e_chunk, e_tok)


def test_resume_that_runs_out_of_pages_keeps_the_sequence_hibernated():
    """A resume that cannot get its pages fails cleanly: the cold copy and the hibernated state stay, and after room has been
    made the same resume gives bit-identical logits (the sequence never decodes on fresh, uninitialised pages)."""
    from layerstorm_b200.runtime.engine import KvPoolExhausted
    cfg, m, _ = build("tiny-deepseek-v32", kv="fp8")
    eng = Engine(m, max_seqs=3, max_ctx=128, prefill_chunk=16, max_batch=1, num_pages=10, use_graph=False)
    eng.enable_kv_tiering(cold_pages=16)
    g = torch.Generator().manual_seed(3)
    pa = torch.randint(0, cfg.vocab, (70,), generator=g).tolist()
    pb = torch.randint(0, cfg.vocab, (100,), generator=g).tolist()
    a = eng.create_sequence()
    ta = eng.prefill(a, pa)
    ref_tok, ref_lg = eng.decode([a], [ta], return_logits=True)
    eng.free_sequence(a)
    a = eng.create_sequence()
    assert eng.prefill(a, pa) == ta
    eng.hibernate(a)
    b = eng.create_sequence()
    eng.prefill(b, pb)                                       # 7 of the 10 pages: a's 5 pages no longer fit
    with pytest.raises(KvPoolExhausted):
        eng.decode([a], [ta])                                # resumes first: no room
    assert a in eng.hibernated and eng.seqs[a].pages == []
    eng.free_sequence(b)
    tok, lg = eng.decode([a], [ta], return_logits=True)
    assert tok == ref_tok and torch.equal(lg, ref_lg)


def test_a_set_error_word_withholds_the_step_output():
    """The bounded device waits report through error words; the engine reads them back with every step's tokens and raises a
    typed error instead of returning a token computed from partial data.  The word is set by hand here (nothing is made to
    hang); it is sticky until cleared."""
    from layerstorm_b200.models.device_model import TcScratch
    from layerstorm_b200.runtime.engine import DeviceWaitError
    cfg, m, _ = build("tiny-mla-moe")
    eng = Engine(m, max_seqs=1, max_ctx=64, prefill_chunk=16, max_batch=1, use_graph=False)
    sid = eng.create_sequence()
    t = eng.prefill(sid, list(range(3, 20)))
    TcScratch.get(m.device).err.fill_(7)
    with pytest.raises(DeviceWaitError) as ei:
        eng.decode([sid], [t])
    assert ei.value.source == "tensor_core" and ei.value.code == 7
    with pytest.raises(DeviceWaitError):
        eng.decode([sid], [t])
    eng.clear_device_errors()
    assert isinstance(eng.decode([sid], [t])[0], int)


@pytest.mark.parametrize("kv", ["fp8", "bf16"])
def test_row_granular_kv_tiering_is_bit_identical_and_frees_pages(kv):
    """Row-granular KV tiering of an active sequence: pages behind the hot window move to pinned host memory and give their HBM
    pages back; the rows the indexer selects from them come back through the staged copy + scatter.  Tokens and logits of the
    decode steps equal the untiered engine's bit for bit."""
    cfg, m, _ = build("tiny-glm5-next", kv=kv)
    prompt = torch.randint(0, cfg.vocab, (150,), generator=torch.Generator().manual_seed(21)).tolist()

    def run(tiered):
        eng = Engine(m, max_seqs=1, max_ctx=256, prefill_chunk=32, max_batch=1, use_graph=False,
                     row_tiering={"hot_window_tokens": 48, "cold_pages": 16} if tiered else None)
        if not tiered:
            m.row_tier, m.idx_identity = None, False
        sid = eng.create_sequence()
        toks = [eng.prefill(sid, prompt)]
        lgs = []
        for _ in range(20):
            out, lg = eng.decode([sid], [toks[-1]], return_logits=True)
            toks.append(out[0]); lgs.append(lg[0].clone())
        free = eng.free_page_count()
        rt_ = eng.row_tier
        eng.free_sequence(sid)
        return toks, torch.stack(lgs), free, rt_

    t0, l0, free0, _ = run(False)
    t1, l1, free1, tier = run(True)
    assert t0 == t1 and torch.equal(l0, l1)
    st = tier.stats
    assert st["demoted_pages"] >= 6 and st["cold_rows_fetched"] > 0 and st["bytes_h2d"] > 0, st
    assert free1 >= free0 + st["demoted_pages"] - 1                 # the demoted pages went back to the pool


@pytest.mark.parametrize("name", ["tiny-mla-moe", "tiny-glm5-next"])
def test_hash_layers_match_oracle_in_prefill_and_graph_decode(name):
    """MoE layers below ``num_hash_layers`` take their experts from the token-id table (DeepSeek-V4 hash layers): the engine's
    chunked prefill, eager decode and graph decode agree with the fp32 oracle, which routes the same rows through the same table."""
    import dataclasses
    cfg = dataclasses.replace(get_preset(name), num_hash_layers=3)
    assert sum(cfg.is_hash_layer(i) for i in range(cfg.n_layers)) >= 2
    w = init_weights(cfg, 0)
    m = DeviceModel.from_state_dict(cfg, w, "cuda", kv_fmt="bf16", page=16, expert_quant="bf16", dense_quant="bf16")
    assert any("tid2eid" in L for L in m.layers)
    oracle = Oracle(cfg, m.effective_state_dict())
    g = torch.Generator().manual_seed(9)
    T = 28
    ids = torch.randint(0, cfg.vocab, (T + 4,), generator=g)
    ref = oracle.forward(ids)
    for use_graph in (False, True):
        eng = Engine(m, max_seqs=2, max_ctx=256, prefill_chunk=16, max_batch=2, use_graph=use_graph)
        sid = eng.create_sequence()
        nxt, lg = eng.prefill(sid, ids[:T].tolist(), want_logits=True)
        assert rel_err(lg, ref[T - 1]) < 3e-2, rel_err(lg, ref[T - 1])
        assert nxt == int(ref[T - 1].argmax())
        for j in range(4):
            out, lg = eng.decode([sid], [int(ids[T + j])], return_logits=True)
            assert rel_err(lg[0], ref[T + j]) < 3e-2, (use_graph, j)
            assert out[0] == int(ref[T + j].argmax())
    # the table decides: another table gives other logits for the same tokens
    hashed = next(L for L in m.layers if "tid2eid" in L)
    hashed["tid2eid"].copy_(hashed["tid2eid"].roll(1, 0))
    eng = Engine(m, max_seqs=1, max_ctx=256, prefill_chunk=16, max_batch=1, use_graph=False)
    sid = eng.create_sequence()
    _, lg2 = eng.prefill(sid, ids[:T].tolist(), want_logits=True)
    assert rel_err(lg2, ref[T - 1]) > 1e-3


@pytest.mark.parametrize("name", ["tiny-glm5-next", "tiny-deepseek-v32"])
def test_spill_of_a_hibernated_sequence_to_a_file_is_bit_identical(name, tmp_path):
    """Second tiering hop: a hibernated sequence's cold pages go to a file and its pinned host slots are free again; the next step
    reads the file back, resumes and continues with the same tokens and logits.  A damaged or missing file raises (the caller drops
    the sequence); freeing a spilled sequence removes its file."""
    import os
    cfg, m, _ = build(name, kv="fp8")
    eng = Engine(m, max_seqs=3, max_ctx=128, prefill_chunk=16, max_batch=1, num_pages=12, use_graph=False)
    eng.enable_kv_tiering(cold_pages=8)
    g = torch.Generator().manual_seed(11)
    pa = torch.randint(0, cfg.vocab, (70,), generator=g).tolist()

    def run(spill):
        a = eng.create_sequence()
        ta = [eng.prefill(a, pa)]
        if spill:
            eng.hibernate(a)
            free_cold = eng.tier.free_cold_slots()
            path = str(tmp_path / f"a-{spill}.kvspill")
            nbytes = eng.spill(a, path)
            assert nbytes == os.path.getsize(path) - 12 - int.from_bytes(open(path, "rb").read(12)[8:], "little")
            assert a in eng.spilled and a not in eng.hibernated and eng.tier.free_cold_slots() == free_cold + 5
            with pytest.raises(RuntimeError):
                eng.spill(a, path)                         # not hibernated any more
        lgs = []
        for _ in range(4):                                 # the first decode reads the file back and resumes the sequence
            out, lg = eng.decode([a], [ta[-1]], return_logits=True)
            ta.append(out[0]); lgs.append(lg[0].clone())
        assert not getattr(eng, "spilled", {}) and not eng.hibernated
        eng.free_sequence(a)
        return ta, torch.stack(lgs)

    t0, l0 = run(0)
    t1, l1 = run(1)
    assert t0 == t1 and torch.equal(l0, l1)
    # a truncated file is refused, the sequence stays spilled; freeing it removes the file
    b = eng.create_sequence()
    eng.prefill(b, pa)
    eng.hibernate(b)
    path = str(tmp_path / "b.kvspill")
    eng.spill(b, path)
    blob = open(path, "rb").read()
    open(path, "wb").write(blob[: len(blob) // 2])
    with pytest.raises(ValueError):
        eng.decode([b], [5])
    assert b in eng.spilled
    eng.free_sequence(b)
    assert not os.path.exists(path)
