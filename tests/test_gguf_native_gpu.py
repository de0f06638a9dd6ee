"""GGUF block types the GPU kernels read without re-quantisation (Q5_K, Q6_K, Q8_0 beside Q4_K): dense layers, expert slots with
a different type for the down matrix, and the many-row path.  The CPU block codec is the oracle of the GPU decoders."""
import dataclasses

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from layerstorm_b200.formats import gguf as g  # noqa: E402


def _need_gpu():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")


@pytest.mark.parametrize("fmt", ["gguf_q5_k", "gguf_q6_k", "gguf_q8_0", "gguf_q4_k"])
@pytest.mark.parametrize("M", [1, 3, 4, 40])
def test_dense_layer_over_gguf_blocks(fmt, M):
    """1-4 rows stream the blocks through the GEMV decoders; 40 rows expand them to bf16 and run the tensor-core GEMM."""
    _need_gpu()
    from layerstorm_b200.models.device_model import QLinear
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev).manual_seed(4)
    N, K = 192 if M < 16 else 256, 1024
    W = QLinear.random(N, K, fmt, dev, gen=gen)
    Wf = W.dequant()
    assert Wf.shape == (N, K) and torch.isfinite(Wf).all() and Wf.abs().max() > 0
    x = torch.randn(M, K, device=dev, generator=gen).to(torch.bfloat16)
    out = torch.zeros(M, N, device=dev)
    W(out, x, M)
    torch.cuda.synchronize()
    ref = x.float() @ Wf.t()
    tol = (2e-3 if M < 16 or fmt == "gguf_q4_k" else 8e-3) * ref.abs().max().item()      # many rows: weights rounded to bf16
    assert (out - ref).abs().max().item() < tol, ((out - ref).abs().max().item(), tol)


class _NativeWeights(dict):
    """A float state dict whose expert matrices are also available as GGUF blocks (what a GGUF checkpoint offers): gate / up as
    ``gu_type``, down as ``dn_type``; the float view is the de-quantised blocks."""

    def __init__(self, w, gu_type, dn_type):
        super().__init__(w)
        self.blocks = {}
        for k in list(self):
            if ".moe.experts." in k or ".moe.shared." in k:
                t = dn_type if k.endswith(".down") else gu_type
                x = self[k].float().numpy()
                raw = g.quantize(t, x)
                self.blocks[k] = (t, raw, x.shape[0], x.shape[1])
                self[k] = torch.from_numpy(g.dequantize(t, raw, x.size)).view(x.shape)

    def native_ggml(self, key):
        return self.blocks.get(key)


@pytest.mark.parametrize("gu,dn", [("Q4_K", "Q6_K"), ("Q6_K", "Q6_K"), ("Q8_0", "Q4_K")])
def test_experts_in_the_files_own_block_types(gu, dn):
    """expert_quant='gguf': every MoE layer takes its experts as the checkpoint's blocks (down in another type than gate / up) and
    the engine matches the fp32 oracle over the de-quantised blocks, through the weight-streaming kernels at every chunk size."""
    _need_gpu()
    from layerstorm_b200.models.config import get_preset
    from layerstorm_b200.models.device_model import EXPERT_FMT, DeviceModel
    from layerstorm_b200.models.reference import Oracle
    from layerstorm_b200.models.weights import init_weights
    from layerstorm_b200.runtime.engine import Engine
    cfg = dataclasses.replace(get_preset("tiny-mla-moe"), moe_inter=256, name="tiny-gguf-mixed")
    w = _NativeWeights(init_weights(cfg, 3), g.GGML_TYPES[gu], g.GGML_TYPES[dn])
    m = DeviceModel.from_state_dict(cfg, w, "cuda", kv_fmt="bf16", page=16, expert_quant="gguf")
    ef = m.layers[1]["arena"].ef
    assert ef.fmt == EXPERT_FMT["gguf_" + gu.lower()]
    assert ef.fmt_down1 == (0 if gu == dn else EXPERT_FMT["gguf_" + dn.lower()] + 1)
    eff = m.effective_state_dict()
    k = "layers.1.moe.experts.2.down"
    assert torch.equal(eff[k], w[k].float())                                   # the blocks arrived bit-exactly
    oracle = Oracle(cfg, eff)
    ids = torch.randint(0, cfg.vocab, (26,), generator=torch.Generator().manual_seed(2))
    ref_logits = oracle.forward(ids)
    for chunk in (8, 32):
        eng = Engine(m, max_seqs=1, max_ctx=128, prefill_chunk=chunk, max_batch=1, use_graph=False)
        sid = eng.create_sequence()
        _, lg = eng.prefill(sid, ids[:24].tolist(), want_logits=True)
        e = float((lg - ref_logits[23]).abs().max() / ref_logits[23].abs().max())
        assert e < 3e-2, (chunk, e)
        out, lg = eng.decode([sid], [int(ids[24])], return_logits=True)
        assert out[0] == int(ref_logits[24].argmax())
        eng.free_sequence(sid)


@pytest.mark.parametrize("gu,dn", [("Q4_K", "Q6_K"), ("Q8_0", "Q4_K")])
def test_live_gguf_source_fills_the_host_store_byte_identically(gu, dn):
    """Capped expert cache over a GGUF checkpoint: the slot images the live source builds from the file's blocks (straight into the
    pinned store, no device arena) are byte-identical to the ones the device path assembles and moves out, and the engine decodes
    the same tokens either way."""
    _need_gpu()
    from layerstorm_b200.models.config import get_preset
    from layerstorm_b200.models.device_model import DeviceModel
    from layerstorm_b200.models.weights import init_weights
    from layerstorm_b200.runtime.engine import Engine
    from layerstorm_b200.runtime.live_gguf import LiveGgufExpertSource
    from layerstorm_b200.runtime.streaming import ExpertStreamer
    cfg = dataclasses.replace(get_preset("tiny-mla-moe"), moe_inter=256, name="tiny-gguf-live")
    w = _NativeWeights(init_weights(cfg, 3), g.GGML_TYPES[gu], g.GGML_TYPES[dn])
    slots = cfg.top_k + cfg.n_shared + 2
    prompt = torch.randint(0, cfg.vocab, (40,), generator=torch.Generator().manual_seed(2)).tolist()

    def tokens(m):
        eng = Engine(m, max_seqs=1, max_ctx=128, prefill_chunk=8, max_batch=1, use_graph=False)
        sid = eng.create_sequence()
        out = [eng.prefill(sid, prompt)]
        for _ in range(5):
            out.append(eng.decode([sid], [out[-1]])[0])
        return out

    ma = DeviceModel.from_state_dict(cfg, w, "cuda", kv_fmt="bf16", page=16, expert_quant="gguf")
    sa = ExpertStreamer(ma, slots_per_layer=slots)
    src = LiveGgufExpertSource(w, cfg, threads=4)
    sb = ExpertStreamer(None, slots_per_layer=slots, cfg=cfg, device="cuda", live_source=src)
    assert all(sb.covers(i) == cfg.is_moe_layer(i) for i in range(cfg.n_layers))
    mb = DeviceModel.from_state_dict(cfg, w, "cuda", kv_fmt="bf16", page=16, expert_quant="gguf", layer_hook=sb.add_layer, skip_experts=sb.covers)
    sb.attach(mb)
    assert set(sa.layers) == set(sb.layers) and src.bytes_built > 0
    for i in sa.layers:
        la, lb = sa.layers[i], sb.layers[i]
        assert la["arena"].ef.stride == lb["arena"].ef.stride and la["arena"].ef.fmt == lb["arena"].ef.fmt and la["arena"].ef.fmt_down1 == lb["arena"].ef.fmt_down1
        for e in la["host_row"]:
            assert torch.equal(la["host"][la["host_row"][e]], lb["host"][lb["host_row"][e]]), (i, e)
    assert tokens(ma) == tokens(mb)
    # a layer with a tensor the kernels do not read natively is not covered: the builder assembles it the ordinary way
    w2 = _NativeWeights(init_weights(cfg, 3), g.GGML_TYPES[gu], g.GGML_TYPES[dn])
    w2.blocks.pop("layers.1.moe.experts.3.up")
    assert LiveGgufExpertSource(w2, cfg).layout(1) is None and LiveGgufExpertSource(w2, cfg).layout(2) is not None
