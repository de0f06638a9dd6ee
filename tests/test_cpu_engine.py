"""The CPU plumbing configuration: tiny MLA-MoE, 64-token random prompt, 32 greedy tokens - on the fp32 reference and on the
native CPU expert kernels (same tokens), and through the orchestrator."""
import torch

from layerstorm_b200.models.config import get_preset
from layerstorm_b200.models.reference import Oracle
from layerstorm_b200.models.weights import init_weights
from layerstorm_b200.runtime.cpu_engine import CpuEngine, cpu_plumbing_run
from layerstorm_b200.serving.orchestrator import InferenceRequest, Orchestrator, SamplingParams


def test_cpu_plumbing_native_experts_match_reference():
    a, _, tps_a = cpu_plumbing_run(native_experts=False, prompt_len=24, new_tokens=8)
    b, _, tps_b = cpu_plumbing_run(native_experts=True, prompt_len=24, new_tokens=8)
    assert a == b and len(a) == 8 and tps_a > 0 and tps_b > 0
    cfg = get_preset("tiny-mla-moe")
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (24,), generator=g).tolist()
    assert Oracle(cfg, init_weights(cfg, 0)).greedy(prompt, 8) == a


def test_cpu_engine_quantised_experts_and_engine_api():
    cfg = get_preset("tiny-mla-moe")
    w = init_weights(cfg, 1)
    eng = CpuEngine(cfg, w, native_experts=True, expert_quant="nvfp4")
    ref = CpuEngine(cfg, w, native_experts=False)
    prompt = list(range(3, 19))
    s1, s2 = eng.create_sequence(), ref.create_sequence()
    n1, l1 = eng.prefill(s1, prompt, want_logits=True)
    n2, l2 = ref.prefill(s2, prompt, want_logits=True)
    assert float((l1 - l2).abs().max() / l2.abs().max()) < 0.15          # 4-bit experts vs fp32 experts
    rows = eng.forward_rows(s1, [5, 6, 7], commit=False)
    assert rows.shape == (3, cfg.vocab) and eng.seq_len(s1) == 16
    child = eng.fork_sequence(s1, 8)
    assert eng.seq_len(child) == 8
    eng.rewind(s1, 10)
    assert eng.seq_len(s1) == 10
    eng.free_sequence(child)


def test_orchestrator_on_cpu_engine():
    cfg = get_preset("tiny-mla-moe")
    eng = CpuEngine(cfg, init_weights(cfg, 2), native_experts=True)
    orch = Orchestrator(eng)
    req = InferenceRequest("r", list(range(10, 22)), SamplingParams(max_tokens=5, ignore_eos=True))
    orch.submit_request(req)
    orch.step()
    assert len(req.output_ids) == 5 and req.finish_reason == "length"
