"""The chunk-parallel KDA formulation equals the token-by-token recurrence (CPU, fp64 and fp32, strong decay, carried state)."""
import pytest
import torch

from layerstorm_b200.models.kda_chunked import kda_chunked, kda_sequential


def _inputs(T, H, Dk, Dv, dtype, seed, lower_bound=-5.0):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(T, H, Dk, generator=g, dtype=dtype)
    k = torch.randn(T, H, Dk, generator=g, dtype=dtype)
    q = q / q.norm(dim=-1, keepdim=True) * Dk ** -0.5
    k = k / k.norm(dim=-1, keepdim=True)
    v = torch.randn(T, H, Dv, generator=g, dtype=dtype)
    beta = torch.sigmoid(torch.randn(T, H, generator=g, dtype=dtype))
    decay = torch.exp(lower_bound * torch.sigmoid(torch.randn(T, H, Dk, generator=g, dtype=dtype) * 2.0))     # (e^-5, 1): the model's range
    return q, k, v, beta, decay


@pytest.mark.parametrize("blockwise", [False, True])
@pytest.mark.parametrize("T,chunk", [(50, 16), (130, 64), (64, 64)])
def test_chunked_equals_sequential_fp64(T, chunk, blockwise):
    q, k, v, beta, decay = _inputs(T, 2, 32, 24, torch.float64, 0)
    S0 = torch.randn(2, 24, 32, dtype=torch.float64, generator=torch.Generator().manual_seed(9))
    o_ref, S_ref = kda_sequential(q, k, v, beta, decay, S0)
    o, S = kda_chunked(q, k, v, beta, decay, S0, chunk=chunk, blockwise=blockwise, sub=16)
    assert (o - o_ref).abs().max() < 1e-10 and (S - S_ref).abs().max() < 1e-10


def test_strong_decay_stays_finite_in_fp32():
    # every channel at the lower bound: cumulative decay over a 64-token chunk is e^-320, far below fp32 range
    T, H, D = 128, 1, 32
    q, k, v, beta, _ = _inputs(T, H, D, D, torch.float32, 1)
    decay = torch.full((T, H, D), float(torch.exp(torch.tensor(-5.0))))
    o_ref, S_ref = kda_sequential(q, k, v, beta, decay)
    for bw in (False, True):
        o, S = kda_chunked(q, k, v, beta, decay, chunk=64, blockwise=bw)
        assert torch.isfinite(o).all() and torch.isfinite(S).all()
        assert (o - o_ref).abs().max() < 1e-5 and (S - S_ref).abs().max() < 1e-5


def test_fp32_and_bf16_operand_error_at_model_width():
    T, H, D = 256, 2, 128
    q, k, v, beta, decay = _inputs(T, H, D, D, torch.float32, 2)
    o_ref, S_ref = kda_sequential(*(t.double() for t in (q, k, v, beta, decay)))
    o32, S32 = kda_chunked(q, k, v, beta, decay, chunk=64, blockwise=True)
    scale = o_ref.abs().max()
    assert (o32.double() - o_ref).abs().max() < 1e-4 * scale and (S32.double() - S_ref).abs().max() < 1e-4 * S_ref.abs().max()
    # bf16 matrix-product operands with fp32 accumulation (what a tensor-core kernel does): error stays at the bf16 rounding level
    o16, S16 = kda_chunked(q, k, v, beta, decay, chunk=64, blockwise=True, operand_dtype=torch.bfloat16)
    rel = (o16.double() - o_ref).norm() / o_ref.norm()
    assert rel < 2e-2, rel
    seq_bf16_inputs = kda_sequential(*(t.bfloat16().double() for t in (q, k, v, beta, decay)))[0]
    assert (o16.double() - o_ref).norm() < 4 * (seq_bf16_inputs - o_ref).norm() + 1e-3 * o_ref.norm()


def test_oracle_with_chunked_kda_matches_the_sequential_oracle():
    from layerstorm_b200.models.config import get_preset
    from layerstorm_b200.models.reference import Oracle
    from layerstorm_b200.models.weights import init_weights
    cfg = get_preset("tiny-glm5-next")
    w = init_weights(cfg, 0)
    toks = torch.randint(0, cfg.vocab, (70,), generator=torch.Generator().manual_seed(4))
    a = Oracle(cfg, w).forward(toks)
    o = Oracle(cfg, w)
    o.kda_chunk = 32
    b = o.forward(toks)
    assert (a - b).abs().max() < 2e-4 * a.abs().max()
    assert torch.equal(a.argmax(-1), b.argmax(-1))


def test_two_phase_form_equals_the_recurrence():
    from layerstorm_b200.models.kda_chunked import kda_chunk_prepare, kda_chunk_scan
    q, k, v, beta, decay = _inputs(150, 3, 32, 40, torch.float64, 5)
    S0 = torch.randn(3, 40, 32, dtype=torch.float64, generator=torch.Generator().manual_seed(1))
    o_ref, S_ref = kda_sequential(q, k, v, beta, decay, S0)
    prep = kda_chunk_prepare(q, k, beta, decay, chunk=64)          # no state, no values: parallel over chunks and heads
    o, S = kda_chunk_scan(prep, v, S0)
    assert (o - o_ref).abs().max() < 1e-10 and (S - S_ref).abs().max() < 1e-10
    # value channels are independent in the scan: any slice of them gives that slice of the result
    o_s, S_s = kda_chunk_scan(prep, v[..., 8:24].contiguous(), S0[:, 8:24].contiguous())
    assert (o_s - o_ref[..., 8:24]).abs().max() < 1e-10 and (S_s - S_ref[:, 8:24]).abs().max() < 1e-10
