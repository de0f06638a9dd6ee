"""tcgen05 / TMA GEMM against a PyTorch fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from layerstorm_b200.ops import _native as nat


def run(M, N, K, out_bf16=False, bias=False, splitk=True, ldx=None, seed=0):
    g = torch.Generator().manual_seed(seed)
    ldx = ldx or K
    x = (torch.randn(M, ldx, generator=g)).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).cuda()
    b = torch.randn(N, generator=g).cuda() if bias else None
    out = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16 if out_bf16 else torch.float32)
    part = torch.zeros(16 * M * N, device="cuda") if splitk else None
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    nat.call("lsb_gemm_bf16_tc", out, x, w, b, M, N, K, ldx, K, N, int(out_bf16), part, 16 * M * N if splitk else 0, err, None)
    torch.cuda.synchronize()
    assert int(err[0]) == 0, f"kernel reported wait timeout code {int(err[0])}"
    ref = x[:, :K].float() @ w.float().T
    if bias:
        ref = ref + b
    tol = 2e-2 if out_bf16 else 2e-3
    e = (out.float() - ref).abs().max() / ref.abs().max()
    assert float(e) < tol, (M, N, K, float(e))


def test_gemm_tc_smallest():
    run(16, 128, 64, splitk=False)


@pytest.mark.parametrize("M,N,K", [(16, 128, 256), (32, 256, 512), (64, 384, 1024), (128, 512, 512), (256, 256, 2048),
                                   (300, 200, 264), (17, 130, 72), (2048, 1024, 512)])
def test_gemm_tc_shapes(M, N, K):
    run(M, N, K, splitk=False)


def test_gemm_tc_splitk_bias_bf16():
    run(32, 256, 4096, splitk=True, bias=True)
    run(48, 512, 2048, splitk=True, out_bf16=True, bias=True)
    run(64, 128, 1024, ldx=1032, splitk=True)


@pytest.mark.parametrize("M,B,N,K", [(64, 4, 128, 64), (300, 8, 512, 256), (2048, 3, 256, 128)])
def test_gemm_tc_batched_strided(M, B, N, K):
    """Per-head products as one launch: x[m, b, :K] (heads interleaved in a row), w[b], out[m, b, :N]."""
    g = torch.Generator().manual_seed(3)
    pad = 64                                            # a rope tail sits between the heads' K columns
    x = torch.randn(M, B, K + pad, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(B, N, K, generator=g) * 0.05).to(torch.bfloat16).cuda()
    out = torch.zeros(M, B, N + 8, device="cuda", dtype=torch.bfloat16)
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    nat.call("lsb_gemm_bf16_tc_batched", out, x, w, M, N, K, B, B * (K + pad), K + pad, K, N * K, B * (N + 8), N + 8, 1, err)
    torch.cuda.synchronize()
    assert int(err[0]) == 0
    ref = torch.einsum("mbk,bnk->mbn", x[:, :, :K].float(), w.float())
    e = (out[:, :, :N].float() - ref).abs().max() / ref.abs().max()
    assert float(e) < 2e-2, float(e)
    assert float(out[:, :, N:].abs().max()) == 0.0      # nothing written past N


@pytest.mark.parametrize("fmt", ["fp8_e4m3", "nvfp4"])
@pytest.mark.parametrize("M,N,K", [(16, 128, 128), (100, 256, 512), (300, 384, 1024)])
def test_quantised_linear_tensor_core_path(fmt, M, N, K):
    """QLinear with many rows (de-quantisation fused into the tcgen05 pipeline) == the same weights through fp32 matmul
    == the row-streaming GEMV path."""
    from layerstorm_b200.models.device_model import QLinear
    g = torch.Generator().manual_seed(11)
    wf = torch.randn(N, K, generator=g) * 0.05
    lin = QLinear.from_float(wf.cuda(), fmt, "cuda")
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    ref = x.float() @ lin.dequant().float().T
    for dt, tol in ((torch.float32, 3e-3), (torch.bfloat16, 2e-2)):
        out = torch.zeros(M, N + 16, device="cuda", dtype=dt)
        lin(out, x, M, ldo=N + 16)
        torch.cuda.synchronize()
        e = (out[:, :N].float() - ref).abs().max() / ref.abs().max()
        assert float(e) < tol, (fmt, dt, float(e))
    few = torch.zeros(4, N, device="cuda")
    lin(few, x, 4)                                       # GEMV path on the first rows
    torch.cuda.synchronize()
    assert float((few - ref[:4]).abs().max() / ref.abs().max()) < 3e-3
