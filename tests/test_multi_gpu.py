"""Tensor/expert-parallel engine on 2 GPUs: fused in-kernel all-reduce (decode) and the NCCL path
(prefill chunks) both reproduce the oracle's greedy tokens."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("name,shard", [("tiny-glm5-next", "ep"), ("tiny-mla-moe", "ep"), ("tiny-glm5-next", "tp"), ("tiny-mla-moe", "tp")])
def test_two_rank_engine_matches_oracle(name, shard):
    """``shard``: whole experts per GPU (expert parallel) or a slice of every expert on every GPU (tensor parallel experts)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", LSB_EXPERT_SHARD=shard)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29533", os.path.join(HERE, "mgpu_worker.py"), name]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert "MGPU_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.parametrize("fmt", ["fp8_e4m3", "nvfp4"])
def test_fused_expert_parallel_ffn(fmt):
    """Dispatch and combine as P2P stores inside the kernels == fp32 reference == NCCL all-to-all baseline."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    n = 4 if torch.cuda.device_count() >= 4 else 2
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29537", os.path.join(HERE, "ep_worker.py"), fmt]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert "EP_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_context_parallel_attention():
    """Token-sharded KV cache: all-gather of the queries, local split-KV attention and the cross-rank log-sum-exp merge, all by
    P2P stores from inside the kernels == fp32 attention over the whole cache."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    n = 4 if torch.cuda.device_count() >= 4 else 2
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29539", os.path.join(HERE, "dcp_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert "DCP_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_spmd_leader_and_followers_drive_the_parallel_engine():
    """Rank 0 issues the engine calls (as the server's orchestrator does), the other ranks replay the announced call stream."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29541", os.path.join(HERE, "spmd_gpu_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert "SPMD_GPU_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
