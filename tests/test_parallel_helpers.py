"""CPU checks of host-side helpers of the parallel components (no GPU, no process group)."""
import torch

from layerstorm_b200.models import reference as ref
from layerstorm_b200.models.config import ModelConfig
from layerstorm_b200.parallel.dcp import local_index, local_length, owner_of


def test_dcp_sharding_is_a_partition_and_compact():
    for world in (1, 2, 4, 8):
        for chunk in (1, 16, 64):
            for length in (0, 1, chunk - 1, chunk, chunk + 1, 3 * chunk * world + 5, 1000):
                seen = []
                for r in range(world):
                    own = [t for t in range(max(length, 0)) if owner_of(t, chunk, world) == r]
                    assert len(own) == local_length(max(length, 0), chunk, world, r)
                    assert [local_index(t, chunk, world) for t in own] == list(range(len(own)))     # order preserving, dense
                    seen += own
                assert sorted(seen) == list(range(max(length, 0)))


def test_hash_routing_reference():
    cfg = ModelConfig(n_routed=8, top_k=2, scoring="softmax", routed_scale=2.0)
    logits = torch.tensor([[0.0, 1.0, 2.0, 3.0, 0.0, 0.0, 0.0, 0.0]] * 3)
    table = torch.tensor([[3, 2], [1, 9], [0, 7]], dtype=torch.int32)
    ids, w = ref.route_hash(cfg, logits, table, torch.tensor([0, 1, 5]))
    assert ids.tolist() == [[3, 2], [1, -1], [-1, -1]]
    p = torch.softmax(logits[0], -1)
    assert torch.allclose(w[0], 2.0 * torch.stack([p[3], p[2]]) / (p[3] + p[2]), atol=1e-6)
    assert float(w[1, 1]) == 0.0 and torch.allclose(w[1, 0], torch.tensor(2.0)) and w[2].abs().sum() == 0
