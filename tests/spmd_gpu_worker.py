"""Multi-GPU worker: rank 0 drives the tensor-parallel engine through SpmdLeader (as the server does), the other ranks replay the
call stream; the greedy tokens must equal the fp32 oracle's."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from layerstorm_b200.models.config import get_preset
from layerstorm_b200.models.device_model import DeviceModel
from layerstorm_b200.models.reference import Oracle
from layerstorm_b200.models.weights import init_weights, round_weights_bf16
from layerstorm_b200.parallel.symm import PeerComm
from layerstorm_b200.runtime.engine import Engine
from layerstorm_b200.runtime.spmd import SpmdLeader, control_group, follower_loop


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    grp = control_group()
    cfg = get_preset("tiny-mla-moe")
    w = round_weights_bf16(init_weights(cfg, 0))
    m = DeviceModel.from_state_dict(cfg, w, dev, kv_fmt="bf16", page=16, tp_rank=rank, tp_size=world)
    comm, comm_amax = PeerComm(16 * cfg.hidden, dev), PeerComm(64, dev)
    m.attach_comm(comm, comm_amax)
    eng = Engine(m, max_seqs=3, max_ctx=128, prefill_chunk=8, max_batch=2, use_graph=True)
    ok = True
    if rank == 0:
        lead = SpmdLeader(eng, grp)
        ids = torch.randint(0, cfg.vocab, (26,), generator=torch.Generator().manual_seed(9))
        ref = Oracle(cfg, w).forward(ids)
        sid = lead.create_sequence()
        ok = lead.prefill(sid, ids[:20].tolist()) == int(ref[19].argmax())
        for j in range(3):
            ok = ok and lead.decode([sid], [int(ids[20 + j])])[0] == int(ref[20 + j].argmax())
        child = lead.fork_sequence(sid)                            # prefix-cache style fork, then both advance together
        out = lead.decode([sid, child], [int(ids[23]), int(ids[23])])
        ok = ok and out[0] == out[1] == int(ref[23].argmax())
        lead.free_sequence(child)
        lead.shutdown()
        print(f"leader tokens_match={ok} calls={lead.calls_announced}", flush=True)
    else:
        follower_loop(eng, grp)
    err = comm.error() or comm_amax.error()
    flag = torch.tensor([1 if (ok and err == 0) else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("SPMD_GPU_OK" if int(flag[0]) == 1 else "SPMD_GPU_FAIL", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if int(flag[0]) == 1 else 1)


if __name__ == "__main__":
    main()
