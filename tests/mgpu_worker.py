"""Multi-GPU worker (one process per GPU, launched by torch.distributed.run): tensor/expert-parallel
engine with the in-kernel NVLink all-reduce vs the single-process fp32 oracle."""
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


def main():
    name = sys.argv[1] if len(sys.argv) > 1 else "tiny-glm5-next"
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    cfg = get_preset(name)
    w = round_weights_bf16(init_weights(cfg, 0))
    m = DeviceModel.from_state_dict(cfg, w, dev, kv_fmt="bf16", page=16, tp_rank=rank, tp_size=world)
    comm = PeerComm(64 * cfg.hidden, dev)       # 64 rows: 8-row prefill chunks (fused GEMM epilogue) and one 64-row chunk (many-row kernels)
    comm_amax = PeerComm(64, dev)
    m.attach_comm(comm, comm_amax)
    oracle = Oracle(cfg, w)
    T = 24
    ids = torch.randint(0, cfg.vocab, (T + 6,), generator=torch.Generator().manual_seed(5))
    ref = oracle.forward(ids)
    ok = True
    for use_graph in (False, True):
        eng = Engine(m, max_seqs=2, max_ctx=128, prefill_chunk=8, max_batch=2, use_graph=use_graph)
        sid = eng.create_sequence()
        nxt = eng.prefill(sid, ids[:T].tolist())                 # chunks of 8 rows: tcgen05 GEMM with the fused all-reduce epilogue
        good = nxt == int(ref[T - 1].argmax())
        for j in range(6):                                       # single rows: fused in-kernel all-reduce
            out = eng.decode([sid], [int(ids[T + j])])
            good = good and out[0] == int(ref[T + j].argmax())
        err = comm.error() or comm_amax.error()
        if rank == 0:
            print(f"graph={use_graph} tokens_match={good} comm_err={err} backend={comm.buf.backend} epochs={comm.epoch()}", flush=True)
        ok = ok and good and err == 0
        eng.free_sequence(sid)
    # three sequences decoded together: 3 rows have no fused GEMV epilogue, the partials go through the push kernel
    seqs = [torch.randint(0, cfg.vocab, (12 + 5,), generator=torch.Generator().manual_seed(40 + b)) for b in range(3)]
    refs = [oracle.forward(s_) for s_ in seqs]
    eng = Engine(m, max_seqs=3, max_ctx=128, prefill_chunk=8, max_batch=3, use_graph=True)
    sids = [eng.create_sequence() for _ in range(3)]
    good = True
    for sid, s_, r_ in zip(sids, seqs, refs):
        good = good and eng.prefill(sid, s_[:12].tolist()) == int(r_[11].argmax())
    for j in range(5):
        out = eng.decode(sids, [int(s_[12 + j]) for s_ in seqs])
        good = good and all(o == int(r_[12 + j].argmax()) for o, r_ in zip(out, refs))
    err = comm.error() or comm_amax.error()
    if rank == 0:
        print(f"batch3 tokens_match={good} comm_err={err}", flush=True)
    ok = ok and good and err == 0
    # one 64-row prefill chunk: the many-row kernels (wide mHC partials, tensor-core attention) consume the cross-rank sums
    long_ids = torch.randint(0, cfg.vocab, (80,), generator=torch.Generator().manual_seed(77))
    long_ref = oracle.forward(long_ids)
    eng = Engine(m, max_seqs=1, max_ctx=128, prefill_chunk=64, max_batch=1, use_graph=False)
    sid = eng.create_sequence()
    good = eng.prefill(sid, long_ids.tolist()) == int(long_ref[79].argmax())
    err = comm.error() or comm_amax.error()
    if rank == 0:
        print(f"chunk64 tokens_match={good} comm_err={err}", flush=True)
    ok = ok and good and err == 0
    # sharded KV (context parallel): every rank stores only its token positions; same greedy tokens as the oracle
    if True:
        from layerstorm_b200.parallel.dcp import DcpAttention, local_length
        dcp = DcpAttention(cfg.n_heads, cfg.kv_lora, cfg.qk_rope, max_rows=8, device=dev, chunk=4, n_splits=2)
        m.enable_dcp(dcp)
        good = True
        for use_graph in (False, True):
            eng = Engine(m, max_seqs=2, max_ctx=128, prefill_chunk=8, max_batch=2, use_graph=use_graph)
            sid = eng.create_sequence()
            good = good and eng.prefill(sid, ids[:T].tolist()) == int(ref[T - 1].argmax())
            for j in range(6):
                good = good and eng.decode([sid], [int(ids[T + j])])[0] == int(ref[T + j].argmax())
            pages = len(eng.seqs[sid].pages)
            good = good and pages == (local_length(T + 6, 4, world, 0) + 15) // 16          # pages for the largest (rank 0's) share on every rank
            eng.free_sequence(sid)
        err = comm.error() or comm_amax.error() or dcp.error()
        if rank == 0:
            print(f"sharded_kv tokens_match={good} err={err} local_pages={pages}", flush=True)
        ok = ok and good and err == 0
        m.dcp = None
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("MGPU_OK" if int(flag[0]) == 1 else "MGPU_FAIL", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if int(flag[0]) == 1 else 1)


if __name__ == "__main__":
    main()
