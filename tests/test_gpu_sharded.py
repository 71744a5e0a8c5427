"""Column-sharded RWKV-4 on two GPUs (one process per GPU) against the single-GPU model: same
logits up to the fp32 summation order.  Two ways of exchanging the output slices: peer stores from
the matmul epilogue with arrival words (the default) and NCCL all-gather calls between launches."""
import copy
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, ret, mode):
    os.environ["RWKV_B200_SHARD_EXCHANGE"] = mode
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from chatrwkv_b200 import synth
        from chatrwkv_b200.model import RWKV
        ck = synth.make_checkpoint(4, n_layer=7, n_embd=256, n_ffn=1024, vocab=1000, seed=3)
        toks = synth.make_tokens(10, 1000, 4)
        m = RWKV(copy.deepcopy(ck), f"cuda:{rank} fp16i8", verbose=False, shard_rank=rank, shard_world=world)
        assert (m._peer is not None) == (mode == "peer")
        outs = []
        lg, st = m.forward(toks[:6], None)
        outs.append(lg.cpu())
        for t in toks[6:]:
            lg, st = m.forward([t], st)
            outs.append(lg.cpu())
        if rank == 0:
            ref = RWKV(copy.deepcopy(ck), "cuda:0 fp16i8", verbose=False)
            lg, st = ref.forward(toks[:6], None)
            worst = (lg.cpu() - outs[0]).abs().max().item()
            for i, t in enumerate(toks[6:]):
                lg, st = ref.forward([t], st)
                worst = max(worst, (lg.cpu() - outs[i + 1]).abs().max().item())
            ret["worst"] = worst
        ret[f"peer_error{rank}"] = m.peer_error()
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["peer", "nccl"])
def test_two_gpu_column_sharded_matches_single_gpu(mode):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    port = 29600 + (os.getpid() % 2000) + (7 if mode == "nccl" else 0)
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(2, port, ret, mode), nprocs=2, join=True)
        assert ret["worst"] < 4e-3, ret["worst"]
        assert ret["peer_error0"] == 0 and ret["peer_error1"] == 0
