"""Two-GPU tests (skipped on a single GPU): the fused peer-memory optimizer step against its NCCL twin, and the P2P
all-gather. Ranks are child processes; NVLS is disabled for NCCL so that a failing rank cannot disturb its peer."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, fused):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from rl_b200.algorithms.loss.loss_functions import NLLLossFn
    from rl_b200.distributed.batched_data_dict import BatchedDataDict
    from rl_b200.models.config import ModelConfig
    from rl_b200.ops.lib import check_status
    from rl_b200.policy.worker import PolicyWorker

    mc = ModelConfig(model_type="llama", vocab_size=4096, hidden_size=512, intermediate_size=1408, num_hidden_layers=2,
                     num_attention_heads=4, num_key_value_heads=2, head_dim=128)
    results = {}
    for mode in ("fused", "nccl"):
        p = PolicyWorker(dict(precision="bfloat16", train_global_batch_size=8, train_micro_batch_size=4, max_total_sequence_length=128,
                              fused_optimizer=(mode == "fused"), max_grad_norm=0.5,
                              optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=1e-3, weight_decay=0.1))),
                         model_cfg=mc, device=f"cuda:{rank}", init_reference_model=False, seed=11)
        assert (p.fused_comm is not None) == (mode == "fused")
        g = torch.Generator().manual_seed(100 + rank)
        ids = torch.randint(1, 4096, (4, 64), generator=g)
        data = BatchedDataDict(input_ids=ids, input_lengths=torch.full((4,), 64), token_mask=torch.ones(4, 64), sample_mask=torch.ones(4))
        norms = []
        for _ in range(3):
            out = p.train(data, NLLLossFn(), gbs=8, mbs=4)
            norms.append(float(out["grad_norm"][0]))
        torch.cuda.synchronize()
        assert check_status() == 0
        results[mode] = (p.flat.flat.float().clone(), norms, p.optimizer.m.clone())
        # all ranks hold identical parameters after the step
        mine = p.flat.flat.float()
        other = mine.clone()
        dist.broadcast(other, src=0)
        assert torch.equal(mine, other)
    pf, nf, mf = results["fused"]
    pn, nn_, mn = results["nccl"]
    assert max(abs(a - b) / max(abs(b), 1e-6) for a, b in zip(nf, nn_)) < 2e-3, (nf, nn_)
    assert (pf - pn).abs().max().item() < 2e-2  # bf16 parameters after 3 steps
    assert (mf - mn).abs().max().item() / (mn.abs().max().item() + 1e-9) < 1e-2
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_optimizer_matches_nccl(native_lib):
    mp.spawn(_worker, args=(2, _free_port(), True), nprocs=2, join=True)
