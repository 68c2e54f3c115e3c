"""Multi-GPU tests on 2 and 4 GPUs (each skipped where the box has fewer): the fused peer-memory optimizer step, the
tensor-parallel GEMM + collective kernels, the peer-memory logits gather, the refit re-shard kernel and the expert-parallel
dispatch, each against its NCCL twin. Ranks are child processes; NVLS is disabled for NCCL so that a failing rank cannot
disturb its peers."""

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
        p = PolicyWorker(dict(precision="bfloat16", train_global_batch_size=4 * world, train_micro_batch_size=4, max_total_sequence_length=128,
                              fused_optimizer=(mode == "fused"), max_grad_norm=0.5,
                              optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=1e-3, weight_decay=0.1))),
                         model_cfg=mc, device=f"cuda:{rank}", init_reference_model=False, seed=11)
        assert (p.fused_comm is not None) == (mode == "fused")
        g = torch.Generator().manual_seed(100 + rank)
        ids = torch.randint(1, 4096, (4, 64), generator=g)
        data = BatchedDataDict(input_ids=ids, input_lengths=torch.full((4,), 64), token_mask=torch.ones(4, 64), sample_mask=torch.ones(4))
        norms = []
        for _ in range(3):
            out = p.train(data, NLLLossFn(), gbs=4 * world, mbs=4)
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


def _need(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")


@pytest.mark.parametrize("world", [2, 4])
def test_fused_optimizer_matches_nccl(native_lib, world):
    _need(world)
    mp.spawn(_worker, args=(world, _free_port(), True), nprocs=world, join=True)


def _tp_kernel_worker(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from rl_b200.ops.lib import check_status
    from rl_b200.parallel.tensor import TPFusedComm, all_gather_rows

    dev = torch.device("cuda", rank)
    comm = TPFusedComm(None, wait_limit_s=5.0)
    g = torch.Generator(device=dev).manual_seed(7 + rank)

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, generator=g, device=dev) * scale).to(torch.bfloat16)

    # (rows per rank, N, K): tile-aligned, ragged rows (tiles straddle two ranks), small
    for it, (rows, N, K) in enumerate([(256, 512, 512), (200, 768, 320), (72, 256, 1024), (1024, 1536, 512), (200, 768, 320)]):
        x = rnd(rows, K)
        w = rnd(N, K, scale=0.05)
        bias = torch.randn(N, generator=g, device=dev)
        xf = all_gather_rows(x, None, world).float()
        # gather: Y = allgather(x) @ w^T + bias
        y = comm.gather_gemm(x, w, bias=bias)
        ref = xf @ w.float().t() + bias
        torch.cuda.synchronize()
        assert check_status() == 0
        assert (y.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-2, ("gather", it)
        assert torch.equal(comm.gathered(world * rows, K).float(), xf), ("staging holds the gathered rows", it)
        # gather with a [K, N] weight (the backward form)
        wt = w.t().contiguous()
        y2 = comm.gather_gemm(x, wt, b_mn=True)
        assert (y2.float() - (ref - bias)).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-2, ("gather b_mn", it)
        # scatter: out = reduce_scatter(a @ w2^T) + residual
        M = world * rows
        a = rnd(M, K)
        w2 = rnd(N, K, scale=0.05)
        res = rnd(rows, N)
        part = a.float() @ w2.float().t()
        tot = part.clone()
        dist.all_reduce(tot)
        out = comm.scatter_gemm(a, w2, residual=res)
        torch.cuda.synchronize()
        assert check_status() == 0
        ref_rs = tot[rank * rows : (rank + 1) * rows] + res.float()
        tol = 2e-2 * ref_rs.abs().max().item() + 2e-2
        assert (out.float() - ref_rs).abs().max().item() <= tol, ("scatter", it, (out.float() - ref_rs).abs().max().item())
        # all-reduce form on a decode-sized batch
        m = 48
        a3 = rnd(m, K)
        res3 = rnd(m, N)
        dist.broadcast(res3, src=0)
        tot3 = a3.float() @ w2.float().t()
        dist.all_reduce(tot3)
        out3 = comm.scatter_gemm(a3, w2, residual=res3, all_reduce=True)
        torch.cuda.synchronize()
        assert check_status() == 0
        assert (out3.float() - (tot3 + res3.float())).abs().max().item() <= 2e-2 * tot3.abs().max().item() + 2e-2, ("allreduce", it)
        # every rank holds bit-identical all-reduced rows (fixed summation order)
        other = out3.clone()
        dist.broadcast(other, src=0)
        assert torch.equal(out3, other)
    # column gather over peer memory (vocabulary-parallel logits), fp32 and bf16, repeated calls (device-resident epoch,
    # alternating staging halves) and a changing row count
    for it, (rows, n, dt) in enumerate([(48, 1024, torch.float32), (48, 1024, torch.float32), (64, 520, torch.bfloat16), (5, 1024, torch.float32)]):
        z = (torch.randn(rows, n, generator=g, device=dev) + rank).to(dt)
        full = comm.gather_cols(z)
        parts = [torch.empty_like(z) for _ in range(world)]
        dist.all_gather(parts, z)
        torch.cuda.synchronize()
        assert check_status() == 0
        assert torch.equal(full, torch.cat(parts, dim=1)), ("gather_cols", it)
    # one-shot all-reduce of decode-sized fp32 partial sums with residual add and fused RMSNorm; changing row counts
    for it, (rows, n, with_norm) in enumerate([(48, 1024, True), (7, 1024, True), (256, 5120, True), (64, 1024, False), (64, 1024, True)]):
        part = torch.randn(rows, n, generator=g, device=dev) + 0.1 * rank
        res = torch.randn(rows, n, generator=g, device=dev).to(torch.bfloat16)
        dist.broadcast(res, src=0)
        wn = (1.0 + 0.1 * torch.randn(n, generator=g, device=dev)).to(torch.bfloat16)
        dist.broadcast(wn, src=0)
        out, out2 = comm.allreduce_rows(part, res, wn if with_norm else None, 1e-6)
        parts = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(parts, part)
        torch.cuda.synchronize()
        assert check_status() == 0
        tot = res.float()
        acc = torch.zeros_like(part)
        for q in parts:                      # the kernel sums the ranks in this order, in fp32
            acc = acc + q
        want = (acc + tot).to(torch.bfloat16)
        assert torch.equal(out, want), ("allreduce_rows", it, (out.float() - want.float()).abs().max().item())
        if with_norm:
            wf = want.float()
            ref2 = (wf * torch.rsqrt(wf.pow(2).mean(-1, keepdim=True) + 1e-6) * wn.float())
            assert (out2.float() - ref2).abs().max().item() <= 2e-2 * ref2.abs().max().item(), ("allreduce_rows norm", it)
        else:
            assert out2 is None
    dist.barrier()
    comm.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_fused_tensor_parallel_gemms(native_lib, world):
    _need(world)
    mp.spawn(_tp_kernel_worker, args=(world, _free_port()), nprocs=world, join=True)


def _tp_decode_worker(rank, world, port):
    """Tensor-parallel generation: the weight-streaming decode step with one-shot peer all-reduces against the layer-by-layer
    step (tile GEMM + all-reduce kernel); both captured in CUDA graphs, greedy."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from rl_b200.distributed.batched_data_dict import BatchedDataDict
    from rl_b200.models.config import ModelConfig
    from rl_b200.ops.lib import check_status
    from rl_b200.policy.worker import PolicyWorker

    mc = ModelConfig(model_type="qwen3", vocab_size=4096, hidden_size=512, intermediate_size=1024, num_hidden_layers=3,
                     num_attention_heads=8, num_key_value_heads=4, head_dim=128, qk_norm=True, tie_word_embeddings=False)
    p = PolicyWorker(dict(precision="bfloat16", train_global_batch_size=4, train_micro_batch_size=2, max_total_sequence_length=256,
                          parallel=dict(tensor_parallel_size=world, sequence_parallel=True),
                          generation=dict(max_new_tokens=40, temperature=1.0, stop_token_ids=[], kv_cache_tokens=8192, block_size=16, max_running=16),
                          optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=1e-3))),
                     model_cfg=mc, device=f"cuda:{rank}", init_reference_model=False, init_optimizer=False, seed=3)
    ids = torch.randint(1, 4096, (6, 24), generator=torch.Generator().manual_seed(10))
    data = BatchedDataDict(input_ids=ids, input_lengths=torch.full((6,), 24))
    gen = p.build_generation()
    gen.prepare_for_generation()
    eng = gen.engine
    assert eng._can_fuse_decode_tp(8)
    fast = gen.generate(data, greedy=True)
    n_graphs = len(eng._graphs)
    os.environ["RLB_FUSED_DECODE_TP"] = "0"
    eng._graphs.clear()
    slow = gen.generate(data, greedy=True)
    os.environ["RLB_FUSED_DECODE_TP"] = "1"
    gen.finish_generation()
    torch.cuda.synchronize()
    assert check_status() == 0 and n_graphs >= 1
    a, b, la, lb = fast["output_ids"], slow["output_ids"], fast["logprobs"], slow["logprobs"]
    same, prefix = 0, []
    for x, y, u, v in zip(a, b, la, lb):
        neq = (x != y).nonzero()
        t = int(neq[0]) if neq.numel() else x.numel()
        same += int(t == x.numel())
        prefix.append((t - 24) / (x.numel() - 24))
        if t > 24:
            assert (u[24:t] - v[24:t]).abs().max().item() < 0.08, (rank, t)
    assert same * 2 >= 6 and sum(prefix) / 6 > 0.6, (rank, same, prefix)
    # every tensor-parallel rank produced the same tokens without exchanging them
    other = a.clone().cuda()
    dist.broadcast(other, src=0)
    assert torch.equal(other.cpu(), a)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_tensor_parallel_decode_with_one_shot_allreduce(native_lib, world):
    _need(world)
    mp.spawn(_tp_decode_worker, args=(world, _free_port()), nprocs=world, join=True)


def _tp_train_worker(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from rl_b200.algorithms.loss.loss_functions import NLLLossFn
    from rl_b200.distributed.batched_data_dict import BatchedDataDict
    from rl_b200.models.config import ModelConfig
    from rl_b200.ops.lib import check_status
    from rl_b200.policy.worker import PolicyWorker

    mc = ModelConfig(model_type="llama", vocab_size=4096, hidden_size=512, intermediate_size=1536, num_hidden_layers=2,
                     num_attention_heads=8, num_key_value_heads=4, head_dim=128)
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(1, 4096, (8, 96), generator=g)
    data = BatchedDataDict(input_ids=ids, input_lengths=torch.tensor([96, 80, 64, 96, 33, 70, 96, 51]), token_mask=torch.ones(8, 96),
                           sample_mask=torch.ones(8))
    res = {}
    for mode in ("fused", "nccl"):
        p = PolicyWorker(dict(precision="bfloat16", train_global_batch_size=8, train_micro_batch_size=4, max_total_sequence_length=128,
                              fused_tensor_parallel=(mode == "fused"), max_grad_norm=1.0, parallel=dict(tensor_parallel_size=world),
                              optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=1e-3, weight_decay=0.0)),
                              generation=dict(max_new_tokens=16, temperature=1.0, stop_token_ids=[], kv_cache_tokens=4096, block_size=16,
                                              max_running=16)),
                         model_cfg=mc, device=f"cuda:{rank}", init_reference_model=False, seed=3)
        if mode == "nccl":
            p.tp.comm = None
            p.pstate.tp_comm = None
        assert (p.tp.comm is not None) == (mode == "fused")
        lp0 = p.get_logprobs(data)["logprobs"]
        outs = [p.train(data, NLLLossFn(), gbs=8, mbs=4) for _ in range(2)]
        gen = p.build_generation()
        gen.prepare_for_generation()
        gout = gen.generate(BatchedDataDict(input_ids=ids[:, :24], input_lengths=torch.full((8,), 24)))
        gen.finish_generation()
        torch.cuda.synchronize()
        assert check_status() == 0
        res[mode] = (lp0, [float(o["loss"][0]) for o in outs], [float(o["grad_norm"][0]) for o in outs], gout["logprobs"])
        # trainer log-probabilities of the sampled tokens agree with the engine's
        tl = p.get_logprobs(BatchedDataDict(input_ids=gout["output_ids"], input_lengths=gout["unpadded_sequence_lengths"]))["logprobs"]
        pos = torch.arange(gout["output_ids"].shape[1])[None, :]
        mask = (pos >= 24) & (pos < gout["unpadded_sequence_lengths"][:, None])
        assert (tl - gout["logprobs"])[mask].abs().max().item() < 0.08, mode
    f, n = res["fused"], res["nccl"]
    assert (f[0] - n[0]).abs().max().item() < 0.05
    assert max(abs(a - b) / abs(b) for a, b in zip(f[1], n[1])) < 5e-3, (f[1], n[1])
    assert max(abs(a - b) / abs(b) for a, b in zip(f[2], n[2])) < 2e-2, (f[2], n[2])
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_tensor_parallel_worker_fused_vs_nccl(native_lib, world):
    _need(world)
    mp.spawn(_tp_train_worker, args=(world, _free_port()), nprocs=world, join=True)


def _refit_worker(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from rl_b200.models.config import ModelConfig
    from rl_b200.models.transformer import PackedBatch, build_model
    from rl_b200.parallel.tensor import TP
    from rl_b200.refit.synchronizer import WeightSynchronizer

    mc = ModelConfig(model_type="qwen3", vocab_size=4096, hidden_size=512, intermediate_size=1536, num_hidden_layers=2,
                     num_attention_heads=8, num_key_value_heads=4, head_dim=128, qk_norm=True, tie_word_embeddings=False)
    dev = f"cuda:{rank}"
    combos = ((2, 1), (1, 2)) if world == 2 else ((4, 1), (1, 4), (2, 4), (4, 2), (1, 2))
    for tp_train, tp_serve in combos:
        tp_group = None
        if 1 < tp_train < world:   # the trainer's tensor-parallel groups inside the job (collective: every rank makes every group)
            for g0 in range(0, world, tp_train):
                grp = dist.new_group(ranks=list(range(g0, g0 + tp_train)))
                if g0 <= rank < g0 + tp_train:
                    tp_group = grp
        tp = TP(tp_group, rank % tp_train, tp_train)
        train = build_model(mc, device=dev, dtype=torch.bfloat16, seed=21, tp=tp)
        ws = WeightSynchronizer(train, mc, tp_serve)
        for it in range(2):
            with torch.no_grad():
                for p in train.parameters():
                    p.mul_(1.0 + 0.25 * it)
            ws.sync_weights()
            got = ws.arena.clone()
            ws.arena.zero_()
            ws.twin_sync()
            torch.cuda.synchronize()
            assert torch.equal(got, ws.arena), (tp_train, tp_serve, it)
        # quantising refit: one kernel writes e4m3 + de-scales (over NVLink for remote pieces); the result must equal
        # quantising the re-sharded bf16 copy afterwards
        from rl_b200.ops import quant as Q

        ws.twin_sync()
        want = {n: Q.quantize_fp8_blockwise(p.data) for n, p in ws.serving_model.named_parameters()
                if p.dim() == 2 and n.rsplit(".", 1)[-1] in ("qkv_proj", "o_proj", "gate_up_proj", "down_proj")}
        ws.arena.zero_()
        ws.sync_weights_fp8()
        torch.cuda.synchronize()
        assert len(ws._fp8_fused) == len(want) > 0, (tp_train, tp_serve, len(ws._fp8_fused), len(want))
        for n, p in ws.serving_model.named_parameters():
            if n in want:
                kind, q, sc = p._rlb_q
                assert torch.equal(q.view(torch.uint8), want[n][0].view(torch.uint8)) and torch.equal(sc, want[n][1]), (tp_train, tp_serve, n)
                assert torch.equal(p._rlb_q_bf16, Q.dequantize_fp8_blockwise(q, sc)), n
        sent, recv = ws.plan.bytes_over_link(rank)
        if tp_train == 1:
            assert sent == 0       # data-parallel training: every serving shard is cut from the rank's own copy
        tot = torch.tensor([float(sent)], device=dev)
        dist.all_reduce(tot)
        assert (tot.item() > 0) == (tp_train > 1)
        if tp_serve == 1:  # the serving model is a complete model: it runs on its own
            ids = torch.randint(0, 4096, (2, 32), device=dev)
            b = PackedBatch.from_padded(ids, torch.tensor([32, 20], device=dev))
            b.input_ids = b.input_ids.to(torch.int32)
            z = ws.serving_model.logits(b)
            assert torch.isfinite(z).all()
        dist.barrier()
        ws.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_refit_reshard_kernel_matches_collective_twin(native_lib, world):
    _need(world)
    mp.spawn(_refit_worker, args=(world, _free_port()), nprocs=world, join=True)


def _ep_worker(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from rl_b200.algorithms.loss.loss_functions import NLLLossFn
    from rl_b200.distributed.batched_data_dict import BatchedDataDict
    from rl_b200.models.config import ModelConfig
    from rl_b200.ops.lib import check_status
    from rl_b200.policy.worker import PolicyWorker

    mc = ModelConfig(model_type="qwen3_moe", vocab_size=4096, hidden_size=512, intermediate_size=0, num_hidden_layers=2,
                     num_attention_heads=4, num_key_value_heads=2, head_dim=128, qk_norm=True, num_experts=8, num_experts_per_tok=2,
                     moe_intermediate_size=256, norm_topk_prob=True)
    g = torch.Generator().manual_seed(50 + rank)
    ids = torch.randint(1, 4096, (4, 96), generator=g)
    data = BatchedDataDict(input_ids=ids, input_lengths=torch.tensor([96, 70, 64, 33]), token_mask=torch.ones(4, 96), sample_mask=torch.ones(4))
    res = {}
    for mode in ("fused", "nccl"):
        p = PolicyWorker(dict(precision="bfloat16", train_global_batch_size=4 * world, train_micro_batch_size=2, max_total_sequence_length=128,
                              max_grad_norm=1.0, parallel=dict(expert_parallel_size=world), logprob_batch_size=4,
                              optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=1e-3, weight_decay=0.0))),
                         model_cfg=mc, device=f"cuda:{rank}", init_reference_model=False, seed=3)
        if mode == "nccl":
            p.ep.comm = None
        assert (p.ep.comm is not None) == (mode == "fused")
        lp0 = p.get_logprobs(data)["logprobs"]
        outs = [p.train(data, NLLLossFn(), gbs=4 * world, mbs=2) for _ in range(2)]
        lp1 = p.get_logprobs(data)["logprobs"]
        torch.cuda.synchronize()
        assert check_status() == 0
        res[mode] = (lp0, [float(o["loss"][0]) for o in outs], [float(o["grad_norm"][0]) for o in outs], lp1)
    f, n = res["fused"], res["nccl"]
    # both paths run the same bf16 kernels on the same rows; what differs is the order of the rows inside an expert's tile
    # and hence nothing but rounding: a misrouted row would move the mean, not just the tail
    d0 = (f[0] - n[0]).abs()
    # (a router near-tie may flip for a single token when an expert's rows run through a differently shaped GEMM)
    assert d0.mean().item() < 5e-3 and d0.flatten().kthvalue(int(0.99 * d0.numel())).values.item() < 0.05, \
        (rank, d0.mean().item(), d0.max().item())
    assert max(abs(a - b) / abs(b) for a, b in zip(f[1], n[1])) < 5e-3, (f[1], n[1])
    assert max(abs(a - b) / abs(b) for a, b in zip(f[2], n[2])) < 3e-2, (f[2], n[2])
    assert (f[3] - n[3]).abs().mean().item() < 0.05
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_fused_dispatch_vs_nccl(native_lib, world):
    _need(world)
    mp.spawn(_ep_worker, args=(world, _free_port()), nprocs=world, join=True)


def _ep_gen_worker(rank, world, port):
    """Expert-parallel generation with uneven work per rank: the captured few-token MoE path (peer-memory gather and
    reduce, ranks in lock step) against the dispatch / combine path over NCCL, run eagerly."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from rl_b200.distributed.batched_data_dict import BatchedDataDict
    from rl_b200.models.config import ModelConfig
    from rl_b200.ops.lib import check_status
    from rl_b200.policy.worker import PolicyWorker

    mc = ModelConfig(model_type="qwen3_moe", vocab_size=4096, hidden_size=512, intermediate_size=0, num_hidden_layers=2,
                     num_attention_heads=4, num_key_value_heads=2, head_dim=128, qk_norm=True, num_experts=8, num_experts_per_tok=2,
                     moe_intermediate_size=256, norm_topk_prob=True)
    p = PolicyWorker(dict(precision="bfloat16", train_global_batch_size=4 * world, train_micro_batch_size=2, max_total_sequence_length=256,
                          parallel=dict(expert_parallel_size=world),
                          generation=dict(max_new_tokens=20 + 11 * rank, temperature=1.0, stop_token_ids=[], kv_cache_tokens=8192,
                                          block_size=16, max_running=16),
                          optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=1e-3))),
                     model_cfg=mc, device=f"cuda:{rank}", init_reference_model=False, init_optimizer=False, seed=3)
    with torch.no_grad():
        p.model.output_weight.mul_(6.0)      # a sharper head: fewer greedy near-ties between the two paths
    g = torch.Generator().manual_seed(10 + rank)
    n = 2 + 3 * rank
    ids = torch.randint(1, 4096, (n, 24), generator=g)
    data = BatchedDataDict(input_ids=ids, input_lengths=torch.full((n,), 24))
    gen = p.build_generation()
    gen.prepare_for_generation()
    fast = gen.generate(data, greedy=True)
    eng = gen.engine
    assert eng.use_graphs and len(eng._graphs) >= 1, "the expert-parallel decode step was not captured"
    comm, p.ep.comm = p.ep.comm, None          # NCCL all-to-all path: no peer kernels, no graphs
    eng.use_graphs = False
    slow = gen.generate(data, greedy=True)
    p.ep.comm = comm
    gen.finish_generation()
    torch.cuda.synchronize()
    assert check_status() == 0
    a, b = fast["output_ids"], slow["output_ids"]
    assert a.shape == b.shape
    # A random-initialised model has many greedy near-ties, and the two paths sum the experts' outputs in different orders
    # (fp32 partial sums over ranks against bf16 scatter-adds), so a sequence may part ways at some token. Up to that token
    # both paths must agree on tokens and log-probabilities; a misrouted expert would break the first token already.
    la, lb = fast["logprobs"], slow["logprobs"]
    same, prefix = 0, []
    for x, y, u, v in zip(a, b, la, lb):
        L = min(x.numel(), y.numel())
        neq = (x[:L] != y[:L]).nonzero()
        t = int(neq[0]) if neq.numel() else L
        same += int(t == L)
        prefix.append((t - 24) / max(1, L - 24))          # share of the generated tokens before the first difference
        if t > 24:   # (the head was sharpened six-fold above, and so are the rounding differences between the two paths)
            dlp = (u[24:t] - v[24:t]).abs()
            # the mean is the criterion: one near-tie token can move by a few tenths under the sharpened head while the
            # two paths still pick the same token
            assert dlp.mean().item() < 0.05 and dlp.median().item() < 0.03, (rank, t, dlp.max().item(), dlp.mean().item())
    assert same * 2 >= n and sum(prefix) / n >= 0.5, (rank, same, n, prefix)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_generation_graphs_vs_dispatch(native_lib, world):
    _need(world)
    mp.spawn(_ep_gen_worker, args=(world, _free_port()), nprocs=world, join=True)


def _split_job_worker(rank, world, port, steps):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      NCCL_NVLS_ENABLE="0")
    from rl_b200.algorithms import grpo, noncolocated as nc
    from rl_b200.data.datasets.synthetic import RandomTokenPromptDataset
    from rl_b200.distributed.roles import init_roles
    from rl_b200.environments.synthetic import HashParityEnv
    from rl_b200.models.config import ModelConfig
    from rl_b200.ops.lib import check_status

    g = world // 2
    cfg = {
        "grpo": dict(num_prompts_per_step=4 * (world - g), num_generations_per_prompt=2, max_num_steps=steps, seed=3, val_period=0,
                     async_grpo=dict(enabled=True, max_trajectory_age_steps=1, in_flight_weight_updates=True, generation_ranks=g)),
        "loss_fn": dict(reference_policy_kl_penalty=0.0, use_importance_sampling_correction=True),
        "policy": dict(model_name=None, precision="bfloat16", train_global_batch_size=8 * (world - g), train_micro_batch_size=4,
                       max_total_sequence_length=96, optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=1e-4, weight_decay=0.0)),
                       generation=dict(max_new_tokens=24, temperature=1.0, stop_token_ids=[], kv_cache_tokens=8192, block_size=16, max_running=16)),
        "checkpointing": dict(enabled=False), "logger": dict(log_dir=f"/tmp/rlb_split_logs_{os.getpid()}"), "data": dict(shuffle=False),
    }
    layout = init_roles(cfg)
    mc = ModelConfig(model_type="llama", vocab_size=4096, hidden_size=512, intermediate_size=1408, num_hidden_layers=2,
                     num_attention_heads=4, num_key_value_heads=2, head_dim=128)
    ds = RandomTokenPromptDataset(cfg["grpo"]["num_prompts_per_step"] * (steps + 2), 12, 24, mc.vocab_size, seed=1, task_name="synthetic")
    env = {"synthetic": HashParityEnv()}
    if layout.role == "generation":
        gen = nc.build_generation_rank(cfg, None, mc, layout.device)
        stats = nc.generation_service(layout, cfg, gen, ds, None, env)
        assert stats["shards"] >= 1 and stats["weight_updates"] >= 2 and stats["final_version"] == steps + 1, stats
    else:
        policy, _, _, _, loss_fn, logger, ck, save_state, cfg = grpo.setup(cfg, None, ds, None, env, model_cfg=mc, build_generation=False)
        seen = []
        nc.noncolocated_grpo_train(policy, layout, loss_fn, None, ck, save_state, cfg, None,
                                   step_callback=lambda s, m: seen.append((s, m["train"]["trajectory_age"], m["train"]["loss"])))
        assert [s for s, _, _ in seen] == list(range(1, steps + 1)) and all(0 <= a <= 1 for _, a, _ in seen), seen
    torch.cuda.synchronize()
    assert check_status() == 0
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_split_job_trains_while_generating_on_gpus(native_lib, world):
    """Asynchronous GRPO with half of the GPUs training and half generating (weights over a raw NCCL communicator,
    trajectories through the TCP store)."""
    _need(world)
    mp.spawn(_split_job_worker, args=(world, _free_port(), 3), nprocs=world, join=True)


def _fsdp_worker(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from rl_b200.algorithms.loss.loss_functions import NLLLossFn
    from rl_b200.distributed.batched_data_dict import BatchedDataDict
    from rl_b200.models.config import ModelConfig
    from rl_b200.ops.lib import check_status
    from rl_b200.policy.worker import PolicyWorker

    mc = ModelConfig(model_type="llama", vocab_size=4096, hidden_size=512, intermediate_size=1408, num_hidden_layers=3,
                     num_attention_heads=4, num_key_value_heads=2, head_dim=128)
    g = torch.Generator().manual_seed(100 + rank)
    ids = torch.randint(1, 4096, (4, 64), generator=g)
    data = BatchedDataDict(input_ids=ids, input_lengths=torch.tensor([64, 40, 64, 25]), token_mask=torch.ones(4, 64), sample_mask=torch.ones(4))
    res = {}
    for mode in ("full", "optimizer"):
        p = PolicyWorker(dict(precision="bfloat16", train_global_batch_size=4 * world, train_micro_batch_size=2, max_total_sequence_length=128,
                              max_grad_norm=0.5, parallel=dict(data_parallel_sharding=mode),
                              optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=1e-3, weight_decay=0.1)),
                              generation=dict(max_new_tokens=8, stop_token_ids=[], kv_cache_tokens=4096, block_size=16, max_running=8)),
                         model_cfg=mc, device=f"cuda:{rank}", init_reference_model=True, seed=11)
        lp0 = p.get_logprobs(data)["logprobs"]
        outs = [p.train(data, NLLLossFn(), gbs=4 * world, mbs=2) for _ in range(3)]
        lp1 = p.get_logprobs(data)["logprobs"]
        ref = p.get_reference_policy_logprobs(data)["reference_logprobs"]
        torch.cuda.synchronize()
        assert check_status() == 0
        if mode == "full":
            sh = p.sharder
            assert sh._peer is not None and sh.stats["prefetch_hits"] > 0      # peer pull kernel, next unit gathered ahead
            assert all(q.numel() == 0 for q in p.model.parameters())
            gen = p.build_generation()
            from rl_b200.algorithms.grpo import refit_policy_generation

            refit_policy_generation(p, gen)
            out = gen.generate(BatchedDataDict(input_ids=ids[:, :16], input_lengths=torch.full((4,), 16)))
            gen.finish_generation()
            assert (out["generation_lengths"] == 8).all()
        res[mode] = (lp0, [float(o["loss"][0]) for o in outs], [float(o["grad_norm"][0]) for o in outs], lp1, ref)
    f, n = res["full"], res["optimizer"]
    assert (f[0] - n[0]).abs().max().item() < 1e-3
    assert max(abs(a - b) / abs(b) for a, b in zip(f[1], n[1])) < 3e-3, (f[1], n[1])
    assert max(abs(a - b) / abs(b) for a, b in zip(f[2], n[2])) < 2e-2, (f[2], n[2])
    assert (f[3] - n[3]).abs().mean().item() < 0.03
    assert (f[4] - f[0]).abs().max().item() < 1e-3          # the reference shard did not move
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_fully_sharded_parameters_match_resident_mode(native_lib, world):
    """ZeRO-3 mode (parameters gathered per unit with the peer pull kernel, gradients reduce-scattered per unit) against
    the resident-parameter mode on the same data."""
    _need(world)
    mp.spawn(_fsdp_worker, args=(world, _free_port()), nprocs=world, join=True)
