"""Model parallelism on CPU (gloo, 2 ranks): a tensor-parallel (+ sequence-parallel) model must reproduce the
single-rank model's log-probabilities, loss and gradients; expert-parallel MoE must match the local-expert loop."""

import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _spawn(fn, world, *args):
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    procs = [ctx.Process(target=_entry, args=(fn, r, world, port, q, args)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    out = {}
    while not q.empty():
        r, v = q.get()
        out[r] = v
    for p in procs:
        assert p.exitcode == 0, f"rank exited with {p.exitcode}: {out}"
    return out


def _entry(fn, rank, world, port, q, args):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.manual_seed(0)
    torch.set_num_threads(2)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q.put((rank, fn(rank, world, *args)))
    finally:
        dist.destroy_process_group()


def _full_model(seed=3, name="tiny-llama-oracle", **over):
    from rl_b200.models.config import preset
    from rl_b200.models.transformer import build_model

    cfg = preset(name, **over)
    return cfg, build_model(cfg, dtype=torch.float32, seed=seed)


def _batch(cfg, T_seqs=(9, 14, 5)):
    from rl_b200.models.transformer import PackedBatch

    g = torch.Generator().manual_seed(1)
    S = max(T_seqs)
    ids = torch.randint(0, cfg.vocab_size, (len(T_seqs), S), generator=g)
    return PackedBatch.from_padded(ids, torch.tensor(T_seqs))


def _tp_worker(rank, world, sp, tied, name="tiny-llama-oracle"):
    from rl_b200.models.hf_io import iter_hf_tensors, load_hf_tensors
    from rl_b200.models.transformer import build_model
    from rl_b200.parallel.state import init_parallel
    from rl_b200.parallel.tensor import TP

    st = init_parallel(tp=world, sequence_parallel=sp)
    cfg, full = _full_model(name=name, tie_word_embeddings=tied)
    sd = dict(iter_hf_tensors(full))
    tp = TP.from_state(st)
    model = build_model(cfg, dtype=torch.float32, seed=99, tp=tp)
    load_hf_tensors(model, sd.get)
    batch = _batch(cfg)
    pb = batch.pad_to_multiple(world) if sp else batch
    T = batch.input_ids.numel()
    ref_lp, ref_ent = full.next_token_logprobs(batch, 0.7, want_entropy=True)
    lp, ent = model.next_token_logprobs(pb, 0.7, want_entropy=True)
    w = torch.linspace(0.5, 1.5, T)
    (ref_lp * w).sum().backward()
    (lp[:T] * w).sum().backward()
    # gather the tp model's gradients back into HF tensors and compare with the full model
    if sp:  # partial gradients of replicated parameters
        for n, p in model.named_parameters():
            if not model.is_tp_sharded(n):
                dist.all_reduce(p.grad)
    full_g = {n: t for n, t in iter_hf_tensors(_GradView(full))}
    tp_g = {n: t for n, t in iter_hf_tensors(_GradView(model))}
    gerr = max(float((full_g[n] - tp_g[n]).abs().max()) for n in full_g)
    # round trip: gathered weights equal the originals
    werr = max(float((sd[n] - t).abs().max()) for n, t in iter_hf_tensors(model))
    return dict(lp=float((lp[:T] - ref_lp).abs().max()), ent=float((ent[:T] - ref_ent).abs().max()), grad=gerr, w=werr,
                logits=float((model.logits(pb)[:T] - full.logits(batch)).abs().max()) if not sp else 0.0)


class _GradView:
    """Presents a model's gradients under its parameter names so that the HF mapping can gather them."""

    def __init__(self, model):
        self.__dict__.update(cfg=model.cfg, tp=model.tp, ep=model.ep, layer_offset=model.layer_offset, layer_ids=model.layer_ids, layers=model.layers,
                             first_stage=model.first_stage, last_stage=model.last_stage)
        self._m = model

    def named_parameters(self):
        for n, p in self._m.named_parameters():
            yield n, (p.grad if p.grad is not None else torch.zeros_like(p))

    def named_buffers(self):
        for n, b in self._m.named_buffers():
            yield n, torch.zeros_like(b)


@pytest.mark.parametrize("sp,tied", [(True, False), (False, False), (True, True)])
def test_tensor_parallel_matches_single_rank(sp, tied):
    out = _spawn(_tp_worker, 2, sp, tied)
    for r, m in out.items():
        assert m["lp"] < 2e-4 and m["ent"] < 2e-4 and m["grad"] < 2e-3 and m["w"] == 0.0 and m["logits"] < 2e-4, (r, m)


def test_tensor_parallel_hybrid_model_matches_single_rank():
    """Nemotron-H under tensor parallelism: the plain MLP blocks and the output head are sharded, the Mamba, attention and
    expert blocks are replicated."""
    out = _spawn(_tp_worker, 2, False, False, "tiny-nemotron-h")
    for r, m in out.items():
        assert m["lp"] < 2e-4 and m["ent"] < 2e-4 and m["grad"] < 2e-3 and m["w"] == 0.0 and m["logits"] < 2e-4, (r, m)


def _ep_worker(rank, world):
    from rl_b200.models.config import preset
    from rl_b200.models.hf_io import iter_hf_tensors, load_hf_tensors
    from rl_b200.models.transformer import build_model
    from rl_b200.parallel.expert import EP
    from rl_b200.parallel.state import init_parallel

    st = init_parallel(ep=world)
    cfg = preset("tiny-llama-oracle", num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, norm_topk_prob=True)
    full = build_model(cfg, dtype=torch.float32, seed=5)
    sd = dict(iter_hf_tensors(full))
    model = build_model(cfg, dtype=torch.float32, seed=77, ep=EP.from_state(st))
    load_hf_tensors(model, sd.get)
    # every rank routes different tokens (data parallel over the expert group)
    batch = _batch(cfg, (7 + rank, 11, 4 + 2 * rank))
    ref, _ = full.next_token_logprobs(batch)
    got, _ = model.next_token_logprobs(batch)
    ref.sum().backward()
    got.sum().backward()
    gl = dict(model.named_parameters())["layers.0.mlp.gate_up_proj"].grad
    gf = dict(full.named_parameters())["layers.0.mlp.gate_up_proj"].grad
    # expert gradients: the ep model accumulates contributions from both ranks' tokens; compare after summing the
    # full model's gradients over the ranks
    dist.all_reduce(gf)
    per = cfg.num_experts // world
    return dict(lp=float((got - ref).abs().max()), g=float((gl - gf[rank * per : (rank + 1) * per]).abs().max()))


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_matches_local_experts(world):
    out = _spawn(_ep_worker, world)
    for r, m in out.items():
        assert m["lp"] < 2e-4 and m["g"] < 2e-3, (r, m)


def _worker_cfg(**par):
    return dict(precision="float32", train_global_batch_size=4, train_micro_batch_size=1, max_total_sequence_length=64, max_grad_norm=1.0,
                logprob_batch_size=2, optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=1e-3, weight_decay=0.0)), parallel=par)


def _train_data():
    from rl_b200.distributed.batched_data_dict import BatchedDataDict

    g = torch.Generator().manual_seed(0)
    return BatchedDataDict(input_ids=torch.randint(0, 2048, (4, 24), generator=g), input_lengths=torch.tensor([24, 17, 9, 20]),
                           token_mask=torch.ones(4, 24), sample_mask=torch.ones(4))


def _pp_worker(rank, world, tied, tp, vpp=1, layers=None):
    from rl_b200.algorithms.loss.loss_functions import NLLLossFn
    from rl_b200.models.config import preset
    from rl_b200.policy.worker import PolicyWorker

    mc = preset("tiny-llama-oracle", torch_dtype="float32", tie_word_embeddings=tied, **({"num_hidden_layers": layers} if layers else {}))
    w = PolicyWorker(_worker_cfg(pipeline_parallel_size=world // tp, tensor_parallel_size=tp, virtual_pipeline_stages=vpp), model_cfg=mc,
                     init_reference_model=False, seed=4)
    if vpp > 1:
        assert w.model.vpp == vpp and len(w.model.chunk_bounds) == vpp and w.pipeline.vpp == vpp
    data = _train_data()
    lp = w.get_logprobs(data)["logprobs"]
    outs = [w.train(data, NLLLossFn(), gbs=4, mbs=1) for _ in range(2)]
    lp2 = w.get_logprobs(data)["logprobs"]
    return dict(lp=lp.sum().item(), lp2=lp2.sum().item(), loss=[float(o["loss"][0]) for o in outs], gn=[float(o["grad_norm"][0]) for o in outs])


def _single_reference(tied, layers=None):
    from rl_b200.algorithms.loss.loss_functions import NLLLossFn
    from rl_b200.models.config import preset
    from rl_b200.parallel.state import reset_parallel
    from rl_b200.policy.worker import PolicyWorker

    reset_parallel()
    mc = preset("tiny-llama-oracle", torch_dtype="float32", tie_word_embeddings=tied, **({"num_hidden_layers": layers} if layers else {}))
    w = PolicyWorker(_worker_cfg(), model_cfg=mc, init_reference_model=False, seed=4)
    data = _train_data()
    lp = w.get_logprobs(data)["logprobs"]
    outs = [w.train(data, NLLLossFn(), gbs=4, mbs=1) for _ in range(2)]
    lp2 = w.get_logprobs(data)["logprobs"]
    return dict(lp=lp.sum().item(), lp2=lp2.sum().item(), loss=[float(o["loss"][0]) for o in outs], gn=[float(o["grad_norm"][0]) for o in outs])


@pytest.mark.parametrize("world,tp,tied", [(2, 1, False), (2, 1, True), (4, 2, True)])
def test_pipeline_parallel_worker_matches_single_rank(world, tp, tied):
    ref = _single_reference(tied)
    out = _spawn(_pp_worker, world, tied, tp)
    for r, m in out.items():
        assert m["lp"] == pytest.approx(ref["lp"], rel=1e-5), (r, m, ref)
        assert m["loss"] == pytest.approx(ref["loss"], rel=1e-4), (r, m, ref)
        assert m["gn"] == pytest.approx(ref["gn"], rel=2e-3), (r, m, ref)
        assert m["lp2"] == pytest.approx(ref["lp2"], rel=1e-4), (r, m, ref)


def _cp_worker(rank, world):
    from rl_b200.algorithms.loss.loss_functions import NLLLossFn
    from rl_b200.models.config import preset
    from rl_b200.policy.worker import PolicyWorker

    mc = preset("tiny-llama-oracle", torch_dtype="float32")
    w = PolicyWorker(_worker_cfg(context_parallel_size=world), model_cfg=mc, init_reference_model=False, seed=4)
    data = _train_data()
    lp = w.get_logprobs(data)["logprobs"]
    outs = [w.train(data, NLLLossFn(), gbs=4, mbs=2) for _ in range(2)]
    lp2 = w.get_logprobs(data)["logprobs"]
    return dict(lp=lp.sum().item(), lp2=lp2.sum().item(), loss=[float(o["loss"][0]) for o in outs], gn=[float(o["grad_norm"][0]) for o in outs])


def _ring_worker(rank, world):
    """Ring attention on the zig-zag shards of a packed stream against dense masked attention on the whole stream."""
    from rl_b200.parallel.context import CP, cp_attention_varlen

    torch.manual_seed(0)
    hq, hkv, d, T = 4, 2, 8, 16 * world
    cu = torch.tensor([0, 5, 5 + 3 * world, T - 2, T], dtype=torch.int32)
    qkv = torch.randn(T, (hq + 2 * hkv) * d, dtype=torch.float64)
    g = torch.randn(T, hq * d, dtype=torch.float64)
    cp = CP(None, rank, world)
    idx = cp.local_index(T)
    x = qkv[idx].clone().requires_grad_(True)
    out = cp_attention_varlen(x, cu, cp, hq, hkv, d, total_rows=T)
    (out * g[idx]).sum().backward()
    # dense statement
    xf = qkv.clone().requires_grad_(True)
    q = xf[:, : hq * d].reshape(T, hq, d)
    k = xf[:, hq * d : (hq + hkv) * d].reshape(T, hkv, d).repeat_interleave(hq // hkv, dim=1)
    v = xf[:, (hq + hkv) * d :].reshape(T, hkv, d).repeat_interleave(hq // hkv, dim=1)
    seq = torch.searchsorted(cu[1:].long(), torch.arange(T), right=True)
    vis = (seq[:, None] == seq[None, :]) & (torch.arange(T)[None, :] <= torch.arange(T)[:, None])
    s = torch.einsum("qhd,khd->hqk", q, k) * d ** -0.5
    p = torch.softmax(s.masked_fill(~vis[None], float("-inf")), -1)
    ref = torch.einsum("hqk,khd->qhd", p, v).reshape(T, hq * d)
    (ref * g).sum().backward()
    order = cp.stream_order(T)
    return dict(fwd=(out.detach() - ref.detach()[idx]).abs().max().item(), bwd=(x.grad - xf.grad[idx]).abs().max().item(),
                perm=bool(torch.equal(torch.cat([CP(None, r, world).local_index(T) for r in range(world)])[order], torch.arange(T))))


@pytest.mark.parametrize("world", [2, 4])
def test_ring_attention_zigzag_matches_dense(world):
    out = _spawn(_ring_worker, world)
    for r, m in out.items():
        assert m["fwd"] < 1e-5 and m["bwd"] < 1e-5 and m["perm"], (r, m)


@pytest.mark.parametrize("world", [2, 4])
def test_context_parallel_worker_matches_single_rank(world):
    ref = _single_reference(False)
    out = _spawn(_cp_worker, world)
    for r, m in out.items():
        assert m["lp"] == pytest.approx(ref["lp"], rel=1e-5), (r, m, ref)
        assert m["loss"] == pytest.approx(ref["loss"], rel=1e-4), (r, m, ref)
        assert m["gn"] == pytest.approx(ref["gn"], rel=2e-3), (r, m, ref)
        assert m["lp2"] == pytest.approx(ref["lp2"], rel=1e-4), (r, m, ref)


def _filtered_worker(rank, world, par):
    from rl_b200.algorithms.loss.loss_functions import NLLLossFn
    from rl_b200.models.config import preset
    from rl_b200.policy.worker import PolicyWorker

    mc = preset("tiny-llama-oracle", torch_dtype="float32")
    w = PolicyWorker(_worker_cfg(**par), model_cfg=mc, init_reference_model=False, seed=4)
    w.train_top_k, w.train_top_p = 50, 0.9
    data = _train_data()
    lp = w.get_logprobs(data)["logprobs"]
    out = w.train(data, NLLLossFn(), gbs=4, mbs=2)
    lp2 = w.get_logprobs(data)["logprobs"]
    return dict(lp=lp.tolist(), lp2=lp2.sum().item(), loss=float(out["loss"][0]), gn=float(out["grad_norm"][0]))


@pytest.mark.parametrize("par", [dict(tensor_parallel_size=2), dict(tensor_parallel_size=2, sequence_parallel=True), dict(context_parallel_size=2)])
def test_filtered_logprobs_under_sharded_layouts_match_single_rank(par):
    """Training log-probabilities under top-k / top-p with a vocabulary-parallel head (all-to-all to row shards, no [T, V]
    on any rank), with sequence parallelism and with context parallelism, against one rank holding everything."""
    from rl_b200.parallel.state import reset_parallel

    reset_parallel()
    ref = _filtered_worker(0, 1, {})
    reset_parallel()
    out = _spawn(_filtered_worker, 2, par)
    for r, m in out.items():
        assert torch.allclose(torch.tensor(m["lp"]), torch.tensor(ref["lp"]), atol=2e-4), (r, par)
        assert m["loss"] == pytest.approx(ref["loss"], rel=1e-4) and m["gn"] == pytest.approx(ref["gn"], rel=2e-3), (r, m["loss"], ref["loss"])
        assert m["lp2"] == pytest.approx(ref["lp2"], rel=1e-4)


def _moe_cfg():
    from rl_b200.models.config import preset

    return preset("tiny-llama-oracle", torch_dtype="float32", model_type="qwen3_moe", qk_norm=True, num_experts=4, num_experts_per_tok=2,
                  moe_intermediate_size=32, norm_topk_prob=True)


def _moe_data():
    from rl_b200.distributed.batched_data_dict import BatchedDataDict

    g = torch.Generator().manual_seed(3)
    return BatchedDataDict(input_ids=torch.randint(0, 2048, (8, 20), generator=g), input_lengths=torch.tensor([20, 17, 9, 20, 12, 20, 15, 8]),
                           token_mask=torch.ones(8, 20), sample_mask=torch.ones(8))


def _ep_train_worker(rank, world):
    from rl_b200.algorithms.loss.loss_functions import NLLLossFn
    from rl_b200.policy.worker import PolicyWorker

    cfg = _worker_cfg(expert_parallel_size=world)
    cfg.update(train_global_batch_size=8, train_micro_batch_size=2)
    w = PolicyWorker(cfg, model_cfg=_moe_cfg(), init_reference_model=True, seed=4)
    assert w.flat_e is not None and w.optimizer_e is not None
    data = _moe_data().slice(rank * 4, rank * 4 + 4)
    lp = w.get_logprobs(data)["logprobs"]
    outs = [w.train(data, NLLLossFn(), gbs=8, mbs=2) for _ in range(2)]
    lp2 = w.get_logprobs(data)["logprobs"]
    ref_lp = w.get_reference_policy_logprobs(data)["reference_logprobs"]
    both = torch.stack([lp.sum(), lp2.sum(), ref_lp.sum()])
    dist.all_reduce(both)
    return dict(lp=both[0].item(), lp2=both[1].item(), ref=both[2].item(), loss=[float(o["loss"][0]) for o in outs],
                gn=[float(o["grad_norm"][0]) for o in outs])


def test_expert_parallel_worker_matches_single_rank():
    from rl_b200.algorithms.loss.loss_functions import NLLLossFn
    from rl_b200.parallel.state import reset_parallel
    from rl_b200.policy.worker import PolicyWorker

    reset_parallel()
    cfg = _worker_cfg()
    cfg.update(train_global_batch_size=8, train_micro_batch_size=2)
    w = PolicyWorker(cfg, model_cfg=_moe_cfg(), init_reference_model=False, seed=4)
    data = _moe_data()
    ref = dict(lp=w.get_logprobs(data)["logprobs"].sum().item())
    outs = [w.train(data, NLLLossFn(), gbs=8, mbs=2) for _ in range(2)]
    ref.update(lp2=w.get_logprobs(data)["logprobs"].sum().item(), loss=[float(o["loss"][0]) for o in outs], gn=[float(o["grad_norm"][0]) for o in outs])
    out = _spawn(_ep_train_worker, 2)
    for r, m in out.items():
        assert m["lp"] == pytest.approx(ref["lp"], rel=1e-5), (r, m, ref)
        assert m["ref"] == pytest.approx(ref["lp"], rel=1e-5), (r, m, ref)   # the reference copy keeps the initial weights
        assert m["loss"] == pytest.approx(ref["loss"], rel=1e-4), (r, m, ref)
        assert m["gn"] == pytest.approx(ref["gn"], rel=2e-3), (r, m, ref)
        assert m["lp2"] == pytest.approx(ref["lp2"], rel=1e-4), (r, m, ref)


def _ckpt_worker(rank, world, mode, path):
    from rl_b200.policy.worker import PolicyWorker

    par = dict(tensor_parallel_size=world) if mode == "tp" else (dict(pipeline_parallel_size=world) if mode == "pp" else dict(expert_parallel_size=world))
    mc = _moe_cfg() if mode == "ep" else __import__("rl_b200.models.config", fromlist=["preset"]).preset("tiny-llama-oracle", torch_dtype="float32")
    w = PolicyWorker(_worker_cfg(**par), model_cfg=mc, init_reference_model=False, seed=9)
    w.save_checkpoint(os.path.join(path, "weights"), os.path.join(path, "optimizer"))
    dist.barrier()
    return sorted(os.listdir(os.path.join(path, "weights")))


@pytest.mark.parametrize("mode", ["tp", "pp", "ep"])
def test_model_parallel_checkpoint_loads_into_single_rank(tmp_path, mode):
    from rl_b200.models.config import preset
    from rl_b200.models.hf_io import load_pretrained
    from rl_b200.models.transformer import build_model
    from rl_b200.parallel.state import reset_parallel

    reset_parallel()
    out = _spawn(_ckpt_worker, 2, mode, str(tmp_path))
    files = out[0]
    assert "config.json" in files and any(f.endswith(".safetensors") for f in files)
    mc = _moe_cfg() if mode == "ep" else preset("tiny-llama-oracle", torch_dtype="float32")
    ref = build_model(mc, dtype=torch.float32, seed=9)
    got = load_pretrained(str(tmp_path / "weights"), dtype=torch.float32)
    for (n, a), (_, b) in zip(ref.named_parameters(), got.named_parameters()):
        assert torch.equal(a, b), n
    assert len(os.listdir(tmp_path / "optimizer")) == 2


def _ep_gen_worker(rank, world):
    from rl_b200.distributed.batched_data_dict import BatchedDataDict
    from rl_b200.policy.worker import PolicyWorker

    cfg = _worker_cfg(expert_parallel_size=world)
    cfg["generation"] = dict(max_new_tokens=6 + 9 * rank, temperature=1.0, stop_token_ids=[], kv_cache_tokens=2048, block_size=16, max_running=8)
    w = PolicyWorker(cfg, model_cfg=_moe_cfg(), init_reference_model=False, init_optimizer=False, seed=4)
    gen = w.build_generation()
    gen.prepare_for_generation()
    g = torch.Generator().manual_seed(10 + rank)
    n = 2 + 3 * rank  # uneven work: rank 1 has more and longer requests
    ids = torch.randint(0, 2048, (n, 10), generator=g)
    out = gen.generate(BatchedDataDict(input_ids=ids, input_lengths=torch.full((n,), 10)), greedy=True)
    gen.finish_generation()
    return out["output_ids"].tolist()


def test_expert_parallel_generation_runs_in_lock_step():
    """Ranks of an expert-parallel group serve different numbers of requests of different lengths; the engine keeps their
    forward passes aligned, and every rank's greedy output equals what a model holding all experts generates."""
    from rl_b200.distributed.batched_data_dict import BatchedDataDict
    from rl_b200.parallel.state import reset_parallel
    from rl_b200.policy.worker import PolicyWorker

    out = _spawn(_ep_gen_worker, 2)
    reset_parallel()
    for rank in range(2):
        cfg = _worker_cfg()
        cfg["generation"] = dict(max_new_tokens=6 + 9 * rank, temperature=1.0, stop_token_ids=[], kv_cache_tokens=2048, block_size=16, max_running=8)
        w = PolicyWorker(cfg, model_cfg=_moe_cfg(), init_reference_model=False, init_optimizer=False, seed=4)
        gen = w.build_generation()
        gen.prepare_for_generation()
        g = torch.Generator().manual_seed(10 + rank)
        n = 2 + 3 * rank
        ids = torch.randint(0, 2048, (n, 10), generator=g)
        ref = gen.generate(BatchedDataDict(input_ids=ids, input_lengths=torch.full((n,), 10)), greedy=True)["output_ids"].tolist()
        assert out[rank] == ref


def _reshard_gen_worker(rank, world, tp_train, tp_serve):
    from rl_b200.algorithms.grpo import refit_policy_generation
    from rl_b200.distributed.batched_data_dict import BatchedDataDict
    from rl_b200.models.config import preset
    from rl_b200.policy.worker import PolicyWorker

    cfg = _worker_cfg(tensor_parallel_size=tp_train)
    cfg["generation"] = dict(max_new_tokens=8, temperature=1.0, stop_token_ids=[], kv_cache_tokens=2048, block_size=16, max_running=8,
                             native_cfg=dict(tensor_parallel_size=tp_serve))
    mc = preset("tiny-llama-oracle", torch_dtype="float32")
    w = PolicyWorker(cfg, model_cfg=mc, init_reference_model=False, seed=4)
    gen = w.build_generation()
    dp_rank = rank // tp_train
    g = torch.Generator().manual_seed(20 + dp_rank)
    ids = torch.randint(0, 2048, (3, 10), generator=g)
    data = BatchedDataDict(input_ids=ids, input_lengths=torch.full((3,), 10))
    outs = []
    for it in range(2):
        refit_policy_generation(w, gen)
        before = gen.engine.stats["generated_tokens"]
        outs.append(gen.generate(data, greedy=True)["output_ids"].tolist())
        gen.finish_generation()
        if tp_serve < tp_train:
            # the engines inside one training group hold the same prompts and split them: this rank generated its share only
            mine = len(range(rank % tp_train // tp_serve, 3, tp_train // tp_serve))
            assert gen.engine.stats["generated_tokens"] - before == mine * 8, (rank, mine)
        if it == 0:  # change the trainer's weights: the next refit must carry them over
            with torch.no_grad():
                w.flat.flat.mul_(1.25)
    return outs


@pytest.mark.parametrize("tp_train,tp_serve", [(1, 2), (2, 1)])
def test_generation_with_a_different_tensor_parallel_size(tp_train, tp_serve):
    """Data-parallel training with tensor-parallel serving (prompts pooled inside the serving group) and the reverse: greedy
    outputs equal those of a single-rank model, before and after a weight change + refit."""
    from rl_b200.distributed.batched_data_dict import BatchedDataDict
    from rl_b200.models.config import preset
    from rl_b200.parallel.state import reset_parallel
    from rl_b200.policy.worker import PolicyWorker

    out = _spawn(_reshard_gen_worker, 2, tp_train, tp_serve)
    reset_parallel()
    mc = preset("tiny-llama-oracle", torch_dtype="float32")
    for rank in range(2):
        cfg = _worker_cfg()
        cfg["generation"] = dict(max_new_tokens=8, temperature=1.0, stop_token_ids=[], kv_cache_tokens=2048, block_size=16, max_running=8)
        w = PolicyWorker(cfg, model_cfg=mc, init_reference_model=False, seed=4)
        gen = w.build_generation()
        g = torch.Generator().manual_seed(20 + rank // tp_train)
        ids = torch.randint(0, 2048, (3, 10), generator=g)
        data = BatchedDataDict(input_ids=ids, input_lengths=torch.full((3,), 10))
        for it in range(2):
            gen.prepare_for_generation()
            ref = gen.generate(data, greedy=True)["output_ids"].tolist()
            gen.finish_generation()
            assert out[rank][it] == ref, (rank, it)
            with torch.no_grad():
                w.flat.flat.mul_(1.25)


def _ep_uneven_worker(rank, world):
    from rl_b200.algorithms.loss.loss_functions import NLLLossFn
    from rl_b200.distributed.batched_data_dict import BatchedDataDict
    from rl_b200.policy.worker import PolicyWorker

    cfg = _worker_cfg(expert_parallel_size=world)
    cfg.update(train_global_batch_size=6, train_micro_batch_size=1, logprob_batch_size=1)
    w = PolicyWorker(cfg, model_cfg=_moe_cfg(), init_reference_model=False, seed=4)
    n = 1 + 4 * rank  # rank 0 has one sample (one micro-batch), rank 1 five
    g = torch.Generator().manual_seed(rank)
    data = BatchedDataDict(input_ids=torch.randint(0, 2048, (n, 12), generator=g), input_lengths=torch.full((n,), 12),
                           token_mask=torch.ones(n, 12), sample_mask=torch.ones(n))
    lp = w.get_logprobs(data)["logprobs"]
    out = w.train(data, NLLLossFn(), gbs=2 * n, mbs=1)   # one optimizer step over each rank's samples
    return dict(lp=float(lp.sum()), loss=float(out["loss"][0]), gn=float(out["grad_norm"][0]))


def test_expert_parallel_ranks_with_unequal_microbatch_counts_do_not_deadlock():
    out = _spawn(_ep_uneven_worker, 2)
    assert out[0]["loss"] == pytest.approx(out[1]["loss"]) and out[0]["gn"] == pytest.approx(out[1]["gn"], rel=1e-4)
    assert all(abs(m["lp"]) > 0 for m in out.values())


def _sc_worker(rank, world):
    """Single-controller GRPO on two data-parallel ranks: every rank runs its own pumps in the fixed interleaved order."""
    from rl_b200.algorithms import grpo
    from rl_b200.algorithms.single_controller import SingleController
    from rl_b200.data.datasets.synthetic import RandomTokenPromptDataset
    from rl_b200.environments.synthetic import TokenFractionEnv
    from rl_b200.models.config import preset

    mc = preset("tiny-llama-oracle", torch_dtype="float32")
    ds = RandomTokenPromptDataset(128, 4, 8, 2048, seed=0)
    env = {"synthetic": TokenFractionEnv({"target_token_id": 7})}
    cfg = {"grpo": dict(num_prompts_per_step=4, num_generations_per_prompt=2, max_num_steps=3, val_period=0, seed=0),
           "loss_fn": dict(use_importance_sampling_correction=True, reference_policy_kl_penalty=0.0),
           "single_controller": dict(pump_mode="interleaved", max_trajectory_age_steps=1, rollout_ahead_batches=2),
           "policy": dict(precision="float32", train_global_batch_size=8, train_micro_batch_size=2, logprob_batch_size=4,
                          max_total_sequence_length=48, max_grad_norm=1.0, optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=1e-3)),
                          generation=dict(max_new_tokens=6, temperature=1.0, stop_token_ids=[], kv_cache_tokens=2048, block_size=8, max_running=16)),
           "logger": dict(log_dir=f"/tmp/rlb_sc_test_{os.getpid()}"), "checkpointing": dict(enabled=False)}
    policy, gen, loader, _, loss_fn, logger, ck, ss, cfg = grpo.setup(cfg, None, ds, None, env, model_cfg=mc)
    hist = []
    sc = SingleController(policy, gen, loader, None, loss_fn, env, cfg, logger=logger, save_state=ss, step_callback=lambda s, m: hist.append(m["train"]))
    sc.run()
    w = next(policy.model.parameters()).detach().double().sum().item()
    return dict(steps=len(hist), loss=[h["loss"] for h in hist], gn=[h["grad_norm"] for h in hist], ages=[h["trajectory_age"] for h in hist], w=w,
                trained=sc.stats["samples_trained"])


def test_single_controller_on_two_ranks_stays_in_lock_step():
    out = _spawn(_sc_worker, 2)
    a, b = out[0], out[1]
    assert a["steps"] == b["steps"] == 3 and a["trained"] == b["trained"] == 3 * 4
    assert a["loss"] == pytest.approx(b["loss"]) and a["gn"] == pytest.approx(b["gn"])     # global-batch metrics agree
    assert a["w"] == pytest.approx(b["w"], rel=1e-12) and max(a["ages"]) <= 1             # replicas hold the same weights


@pytest.mark.parametrize("world,tp,tied,vpp,layers", [(2, 1, False, 2, 4), (2, 1, True, 2, 5), (4, 2, False, 3, 6)])
def test_interleaved_pipeline_worker_matches_single_rank(world, tp, tied, vpp, layers):
    """Virtual pipeline stages: every rank owns ``vpp`` runs of layers (the last run may be short or empty) and the interleaved
    schedule gives the single-rank losses, gradient norms and updated log-probabilities."""
    ref = _single_reference(tied, layers)
    out = _spawn(_pp_worker, world, tied, tp, vpp, layers)
    for r, m in out.items():
        assert m["lp"] == pytest.approx(ref["lp"], rel=1e-5), (r, m, ref)
        assert m["loss"] == pytest.approx(ref["loss"], rel=1e-4), (r, m, ref)
        assert m["gn"] == pytest.approx(ref["gn"], rel=2e-3), (r, m, ref)
        assert m["lp2"] == pytest.approx(ref["lp2"], rel=1e-4), (r, m, ref)


@pytest.mark.parametrize("P,V,n", [(2, 2, 4), (3, 2, 6), (4, 2, 8), (4, 4, 16), (8, 3, 16), (4, 2, 5), (3, 4, 1)])
def test_interleaved_schedule_is_complete_ordered_and_tight(P, V, n):
    from rl_b200.parallel.pipeline import interleaved_schedule

    for train in (True, False):
        ticks = interleaved_schedule(P, V, n, train)
        arrived, done = set(), set()
        for ops, msgs in ticks:
            for r, o in enumerate(ops):
                if o is None:
                    continue
                kind, m, c = o
                s = c * P + r
                assert (r, kind, m, c) not in done
                if kind == "F":
                    assert s == 0 or (r, "F", m, c) in arrived           # the activation got here in an earlier tick
                else:
                    assert (r, "F", m, c) in done and (s == P * V - 1 or (r, "B", m, c) in arrived)
                done.add((r, kind, m, c))
            for (src, dst, kind, m, c) in msgs:
                assert ops[src] is not None and dst == (src + (1 if kind == "F" else -1)) % P
                arrived.add((dst, kind, m, c))
        assert len(done) == (2 if train else 1) * n * V * P              # every chunk of every micro-batch ran on every rank
        if n % P == 0 and train:   # the bubble is 2 (P - 1) chunk-sized slots, i.e. 1 / V of the plain schedule's
            assert len(ticks) == 2 * n * V + 2 * (P - 1)
        if not train:
            assert len(ticks) >= n * V + P - 1


def test_parallel_sizes_reads_both_spellings_of_virtual_stages():
    from rl_b200.policy.worker import parallel_sizes

    assert parallel_sizes(dict(parallel=dict(pipeline_parallel_size=2, virtual_pipeline_stages=3)))["vpp"] == 3
    mg = dict(megatron_cfg=dict(enabled=True, pipeline_model_parallel_size=4, virtual_pipeline_model_parallel_size=2))
    assert parallel_sizes(mg)["vpp"] == 2 and parallel_sizes(mg)["pp"] == 4
    mg = dict(megatron_cfg=dict(enabled=True, pipeline_model_parallel_size=2, num_layers_per_virtual_pipeline_stage=4))
    assert parallel_sizes(mg, num_layers=32)["vpp"] == 4 and parallel_sizes(mg)["vpp"] == 1
    with pytest.raises(ValueError):
        parallel_sizes(dict(parallel=dict(virtual_pipeline_stages=2)))


def test_interleaved_stages_cover_the_checkpoint_names_once():
    """The chunks of all pipeline ranks together hold every HF tensor exactly once (the embedding twice when it is tied and the
    last rank needs it for the output head), under the same names and values as the whole model."""
    from rl_b200.models.config import preset
    from rl_b200.models.hf_io import iter_hf_tensors, load_hf_tensors
    from rl_b200.models.transformer import build_model

    cfg = preset("tiny-llama-oracle", torch_dtype="float32", num_hidden_layers=7)
    full = build_model(cfg, dtype=torch.float32, seed=3)
    sd = dict(iter_hf_tensors(full))
    seen: dict = {}
    for r in range(2):
        part = build_model(cfg, dtype=torch.float32, seed=50 + r, pp_rank=r, pp_size=2, vpp=3)
        assert part.layer_ids == [i for c in range(3) for i in range((c * 2 + r) * 2, min(7, (c * 2 + r) * 2 + 2))]
        load_hf_tensors(part, sd.get)
        for n, t in iter_hf_tensors(part):
            assert n not in seen and torch.equal(t, sd[n]), n
            seen[n] = r
    assert set(seen) == set(sd)
