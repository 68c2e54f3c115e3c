"""Fully sharded parameters (ZeRO-3) against the resident-parameter mode: same losses, gradient norms, log-probabilities
and weights after optimizer steps, on one rank and on two gloo ranks; reference-policy swap, HF save / load and the
serving copy used for generation."""

import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from test_parallel_cpu import _spawn  # noqa: E402


def _cfg(full: bool, **over):
    c = dict(precision="float32", train_global_batch_size=8, train_micro_batch_size=2, max_total_sequence_length=64, max_grad_norm=0.5,
             optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=5e-3, weight_decay=0.01)),
             parallel=dict(data_parallel_sharding="full" if full else "optimizer"),
             generation=dict(max_new_tokens=6, temperature=1.0, stop_token_ids=[], kv_cache_tokens=2048, block_size=16, max_running=8))
    c.update(over)
    return c


def _data(world, rank, n=8, S=20):
    from rl_b200.distributed.batched_data_dict import BatchedDataDict

    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 2048, (n, S), generator=g)
    lens = torch.tensor([20, 13, 17, 20, 9, 20, 15, 11][:n])
    per = n // world
    sl = slice(rank * per, (rank + 1) * per)
    return BatchedDataDict(input_ids=ids[sl], input_lengths=lens[sl], token_mask=torch.ones(per, S), sample_mask=torch.ones(per))


def _run(rank, world, full, tmp, name="tiny-llama-oracle"):
    from rl_b200.algorithms.loss.loss_functions import NLLLossFn
    from rl_b200.models.config import preset
    from rl_b200.policy.worker import PolicyWorker

    mc = preset(name, torch_dtype="float32")
    w = PolicyWorker(_cfg(full), model_cfg=mc, device="cpu", init_reference_model=True, seed=5)
    assert (w.sharder is not None) == full
    data = _data(world, rank)
    out = dict(lp0=w.get_logprobs(data)["logprobs"])
    res = [w.train(data, NLLLossFn(), gbs=8, mbs=2) for _ in range(2)]
    out["loss"] = [float(r["loss"][0]) for r in res]
    out["gn"] = [float(r["grad_norm"][0]) for r in res]
    out["lp2"] = w.get_logprobs(data)["logprobs"]
    out["ref"] = w.get_reference_policy_logprobs(data)["reference_logprobs"]
    if full:
        st = w.sharder.stats
        assert st["gathers"] > 0 and st["reduce_scatters"] > 0
        # every parameter is released again: nothing full-size stays resident
        assert all(p.numel() == 0 for p in w.model.parameters())
        # generation from the serving copy, HF save / load round trip
        gen = w.build_generation()
        from rl_b200.algorithms.grpo import refit_policy_generation

        refit_policy_generation(w, gen)
        g = gen.generate(data, greedy=True)
        out["gen"] = g["output_ids"].tolist()
        gen.finish_generation()
        path = os.path.join(tmp, "ckpt")
        w.save_checkpoint(path, None, None)
        w2 = PolicyWorker(_cfg(True), model_cfg=mc, device="cpu", init_reference_model=False, seed=77)
        w2.load_checkpoint(path, None)
        out["lp_reload"] = w2.get_logprobs(data)["logprobs"]
    else:
        gen = w.build_generation()
        gen.prepare_for_generation()
        out["gen"] = gen.generate(data, greedy=True)["output_ids"].tolist()
        gen.finish_generation()
    # plain lists: tensors do not survive the trip through the result queue once the child has exited
    return {k: (v.tolist() if isinstance(v, torch.Tensor) else v) for k, v in out.items()}


@pytest.mark.parametrize("world,name", [(1, "tiny-llama-oracle"), (2, "tiny-llama-oracle"), (2, "tiny-nemotron-h")])
def test_fully_sharded_matches_resident_parameters(tmp_path, world, name):
    """(the hybrid model adds Mamba-2 blocks, stacked experts without expert parallelism and a stored router buffer)"""
    if world == 1:
        from rl_b200.parallel.state import reset_parallel

        reset_parallel()
        res = {0: _run(0, 1, False, str(tmp_path), name)}
        reset_parallel()
        full = {0: _run(0, 1, True, str(tmp_path), name)}
    else:
        res = _spawn(_run, world, False, str(tmp_path), name)
        full = _spawn(_run, world, True, str(tmp_path), name)
    for r in range(world):
        a = {k: (torch.tensor(v) if k.startswith(("lp", "ref")) else v) for k, v in res[r].items()}
        b = {k: (torch.tensor(v) if k.startswith(("lp", "ref")) else v) for k, v in full[r].items()}
        assert torch.allclose(a["lp0"], b["lp0"], atol=1e-5)
        assert a["loss"] == pytest.approx(b["loss"], rel=1e-5)
        assert a["gn"] == pytest.approx(b["gn"], rel=1e-4)
        assert torch.allclose(a["lp2"], b["lp2"], atol=2e-5)            # same weights after two clipped AdamW steps
        assert torch.allclose(a["ref"], b["ref"], atol=1e-5)            # the reference policy did not move
        assert not torch.allclose(a["lp0"], a["lp2"], atol=1e-4)
        assert a["gen"] == b["gen"]                                     # the engine serves the trained weights
        assert torch.allclose(b["lp_reload"], b["lp2"], atol=1e-6)      # HF save -> load into a fresh sharded worker


def _hsdp_run(rank, world, rep):
    from rl_b200.algorithms.loss.loss_functions import NLLLossFn
    from rl_b200.models.config import preset
    from rl_b200.policy.worker import PolicyWorker

    mc = preset("tiny-llama-oracle", torch_dtype="float32")
    cfg = _cfg(False)
    cfg["parallel"] = dict(data_parallel_replicate_size=rep)
    w = PolicyWorker(cfg, model_cfg=mc, device="cpu", init_reference_model=False, seed=5)
    data = _data(world, rank)
    res = [w.train(data, NLLLossFn(), gbs=8, mbs=2) for _ in range(2)]
    shard = w.optimizer.shard_numel * (world if rep == 1 else world // rep)
    return dict(loss=[float(r["loss"][0]) for r in res], gn=[float(r["grad_norm"][0]) for r in res], lp=w.get_logprobs(data)["logprobs"].tolist(),
                opt_world=w.optimizer.world, replicas=w.optimizer.replicas_of_shard, covered=shard == w.flat.padded)


@pytest.mark.parametrize("rep", [2, 4])
def test_hybrid_sharding_matches_fully_sharded_optimizer_state(rep):
    """Optimizer state cut inside shard groups of dp / R ranks and replicated over R groups (R = 4: plain replication) takes
    the steps that sharding over all ranks takes."""
    base = _spawn(_hsdp_run, 4, 1)
    hs = _spawn(_hsdp_run, 4, rep)
    for r in range(4):
        assert hs[r]["opt_world"] == 4 // rep and hs[r]["replicas"] == rep and hs[r]["covered"] and base[r]["opt_world"] == 4
        assert hs[r]["loss"] == pytest.approx(base[r]["loss"], rel=1e-5) and hs[r]["gn"] == pytest.approx(base[r]["gn"], rel=1e-4)
        assert torch.allclose(torch.tensor(hs[r]["lp"]), torch.tensor(base[r]["lp"]), atol=2e-5)
