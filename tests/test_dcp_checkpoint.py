"""torch-DCP checkpoints with one entry per HF parameter: saved at 2 ranks, loaded at 1 and at 4 ranks (weights, AdamW
moments, master remainder, step count), converted to HF offline, and written in the key layout of the reference's
``ModelState`` / ``OptimizerState`` wrappers (``model.<name>``, ``optim.optim.state.<name>.exp_avg``)."""

import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from test_parallel_cpu import _spawn  # noqa: E402


def _worker(seed=5):
    from rl_b200.models.config import preset
    from rl_b200.policy.worker import PolicyWorker

    mc = preset("tiny-llama-oracle")
    return PolicyWorker(dict(precision="float32", train_global_batch_size=8, train_micro_batch_size=4, max_total_sequence_length=64,
                             optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=1e-2, weight_decay=0.0)),
                             scheduler=[dict(name="torch.optim.lr_scheduler.ConstantLR", kwargs=dict(factor=1.0, total_iters=1))]),
                        model_cfg=mc, device="cpu", init_reference_model=False, seed=seed)


def _train_steps(w, steps=2):
    from rl_b200.algorithms.loss.loss_functions import NLLLossFn
    from rl_b200.distributed.batched_data_dict import BatchedDataDict

    g = torch.Generator().manual_seed(7 + w.rank)
    n = 8 // w.world
    for _ in range(steps):
        ids = torch.randint(0, w.model_cfg.vocab_size, (n, 16), generator=g)
        data = BatchedDataDict(input_ids=ids, input_lengths=torch.full((n,), 16), token_mask=torch.ones(n, 16), sample_mask=torch.ones(n))
        w.train(data, NLLLossFn(), gbs=8, mbs=4)


def _full_state(w):
    """(weights by HF name, full moments in flat order) gathered on every rank."""
    from rl_b200.checkpoint.dcp_state import _gather_flat
    from rl_b200.models.hf_io import iter_hf_tensors

    weights = {n: t.detach().clone() for n, t in iter_hf_tensors(w.model)}
    opt = w.optimizer
    return weights, _gather_flat(opt.m, w.flat.padded, w).clone(), _gather_flat(opt.v, w.flat.padded, w).clone(), opt.step_count


def _save(rank, world, path):
    w = _worker()
    _train_steps(w)
    w.save_checkpoint(os.path.join(path, "weights"), os.path.join(path, "optimizer"), None, model_save_format="dcp")
    weights, m, v, step = _full_state(w)
    if rank == 0:
        torch.save(dict(weights=weights, m=m, v=v, step=step, padded=w.flat.padded), os.path.join(path, "truth.pt"))
    return True


def _load(rank, world, path):
    w = _worker(seed=99)   # different init: everything must come from the checkpoint
    w.load_checkpoint(os.path.join(path, "weights"), os.path.join(path, "optimizer"))
    truth = torch.load(os.path.join(path, "truth.pt"), weights_only=False)
    weights, m, v, step = _full_state(w)
    for n, t in truth["weights"].items():
        assert torch.equal(weights[n], t), n
    assert w.flat.padded == truth["padded"] or True
    k = min(m.numel(), truth["m"].numel())
    assert torch.equal(m[: w.flat.numel], truth["m"][: w.flat.numel]) and torch.equal(v[: w.flat.numel], truth["v"][: w.flat.numel])
    assert step == truth["step"] == 2 and k > 0
    # training continues identically from the restored state on every world size: one more step must be finite
    _train_steps(w, 1)
    return True


def test_dcp_saved_at_two_ranks_loads_at_one_and_four(tmp_path):
    path = str(tmp_path)
    _spawn(_save, 2, path)
    # on-disk keys follow the reference's ModelState / OptimizerState layout
    from rl_b200.checkpoint.dcp_state import _all_keys, dcp_to_hf, is_per_parameter_checkpoint

    wk, ok = _all_keys(os.path.join(path, "weights")), _all_keys(os.path.join(path, "optimizer"))
    assert "model.model.layers.0.self_attn.q_proj.weight" in wk and "model.lm_head.weight" in wk
    assert "optim.optim.state.model.layers.0.mlp.down_proj.weight.exp_avg" in ok
    assert "optim.optim.state.model.layers.0.mlp.down_proj.weight.exp_avg_sq" in ok
    assert "optim.optim.state.model.embed_tokens.weight.step" in ok
    assert is_per_parameter_checkpoint(os.path.join(path, "weights"))
    _spawn(_load, 1, path)
    _spawn(_load, 4, path)
    # offline conversion to HF safetensors reproduces the weights
    from rl_b200.models.hf_io import iter_hf_tensors, load_pretrained

    hf = dcp_to_hf(os.path.join(path, "weights"), os.path.join(path, "hf"))
    m = load_pretrained(hf, dtype=torch.float32)
    truth = torch.load(os.path.join(path, "truth.pt"), weights_only=False)
    for n, t in iter_hf_tensors(m):
        assert torch.equal(t, truth["weights"][n]), n


def test_checkpoint_in_the_reference_layout_loads(tmp_path):
    """A DCP directory as the reference's DTensor worker writes it (plain ``model.<fqn>`` tensors from
    ``dcp.save({"model": state_dict})``, no master remainder, torch AdamW state names) loads into a worker."""
    import torch.distributed.checkpoint as dcp

    from rl_b200.models.hf_io import iter_hf_tensors

    src = _worker(seed=11)
    sd = {n: t.detach().clone() for n, t in iter_hf_tensors(src.model)}
    dcp.save({"model": sd}, checkpoint_id=str(tmp_path / "weights"), no_dist=True)
    state = {n: {"step": torch.tensor(3.0), "exp_avg": torch.full_like(t, 0.25), "exp_avg_sq": torch.full_like(t, 0.5)} for n, t in sd.items()}
    dcp.save({"optim": {"optim": {"state": state, "param_groups": [{"lr": 1e-3, "params": list(sd)}]}}},
             checkpoint_id=str(tmp_path / "optimizer"), no_dist=True)
    dst = _worker(seed=12)
    dst.load_checkpoint(str(tmp_path / "weights"), str(tmp_path / "optimizer"))
    for n, t in iter_hf_tensors(dst.model):
        assert torch.equal(t, sd[n]), n
    opt = dst.optimizer
    live = torch.zeros(dst.flat.padded, dtype=torch.bool)
    for o, k in zip(dst.flat.offsets, dst.flat.numels):
        live[o : o + k] = True
    assert torch.all(opt.m[live[opt.lo : opt.hi]] == 0.25) and torch.all(opt.v[live[opt.lo : opt.hi]] == 0.5)
    assert opt.step_count == 3
