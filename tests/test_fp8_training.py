"""MXFP8 training of the linear layers: the autograd function against the quantise / de-quantise statement of the same
arithmetic, and a loss-curve comparison with full-precision training on the tiny model."""

import pytest
import torch

from rl_b200.ops import functional as F


@pytest.fixture(autouse=True)
def _reset_fp8():
    yield
    F.Fp8Training.configure(None)


def test_mx_linear_gradients_follow_quantised_operands():
    torch.manual_seed(0)
    x = torch.randn(24, 96, requires_grad=True)
    w = torch.randn(64, 96, requires_grad=True)
    dy = torch.randn(24, 64)
    F.Fp8Training.configure(dict(enabled=True, fp8_recipe="mxfp8"))
    y = F.linear(x, w)
    y.backward(dy)
    # every GEMM contracts operands that were rounded to e4m3 with one power-of-two scale per 32 elements ALONG ITS OWN
    # contraction dimension: forward over K, input gradient over N, weight gradient over the tokens
    fq = F._mx_fake
    assert torch.allclose(y, fq(x.detach()) @ fq(w.detach()).t(), atol=1e-4)
    assert torch.allclose(x.grad, fq(dy) @ fq(w.detach().t().contiguous()).t(), atol=1e-4)
    assert torch.allclose(w.grad, fq(dy.t().contiguous()) @ fq(x.detach().t().contiguous()).t(), atol=1e-4)
    ref = x.detach() @ w.detach().t()
    assert (y - ref).abs().max() / ref.abs().max() < 0.08          # e4m3 has three mantissa bits
    assert F.Fp8Training.stats["fwd"] >= 1 and F.Fp8Training.stats["wgrad"] >= 1


def _train(fp8: bool, steps: int = 6):
    from rl_b200.algorithms.loss.loss_functions import NLLLossFn
    from rl_b200.distributed.batched_data_dict import BatchedDataDict
    from rl_b200.models.config import preset
    from rl_b200.parallel.state import reset_parallel
    from rl_b200.policy.worker import PolicyWorker

    reset_parallel()
    mc = preset("tiny-llama-oracle", torch_dtype="float32")
    cfg = dict(precision="float32", train_global_batch_size=8, train_micro_batch_size=4, max_total_sequence_length=64,
               optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=3e-3, weight_decay=0.0)),
               fp8_cfg=dict(enabled=fp8, fp8="e4m3", fp8_recipe="mxfp8"))
    w = PolicyWorker(cfg, model_cfg=mc, device="cpu", init_reference_model=False, seed=5)
    assert w.fp8_training == fp8
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, 64, (8, 24), generator=g)          # a small token set: the model can learn it in a few steps
    data = BatchedDataDict(input_ids=ids, input_lengths=torch.full((8,), 24), token_mask=torch.ones(8, 24), sample_mask=torch.ones(8))
    losses = [float(w.train(data, NLLLossFn(), gbs=8, mbs=4)["loss"][0]) for _ in range(steps)]
    return losses, w


def test_mxfp8_training_tracks_full_precision_loss_curve():
    full, _ = _train(False)
    fp8, w = _train(True)
    assert full[-1] < full[0] - 0.5 and fp8[-1] < fp8[0] - 0.5            # both learn
    assert max(abs(a - b) / a for a, b in zip(full, fp8)) < 0.06, (full, fp8)   # and stay within a few per cent of each other
    # the output head, embedding and norms were kept out of FP8
    assert getattr(w.model.lm_head, "_rlb_keep_bf16", False) and getattr(w.model.embed_tokens, "_rlb_keep_bf16", False)
