"""Low-precision rollout: quantised weight copies are used only inside the engine's generation phase, are refreshed in
place on refit, and give log-probabilities close to the bf16 policy."""

import torch

from rl_b200.engine import quantized as QZ
from rl_b200.engine.engine import GenerationEngine, SamplingParams
from rl_b200.models.config import ModelConfig
from rl_b200.models.transformer import CausalLM, PackedBatch
from rl_b200.ops import functional as F


def _model():
    mc = ModelConfig(vocab_size=128, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                     head_dim=32, torch_dtype="float32")
    return CausalLM(mc, dtype=torch.float32, device="cpu", seed=1)


def test_quantized_linear_is_scoped_and_close():
    torch.manual_seed(0)
    m = _model()
    for kind, tol in (("mxfp8", 0.08), ("fp8", 0.05)):
        info = QZ.quantize_model(m, kind)
        assert info["tensors"] == 2 * 4 and info["quantized_bytes"] < 0.6 * info["bf16_bytes"]
        w = m.layers[0].mlp.down_proj
        x = torch.randn(5, w.shape[1])
        ref = x @ w.t()
        with torch.no_grad():
            assert torch.equal(F.linear(x, w), ref)                        # outside the generation phase: full precision
            with QZ.quantized_inference(True):
                y = F.linear(x, w)
                yr = F.linear(x, w, None, torch.ones_like(ref))
        assert not torch.equal(y, ref) and (y - ref).norm() / ref.norm() < tol and torch.allclose(yr, y + 1, atol=1e-5)
        with QZ.quantized_inference(True):
            assert torch.equal(F.linear(x, w), ref)                        # autograd on: training never sees quantised weights
        bufs = [p._rlb_q[1] for _, p in m.named_parameters() if hasattr(p, "_rlb_q")]
        with torch.no_grad():
            w.mul_(2.0)
        QZ.quantize_model(m, kind)
        assert all(a is p._rlb_q[1] for a, (_, p) in zip(bufs, [(n, p) for n, p in m.named_parameters() if hasattr(p, "_rlb_q")]))  # in place
        with torch.no_grad(), QZ.quantized_inference(True):
            y2 = F.linear(x, w)
        assert (y2 - 2 * ref).norm() / (2 * ref).norm() < tol
        with torch.no_grad():
            w.mul_(0.5)
        QZ.clear_model(m)
        assert not any(hasattr(p, "_rlb_q") for p in m.parameters())


def test_engine_generates_with_quantized_weights_near_policy():
    m = _model()
    eng = GenerationEngine(m, block_size=4, num_blocks=128, max_running=8, max_model_len=64, use_cuda_graphs=False, quantization="mxfp8")
    assert eng.requantize()["tensors"] == 8
    prompts = [[1, 2, 3, 4, 5], [9, 8, 7]]
    recs = eng.generate(prompts, SamplingParams(max_new_tokens=8, stop_token_ids=[], seed=3, temperature=1.0))
    gaps = []
    for r in recs:
        seq = torch.tensor([r.prompt + r.out_tokens])
        b = PackedBatch.from_padded(seq, torch.tensor([seq.shape[1]]))
        with torch.no_grad():
            lp, _ = m.next_token_logprobs(b)
        gaps.append((lp[len(r.prompt):] - torch.tensor(r.out_logprobs)).abs())
    g = torch.cat(gaps)
    assert 0 < g.max() < 0.3            # a different (quantised) policy, but a close one
    eng_bf16 = GenerationEngine(m, block_size=4, num_blocks=128, max_running=8, max_model_len=64, use_cuda_graphs=False)
    assert eng_bf16.requantize() is None
    r2 = eng_bf16.generate(prompts, SamplingParams(max_new_tokens=8, stop_token_ids=[], seed=3, temperature=1.0))
    seq = torch.tensor([r2[0].prompt + r2[0].out_tokens])
    with torch.no_grad():
        lp, _ = m.next_token_logprobs(PackedBatch.from_padded(seq, torch.tensor([seq.shape[1]])))
    assert (lp[len(r2[0].prompt):] - torch.tensor(r2[0].out_logprobs)).abs().max() < 1e-4   # bf16 engine unaffected by leftovers
