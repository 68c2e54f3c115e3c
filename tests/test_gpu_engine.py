"""Generation engine on the GPU: scheduler + paged KV + CUDA-graph decode + sampler, checked against the trainer's
own log-probabilities of the generated tokens (the two halves of a GRPO step must agree), plus prefix sharing and
a training step through the native kernels."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _policy(layers=2, **gen):
    from rl_b200.models.config import ModelConfig
    from rl_b200.policy.worker import PolicyWorker

    mc = ModelConfig(model_type="llama", vocab_size=8192, hidden_size=512, intermediate_size=1408, num_hidden_layers=layers,
                     num_attention_heads=8, num_key_value_heads=2, head_dim=128, rope_theta=500000.0)
    g = dict(max_new_tokens=24, stop_token_ids=[], kv_cache_tokens=16384, block_size=16, max_running=32)
    g.update(gen)
    p = PolicyWorker(dict(precision="bfloat16", train_global_batch_size=8, train_micro_batch_size=4, max_total_sequence_length=512,
                          optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=1e-4)), generation=g),
                     model_cfg=mc, device="cuda:0", init_reference_model=True, seed=3)
    return p, p.build_generation()


@pytest.mark.parametrize("graphs", [True, False])
def test_engine_matches_trainer_logprobs(native_lib, graphs):
    from rl_b200.distributed.batched_data_dict import BatchedDataDict
    from rl_b200.ops.lib import check_status

    torch.manual_seed(0)
    policy, gen = _policy(use_cuda_graphs=graphs)
    B, P = 12, 40
    lens = torch.randint(20, P + 1, (B,))
    ids = torch.zeros((B, P), dtype=torch.long)
    for i in range(B):
        ids[i, : lens[i]] = torch.randint(1, 8192, (int(lens[i]),))
    # rows 0..3 share one prompt (prefix sharing path)
    for i in range(1, 4):
        ids[i] = ids[0]
        lens[i] = lens[0]
    out = gen.generate(BatchedDataDict(input_ids=ids, input_lengths=lens))
    assert check_status() == 0
    assert (out["generation_lengths"] == 24).all()
    # siblings sample different continuations
    g0 = out["output_ids"][0, int(lens[0]) : int(lens[0]) + 24]
    g1 = out["output_ids"][1, int(lens[1]) : int(lens[1]) + 24]
    assert not torch.equal(g0, g1)
    data = BatchedDataDict(input_ids=out["output_ids"], input_lengths=out["unpadded_sequence_lengths"])
    lp = policy.get_logprobs(data)["logprobs"]
    mask = out["logprobs"] != 0
    err = (lp - out["logprobs"]).abs()[mask]
    assert err.mean().item() < 0.03, f"mean |trainer - engine| logprob gap {err.mean().item():.4f}"
    assert err.max().item() < 0.5


def test_greedy_is_deterministic_and_consistent(native_lib):
    from rl_b200.distributed.batched_data_dict import BatchedDataDict

    policy, gen = _policy()
    ids = torch.randint(1, 8192, (5, 33))
    lens = torch.full((5,), 33)
    a = gen.generate(BatchedDataDict(input_ids=ids, input_lengths=lens), greedy=True)
    b = gen.generate(BatchedDataDict(input_ids=ids, input_lengths=lens), greedy=True)
    assert torch.equal(a["output_ids"], b["output_ids"])


def test_preemption_under_tight_cache(native_lib):
    from rl_b200.distributed.batched_data_dict import BatchedDataDict

    # 20 sequences x (32 + 64) tokens need 120 blocks of 16; give the cache 64 so that the scheduler must queue / preempt
    policy, gen = _policy(kv_cache_tokens=None, max_new_tokens=64)
    gen.engine.sleep(True)
    from rl_b200.engine.engine import GenerationEngine

    gen.engine = GenerationEngine(policy.model, block_size=16, num_blocks=64, max_running=32, max_model_len=512)
    ids = torch.randint(1, 8192, (20, 32))
    out = gen.generate(BatchedDataDict(input_ids=ids, input_lengths=torch.full((20,), 32)))
    assert (out["generation_lengths"] == 64).all()


def test_train_step_changes_weights_and_ref_is_frozen(native_lib):
    from rl_b200.algorithms.loss.loss_functions import NLLLossFn
    from rl_b200.distributed.batched_data_dict import BatchedDataDict
    from rl_b200.ops.lib import check_status

    policy, _ = _policy()
    ids = torch.randint(1, 8192, (8, 64))
    data = BatchedDataDict(input_ids=ids, input_lengths=torch.full((8,), 64), token_mask=torch.ones(8, 64), sample_mask=torch.ones(8))
    before = policy.flat.flat.clone()
    l0 = policy.get_logprobs(data)["logprobs"]
    r0 = policy.get_reference_policy_logprobs(data)["reference_logprobs"]
    assert torch.allclose(l0, r0)
    losses = []
    for _ in range(3):
        losses.append(float(policy.train(data, NLLLossFn(), gbs=8, mbs=4)["loss"][0]))
    assert check_status() == 0
    assert losses[-1] < losses[0], losses
    assert not torch.equal(before, policy.flat.flat)
    r1 = policy.get_reference_policy_logprobs(data)["reference_logprobs"]
    assert torch.equal(r0, r1)


def test_model_matches_fp32_reference(native_lib):
    """Native bf16 forward/backward vs the same model evaluated by the PyTorch restatement in fp32 on CPU."""
    from rl_b200.models.config import ModelConfig
    from rl_b200.models.transformer import CausalLM, PackedBatch

    mc = ModelConfig(model_type="qwen3", vocab_size=4096, hidden_size=256, intermediate_size=768, num_hidden_layers=2,
                     num_attention_heads=4, num_key_value_heads=2, head_dim=128, qk_norm=True, rope_theta=1e6, rms_norm_eps=1e-6)
    ref = CausalLM(mc, dtype=torch.float32, device="cpu", seed=5)
    gpu = CausalLM(mc, dtype=torch.bfloat16, device="cuda:0", seed=5)
    with torch.no_grad():
        for a, b in zip(gpu.parameters(), ref.parameters()):
            b.copy_(a.float().cpu())
    ids = torch.randint(0, 4096, (3, 50))
    lens = torch.tensor([50, 31, 17])
    bc = PackedBatch.from_padded(ids, lens)
    bg = PackedBatch.from_padded(ids.cuda(), lens.cuda())
    bg.input_ids = bg.input_ids.to(torch.int32)
    lr, _ = ref.next_token_logprobs(bc)
    lg, _ = gpu.next_token_logprobs(bg)
    assert (lr - lg.cpu()).abs().max().item() < 0.15
    lr.sum().backward()
    lg.sum().backward()
    for (n, a), b in zip(gpu.named_parameters(), ref.parameters()):
        ga, gb = a.grad.float().cpu(), b.grad
        denom = gb.abs().max().item() + 1e-6
        assert (ga - gb).abs().max().item() / denom < 0.08, n


def test_windowed_decode_matches_single_step_decode(native_lib):
    """The device-resident multi-step decode (the host looks once per window) must produce exactly the tokens and
    log-probabilities of one host visit per step: same seeds, ragged length limits, a stop token in the vocabulary."""
    from rl_b200.engine.engine import GenerationEngine, SamplingParams
    from rl_b200.ops.lib import check_status

    policy, _ = _policy()
    torch.manual_seed(1)
    prompts = [torch.randint(1, 8192, (int(n),)).tolist() for n in torch.randint(5, 60, (11,))]
    limits = [3, 40, 17, 16, 1, 33, 40, 2, 25, 40, 31]
    outs = []
    for window in (1, 16, 5):
        eng = GenerationEngine(policy.model, block_size=16, kv_cache_tokens=8192, max_running=8, max_model_len=512, decode_window=window)
        assert eng.decode_window == window
        # a sampled id below 200 ends a sequence: some rows stop in the middle of a window
        sp = SamplingParams(temperature=1.0, max_new_tokens=40, stop_token_ids=list(range(200)), seed=5)
        recs = eng.generate(prompts, sp, max_new_tokens=limits)
        assert check_status() == 0
        outs.append([(r.out_tokens, r.out_logprobs, r.truncated) for r in recs])
        steps = eng.stats["decode_steps"]
        eng.sleep(True)
    for a, b in zip(outs[0], outs[1]):
        assert a[0] == b[0] and a[2] == b[2]
        assert max(abs(x - y) for x, y in zip(a[1], b[1])) < 1e-5
    assert [o[0] for o in outs[0]] == [o[0] for o in outs[2]]
    assert any(len(o[0]) < lim for o, lim in zip(outs[0], limits))      # some row hit a stop token
    assert any(len(o[0]) == lim and o[2] for o, lim in zip(outs[0], limits))   # some row ran into its limit


def test_fused_decode_step_matches_layer_by_layer_decode(native_lib, monkeypatch):
    """Greedy decoding with the norms and SwiGLU folded into the projections must pick the same tokens as the
    layer-by-layer decode step, with log-probabilities equal to bf16 rounding."""
    from rl_b200.engine.engine import GenerationEngine, SamplingParams

    policy, _ = _policy(layers=3)
    torch.manual_seed(2)
    prompts = [torch.randint(1, 8192, (int(n),)).tolist() for n in torch.randint(8, 50, (9,))]
    outs = []
    for fused in ("1", "0"):
        monkeypatch.setenv("RLB_FUSED_DECODE", fused)
        eng = GenerationEngine(policy.model, block_size=16, kv_cache_tokens=8192, max_running=16, max_model_len=256)
        assert eng._can_fuse_decode(9) == (fused == "1")
        recs = eng.generate(prompts, SamplingParams(max_new_tokens=12, stop_token_ids=[], greedy=True, seed=0))
        outs.append(recs)
        eng.sleep(True)
    same = sum(a.out_tokens == b.out_tokens for a, b in zip(*outs))
    assert same >= len(prompts) - 1      # a near-tie may flip under a different rounding point; not more than one row
    for a, b in zip(*outs):
        if a.out_tokens == b.out_tokens:
            assert max(abs(x - y) for x, y in zip(a.out_logprobs, b.out_logprobs)) < 0.08


def test_prefix_cache_and_chunked_prefill_match_plain_prefill(native_lib):
    """A second generate call whose prompts extend the first call's prompts (the next turn of a rollout) prefills only the
    new tokens, and a prompt longer than the prefill budget runs in chunks; both give the tokens and log-probabilities of
    a plain full prefill."""
    from rl_b200.engine.engine import GenerationEngine, SamplingParams
    from rl_b200.ops.lib import check_status

    policy, _ = _policy(layers=2)
    torch.manual_seed(4)
    first = [torch.randint(1, 8192, (int(n),)).tolist() for n in (70, 33, 100)]
    sp = SamplingParams(max_new_tokens=6, stop_token_ids=[], greedy=True, seed=0)

    def run(prefix_cache, budget):
        eng = GenerationEngine(policy.model, block_size=16, kv_cache_tokens=8192, max_running=8, max_model_len=512,
                               max_prefill_tokens=budget, enable_prefix_caching=prefix_cache)
        a = eng.generate(first, sp)
        turn2 = [p + r.out_tokens + torch.randint(1, 8192, (9,), generator=torch.Generator().manual_seed(i)).tolist()
                 for i, (p, r) in enumerate(zip(first, a))]
        t0 = eng.stats["prefill_tokens"]
        b = eng.generate(turn2, sp)
        stats = dict(eng.stats, second_call_prefill=eng.stats["prefill_tokens"] - t0,
                     cache=eng.sched.cache_stats() if prefix_cache else None)
        assert check_status() == 0
        eng.sleep(True)
        return [(r.out_tokens, r.out_logprobs) for r in a + b], stats, [len(t) for t in turn2]

    plain, st_plain, lens2 = run(False, 16384)
    cached, st_cached, _ = run(True, 16384)
    chunked, st_chunk, _ = run(False, 48)           # every prompt above 48 tokens is split into chunks
    both, st_both, _ = run(True, 40)
    for other in (cached, chunked, both):
        for (t0, l0), (t1, l1) in zip(plain, other):
            assert t0 == t1
            assert max(abs(x - y) for x, y in zip(l0, l1)) < 0.05
    # second call without the cache prefills whole prompts; with it only what lies beyond the cached full blocks
    assert st_plain["second_call_prefill"] == sum(lens2)
    want_new = sum(L - min((len(p) // 16) * 16, ((L - 1) // 16) * 16) for p, L in zip(first, lens2))
    assert st_cached["second_call_prefill"] == want_new, (st_cached, want_new)
    assert st_cached["cache"]["hits"] == 3 and st_cached["cached_prefix_tokens"] == sum(lens2) - want_new
    assert st_both["second_call_prefill"] == want_new
