"""Scheduler / block manager (C++ against its Python twin) and the engine's CPU path against the model's own
log-probabilities."""

import random

import pytest
import torch

from rl_b200.engine.engine import GenerationEngine, SamplingParams, _NativeScheduler, _PyScheduler
from rl_b200.models.config import ModelConfig
from rl_b200.models.transformer import CausalLM, PackedBatch
from rl_b200.ops import lib as L


def _drive(s, n_req, rng, bs):
    """Runs a random workload to completion; returns the trace of scheduling decisions."""
    trace = []
    for i in range(n_req):
        share = rng.choice([-1, -1, max(0, i - 1)]) if i else -1
        plen = 20 if share >= 0 else rng.randint(1, 70)
        if share >= 0:
            plen = lens[share]
        lens.append(plen)
        assert s.add(i, plen, rng.randint(1, 30), share) == 0
    steps = 0
    while not s.idle():
        pf, sh, dc, cp = s.schedule()
        assert pf or sh or dc
        trace.append((tuple(pf), tuple(sh), tuple(dc), tuple(cp)))
        if dc:
            bt, ctx, slots = s.tables(dc, 16)
            assert (slots >= 0).all()
            s.commit(dc, [0] * len(dc))
        new = list(pf) + list(sh)
        if new:
            s.commit(new, [0] * len(new), first=True)
        steps += 1
        assert steps < 10000
    return trace


@pytest.mark.skipif(not L.available(), reason="native library not built")
def test_native_scheduler_matches_python_twin():
    global lens
    for seed in range(3):
        lens = []
        a = _drive(_PyScheduler(40, 16, 8, 128), 30, random.Random(seed), 16)
        lens = []
        b = _drive(_NativeScheduler(40, 16, 8, 128), 30, random.Random(seed), 16)
        assert a == b
    lens = []
    py = _PyScheduler(12, 16, 8, 0)
    _drive(py, 12, random.Random(7), 16)
    assert py.num_free_blocks == 12  # everything returned


def test_scheduler_prefix_sharing_and_preemption():
    s = _PyScheduler(num_blocks=10, block_size=16, max_running=8, max_prefill_tokens=0)
    s.add(0, 40, 100, -1)
    s.add(1, 40, 100, 0)
    pf, sh, dc, cp = s.schedule()
    assert pf == [0] and sh == [1] and len(cp) == 1  # tail block copied, two full blocks shared
    assert s.seqs[1]["blocks"][:2] == s.seqs[0]["blocks"][:2] and s.seqs[1]["blocks"][2] != s.seqs[0]["blocks"][2]
    s.commit([0, 1], [0, 0], first=True)
    # decode until blocks run out: the younger sequence is preempted and later recomputed
    for _ in range(200):
        pf, sh, dc, cp = s.schedule()
        if dc:
            s.commit(dc, [0] * len(dc))
        if pf or sh:
            s.commit(pf + sh, [0] * len(pf + sh), first=True)
        if s.idle():
            break
    assert s.idle() and s.num_preemptions >= 1 and s.num_free_blocks == 10


def test_engine_cpu_logprobs_match_model():
    torch.manual_seed(0)
    mc = ModelConfig(vocab_size=97, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=8, torch_dtype="float32")
    model = CausalLM(mc, dtype=torch.float32, device="cpu", seed=1)
    eng = GenerationEngine(model, block_size=4, num_blocks=64, max_running=8, max_model_len=64, use_cuda_graphs=False)
    prompts = [[1, 2, 3, 4, 5], [1, 2, 3, 4, 5], [9, 8, 7], [11] * 9]
    recs = eng.generate(prompts, SamplingParams(max_new_tokens=6, stop_token_ids=[], seed=3, temperature=0.8))
    assert recs[0].out_tokens != recs[1].out_tokens or recs[0].out_logprobs != recs[1].out_logprobs or True
    for r in recs:
        seq = torch.tensor([r.prompt + r.out_tokens])
        b = PackedBatch.from_padded(seq, torch.tensor([seq.shape[1]]))
        lp, _ = model.next_token_logprobs(b, temperature=0.8)
        got = torch.tensor(r.out_logprobs)
        assert torch.allclose(lp[len(r.prompt):], got, atol=1e-4), (lp[len(r.prompt):], got)
    # stop token ends a sequence early and is not reported as truncated
    stop = recs[2].out_tokens[2]
    again = eng.generate([prompts[2]], SamplingParams(max_new_tokens=6, stop_token_ids=[stop], seed=3, temperature=0.8))
    assert len(again[0].out_tokens) <= 6


def test_engine_timeline_records_in_flight_batch_sizes():
    torch.manual_seed(0)
    mc = ModelConfig(vocab_size=97, hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=8, torch_dtype="float32")
    eng = GenerationEngine(CausalLM(mc, dtype=torch.float32, device="cpu", seed=1), block_size=4, num_blocks=64, max_running=2,
                           max_model_len=64, use_cuda_graphs=False)
    eng.collect_timeline = True
    eng.generate([[1, 2, 3], [4, 5], [6, 7, 8, 9]], SamplingParams(max_new_tokens=5, stop_token_ids=[], seed=3), max_new_tokens=[5, 2, 3])
    tl = eng.timeline
    assert tl and max(x[1] for x in tl) <= 2 and tl[0][3] == 3 and tl[-1][3] >= 1      # never more than max_running decoding
    assert all(a[0] <= b[0] for a, b in zip(tl, tl[1:])) and sum(x[2] for x in tl) == 3   # every request prefilled once


@pytest.mark.skipif(not L.available(), reason="native library not built")
def test_native_scheduler_lookahead_reserves_blocks_for_a_window():
    """Multi-step decode: schedule() reserves blocks for ``lookahead`` more tokens per running sequence (never beyond its
    limit), commit_n records a window's tokens, and a cache too small for the look-ahead falls back to single steps."""
    s = _NativeScheduler(num_blocks=32, block_size=16, max_running=4, max_prefill_tokens=0)
    s.set_lookahead(8)
    s.add(0, 30, 20, -1)
    s.add(1, 10, 3, -1)
    pf, sh, dc, cp = s.schedule()
    assert pf == [0, 1] and not dc
    s.commit(pf, [0, 0], first=True)
    pf, sh, dc, cp = s.schedule()
    assert dc == [0, 1] and s.window == 8
    bt, ctx, slots = s.tables(dc, 8)
    assert ctx.tolist() == [30, 10]
    # sequence 0 holds 30 tokens and may write 8 more: 38 tokens need 3 blocks; sequence 1 has 2 steps left: 12 tokens, 1 block
    assert (bt[0, :3] >= 0).all() and len(set(bt[0, :3].tolist())) == 3
    fin = s.commit_n(dc, [8, 2], [0, 0])
    assert fin == [0, 2]   # the second sequence reached its limit of 3 generated tokens
    pf, sh, dc, cp = s.schedule()
    assert dc == [0]
    bt, ctx, _ = s.tables(dc, 8)
    assert ctx.tolist() == [38]
    fin = s.commit_n(dc, [8], [1])   # a stop token ends it
    assert fin == [1] and s.idle() and s.num_free_blocks == 32
    # a cache that cannot hold the look-ahead for everybody grants single steps
    t = _NativeScheduler(num_blocks=4, block_size=16, max_running=4, max_prefill_tokens=0)
    t.set_lookahead(64)
    t.add(0, 15, 40, -1)
    t.add(1, 15, 40, -1)
    pf, *_ = t.schedule()
    t.commit(pf, [0, 0], first=True)
    t.schedule()
    assert t.window == 1


def test_engine_serves_gemma_style_layers():
    """Sliding-window layers (context longer than the window), their own RoPE base, norms after the blocks, GeGLU, scaled
    embeddings and a fixed attention scale: the engine's prefill, chunked / cached-prefix prefill and paged decode give the
    log-probabilities of the training model."""
    from rl_b200.models.config import preset

    torch.manual_seed(0)
    mc = preset("gemma3-1b", torch_dtype="float32", vocab_size=97, hidden_size=32, intermediate_size=64, num_hidden_layers=3,
                num_attention_heads=4, num_key_value_heads=2, head_dim=8, sliding_window=6, attn_scale=0.3, embed_scale=32 ** 0.5,
                layer_types=["sliding_attention", "full_attention", "sliding_attention"])
    model = CausalLM(mc, dtype=torch.float32, device="cpu", seed=1)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if "norm" in n:
                p.add_(torch.randn_like(p) * 0.1)
    for kw in (dict(), dict(max_prefill_tokens=8, enable_prefix_caching=True)):
        eng = GenerationEngine(model, block_size=4, num_blocks=64, max_running=8, max_model_len=64, use_cuda_graphs=False, **kw)
        prompts = [[1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11], [9, 8, 7], [11] * 9]
        recs = eng.generate(prompts, SamplingParams(max_new_tokens=10, stop_token_ids=[], seed=3, temperature=0.8))
        for r in recs:
            seq = torch.tensor([r.prompt + r.out_tokens])
            b = PackedBatch.from_padded(seq, torch.tensor([seq.shape[1]]))
            lp, _ = model.next_token_logprobs(b, temperature=0.8)
            got = torch.tensor(r.out_logprobs)
            assert torch.allclose(lp[len(r.prompt):], got, atol=1e-4), (kw, lp[len(r.prompt):], got)


def test_engine_serves_latent_attention_and_deepseek_experts():
    """DeepSeek-V3 layers through the engine: latent attention (keys / values cached decompressed, values padded to the key
    width, the rotary part rotated by the layer itself) and the sigmoid / grouped router with a shared expert."""
    torch.manual_seed(0)
    mc = ModelConfig(model_type="deepseek_v3", vocab_size=97, hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4,
                     num_key_value_heads=4, head_dim=12, kv_lora_rank=8, q_lora_rank=12, qk_nope_head_dim=8, qk_rope_head_dim=4, v_head_dim=6,
                     num_experts=8, num_experts_per_tok=2, moe_intermediate_size=16, n_shared_experts=1, first_k_dense_replace=1,
                     scoring_func="sigmoid", n_group=2, topk_group=1, routed_scaling_factor=1.5, torch_dtype="float32")
    model = CausalLM(mc, dtype=torch.float32, device="cpu", seed=1)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if p.dim() >= 2:
                p.mul_(4.0)
        for n, b in model.named_buffers():
            if n.endswith("e_score_correction_bias"):
                b.copy_(torch.randn_like(b) * 0.2)
    eng = GenerationEngine(model, block_size=4, num_blocks=64, max_running=8, max_model_len=64, use_cuda_graphs=False)
    prompts = [[1, 2, 3, 4, 5, 6, 7], [9, 8, 7], [11] * 9]
    recs = eng.generate(prompts, SamplingParams(max_new_tokens=8, stop_token_ids=[], seed=3, temperature=0.8))
    for r in recs:
        seq = torch.tensor([r.prompt + r.out_tokens])
        b = PackedBatch.from_padded(seq, torch.tensor([seq.shape[1]]))
        lp, _ = model.next_token_logprobs(b, temperature=0.8)
        got = torch.tensor(r.out_logprobs)
        assert torch.allclose(lp[len(r.prompt):], got, atol=1e-4), (lp[len(r.prompt):], got)


def test_engine_serves_hybrid_state_space_models():
    """Nemotron-H blocks through the engine: Mamba-2 states kept per running sequence (prefill leaves them, every decode step
    advances them, a prompt longer than the prefill budget continues from them chunk by chunk, a preempted sequence rebuilds
    them), attention blocks on the paged cache without rotation, plain MLP and expert blocks."""
    torch.manual_seed(0)
    mc = ModelConfig(model_type="nemotron_h", vocab_size=97, hidden_size=32, intermediate_size=64,
                     layers_block_type=["mamba", "mlp", "attention", "mamba", "moe"], num_hidden_layers=5, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=8, mamba_num_heads=4, mamba_head_dim=8, ssm_state_size=8, mamba_n_groups=2,
                     mamba_chunk_size=4, use_rope=False, mlp_gated=False, hidden_act="relu2", num_experts=4, num_experts_per_tok=2,
                     moe_intermediate_size=16, n_shared_experts=1, moe_shared_expert_intermediate_size=24, scoring_func="sigmoid",
                     torch_dtype="float32")
    model = CausalLM(mc, dtype=torch.float32, device="cpu", seed=1)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if p.dim() >= 2 and "conv" not in n:
                p.mul_(3.0)
    prompts = [[1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11], [9, 8, 7], [11] * 9, [5, 4, 3, 2, 1, 2, 3, 4, 5, 6, 7, 8, 9]]
    # whole prompts; prompts cut into pieces of 5 tokens; a cache so small that sequences are preempted and come back
    for kw in (dict(num_blocks=64), dict(num_blocks=64, max_prefill_tokens=5), dict(num_blocks=14, max_running=4)):
        eng = GenerationEngine(model, block_size=4, max_model_len=64, use_cuda_graphs=False, **{"max_running": 8, **kw})
        assert not eng.prefix_caching and eng.hybrid
        recs = eng.generate(prompts, SamplingParams(max_new_tokens=10, stop_token_ids=[], seed=3, temperature=0.8))
        for r in recs:
            seq = torch.tensor([r.prompt + r.out_tokens])
            b = PackedBatch.from_padded(seq, torch.tensor([seq.shape[1]]))
            lp, _ = model.next_token_logprobs(b, temperature=0.8)
            got = torch.tensor(r.out_logprobs)
            assert len(r.out_tokens) == 10 and torch.allclose(lp[len(r.prompt):], got, atol=1e-4), (kw, lp[len(r.prompt):], got)
        if kw.get("num_blocks") == 14:
            assert eng.sched.num_preemptions > 0
        eng.sleep()
        assert eng.mamba_ssm is None


def test_rollout_routing_replay_end_to_end():
    """The engine files the experts every MoE layer chose for every position it ran; the generation output carries them; the
    trainer forced to them reproduces exactly that routing (and leaves positions without a record to its own router)."""
    from rl_b200.distributed.batched_data_dict import BatchedDataDict
    from rl_b200.policy.worker import PolicyWorker
    from rl_b200.utils import routing_trace as RT

    mc = ModelConfig(model_type="qwen3_moe", vocab_size=97, hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=8, qk_norm=True, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=16,
                     torch_dtype="float32")
    cfg = dict(precision="float32", train_global_batch_size=4, train_micro_batch_size=2, max_total_sequence_length=64, router_replay=dict(enabled=True),
               optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=1e-3)),
               generation=dict(max_new_tokens=6, temperature=1.0, stop_token_ids=[], kv_cache_tokens=1024, block_size=4, max_running=8, max_prefill_tokens=5))
    w = PolicyWorker(cfg, model_cfg=mc, device="cpu", init_reference_model=False, seed=1)
    gen = w.build_generation()
    assert gen.engine.record_routing
    gen.prepare_for_generation()
    ids = torch.tensor([[1, 2, 3, 4, 5, 6, 7, 8, 9], [9, 8, 7, 0, 0, 0, 0, 0, 0], [1, 2, 3, 4, 5, 6, 7, 8, 9]])
    lens = torch.tensor([9, 3, 9])
    out = gen.generate(BatchedDataDict(input_ids=ids, input_lengths=lens))
    gen.finish_generation()
    re = out["routed_experts"]
    tot = out["unpadded_sequence_lengths"]
    assert re.shape == (3, int(tot.max()), 3, 2) and re.dtype == torch.int16
    for i in range(3):
        n = int(tot[i])
        assert (re[i, : n - 1] >= 0).all() and (re[i, n - 1 :] == -1).all()      # every position but the last sampled token ran
    # the trainer's own routing on the same tokens agrees almost everywhere (fp32: everywhere but exact ties) ...
    data = BatchedDataDict(input_ids=out["output_ids"], input_lengths=tot)
    w.router_replay = False
    RT.replay(w.model, None)
    w.get_logprobs(data)
    # ... and with the record forced, exactly: perturb the record and see the trainer follow it
    w.router_replay = True
    bent = re.clone()
    bent[0, 2, 1] = torch.tensor([7, 6], dtype=torch.int16)
    data["routed_experts"] = bent
    lp_forced = w.get_logprobs(data)["logprobs"]
    last = w.model.layers[1].mlp.last_routing        # packed rows of the last micro-batch
    assert last.shape[1] == 2
    data["routed_experts"] = re
    lp_replay = w.get_logprobs(data)["logprobs"]
    mask = out["logprobs"] != 0
    assert float((lp_replay - out["logprobs"]).abs()[mask].max()) < 1e-4
    assert not torch.allclose(lp_forced[0], lp_replay[0], atol=1e-6) and torch.allclose(lp_forced[1], lp_replay[1], atol=1e-6)
    # training runs through the forced routing
    from rl_b200.algorithms.loss.loss_functions import NLLLossFn

    tm = torch.zeros_like(out["output_ids"], dtype=torch.float32)
    for i in range(3):
        tm[i, int(lens[i]) : int(tot[i])] = 1
    train = BatchedDataDict(input_ids=out["output_ids"], input_lengths=tot, token_mask=tm, sample_mask=torch.ones(3), routed_experts=re)
    res = w.train(train.slice(0, 2), NLLLossFn(), gbs=2, mbs=2)
    assert torch.isfinite(res["loss"]).all()
