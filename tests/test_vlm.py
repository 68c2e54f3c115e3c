"""Vision-language path: packed image tensors, patch helpers, the VLM's embedding splice, SFT and GRPO on synthetic images."""

import torch

from rl_b200.algorithms import grpo, sft
from rl_b200.algorithms.loss.loss_functions import NLLLossFn
from rl_b200.data.collate import rl_collate_fn, sft_collate_fn
from rl_b200.data.datasets.vlm import ProcessedVLMDataset, SyntheticColourDataset
from rl_b200.data.multimodal_utils import PackedTensor, content_key, expand_image_tokens, patchify, unpatchify
from rl_b200.data.tokenizers import ByteTokenizer
from rl_b200.environments.vlm_environment import VLMEnvironment, extract_answer
from rl_b200.models.config import ModelConfig

IMG_TOK = 511


def _mc():
    return ModelConfig(vocab_size=512, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                       head_dim=8, torch_dtype="float32", image_token_id=IMG_TOK,
                       vision=dict(patch_size=4, channels=3, hidden_size=16, intermediate_size=32, num_layers=1, num_heads=2, max_patches=64))


def test_packed_tensor_and_patch_helpers():
    img = torch.rand(3, 8, 12)
    p = patchify(img, 4)
    assert p.shape == (6, 48) and torch.equal(unpatchify(p, 3, 8, 12, 4), img)
    assert torch.equal(p[1], img[:, 0:4, 4:8].reshape(-1))
    pt = PackedTensor([p, None, p[:2]])
    assert pt.sizes() == [6, 0, 2] and pt.as_tensor().shape == (8, 48) and isinstance(pt[0:2], PackedTensor)
    assert PackedTensor.concat([pt, pt.select([2])]).sizes() == [6, 0, 2, 2] and PackedTensor([None]).as_tensor() is None
    assert expand_image_tokens([1, 9, 2, 9], 9, [2, 3]) == [1, 9, 9, 2, 9, 9, 9]
    assert content_key(p) == content_key(p.clone()) != content_key(p + 1)
    assert extract_answer("so <answer> Red </answer>") == "Red" and extract_answer("x \\boxed{blue}") == "blue"
    env = VLMEnvironment({})
    out = env.step([[{"role": "assistant", "content": "It is red."}], [{"role": "assistant", "content": "reddish"}]],
                   [{"ground_truth": "red"}, {"ground_truth": "red"}])
    assert out.rewards.tolist() == [1.0, 0.0]


def test_processor_collate_and_model_splice():
    tok = ByteTokenizer(512)
    raw = SyntheticColourDataset(8, image_size=8, seed=0)
    ds = ProcessedVLMDataset(raw, tok, patch=4, image_token_id=IMG_TOK, with_answer=True)
    d = ds[0]
    user = d["message_log"][0]
    assert int((user["token_ids"] == IMG_TOK).sum()) == 4 == user["pixel_patches"].shape[0] and user["image_sizes"] == [4]
    batch = sft_collate_fn([ds[i] for i in range(4)], pad_token_id=tok.pad_token_id)
    assert len(batch["pixel_patches"]) == 4 and batch["image_sizes"] == [[4]] * 4 and batch["token_mask"].sum() > 0
    half = batch.slice(2, 4)
    assert len(half["pixel_patches"]) == 2 and torch.equal(half["pixel_patches"][0], batch["pixel_patches"][2])
    from rl_b200.policy.worker import PolicyWorker

    w = PolicyWorker(dict(precision="float32", train_global_batch_size=4, train_micro_batch_size=2, logprob_batch_size=2,
                          max_total_sequence_length=96, optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=1e-3))),
                     model_cfg=_mc(), init_reference_model=False, seed=0)
    lp = w.get_logprobs(batch)["logprobs"]
    other = batch.slice(0, 4)
    other["pixel_patches"] = PackedTensor([t.flip(0) * 0.5 for t in batch["pixel_patches"]])
    lp2 = w.get_logprobs(other)["logprobs"]
    first_img = int((batch["input_ids"][0] == IMG_TOK).nonzero()[0])
    assert torch.equal(lp[:, : first_img + 1], lp2[:, : first_img + 1])           # tokens before the image do not see it
    assert (lp[:, first_img + 1 :] - lp2[:, first_img + 1 :]).abs().max() > 1e-5   # tokens after it do


def test_vlm_sft_learns_the_colours(tmp_path):
    tok = ByteTokenizer(512)
    train = ProcessedVLMDataset(SyntheticColourDataset(128, image_size=8, colours=["red", "blue"], seed=0), tok, 4, IMG_TOK, True)
    val = ProcessedVLMDataset(SyntheticColourDataset(16, image_size=8, colours=["red", "blue"], seed=1), tok, 4, IMG_TOK, True)
    cfg = {"sft": dict(max_num_steps=48, max_num_epochs=6, val_period=0, seed=0),
           "policy": dict(precision="float32", train_global_batch_size=16, train_micro_batch_size=8, logprob_batch_size=8, max_total_sequence_length=96,
                          max_grad_norm=1.0, optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=5e-3, weight_decay=0.0))),
           "logger": dict(log_dir=str(tmp_path)), "checkpointing": dict(enabled=False), "data": dict(shuffle=True)}
    policy, loader, val_loader, loss_fn, logger, ck, ss, cfg = sft.setup_sft(cfg, tok, train, val, model_cfg=_mc())
    hist = []
    sft.sft_train(policy, loader, val_loader, tok, loss_fn, logger, ck, ss, cfg, step_callback=lambda s, m: hist.append(m["train"]["loss"]))
    assert hist[-1] < 0.5 * hist[0]
    # the answer token after the generation prompt depends on the image: per-sample NLL of the right colour beats the wrong one
    batch = sft_collate_fn([val[i] for i in range(16)], pad_token_id=tok.pad_token_id)
    right = policy.get_logprobs(batch)["logprobs"]
    wrong = batch.slice(0, 16)
    wrong["pixel_patches"] = PackedTensor([batch["pixel_patches"][(i + 1) % 16] if val.raw[i]["answer"] != val.raw[(i + 1) % 16]["answer"]
                                           else batch["pixel_patches"][i] for i in range(16)])
    lw = policy.get_logprobs(wrong)["logprobs"]
    m = batch["token_mask"]
    assert (right * m).sum() > (lw * m).sum() + 1.0


def test_vlm_grpo_steps_with_engine_logprobs_matching(tmp_path):
    tok = ByteTokenizer(512)
    ds = ProcessedVLMDataset(SyntheticColourDataset(64, image_size=8, seed=0), tok, 4, IMG_TOK, False)
    env = {"vlm": VLMEnvironment({})}
    cfg = {"grpo": dict(num_prompts_per_step=4, num_generations_per_prompt=4, max_num_steps=2, val_period=0, seed=0),
           "loss_fn": dict(reference_policy_kl_penalty=0.0),
           "policy": dict(precision="float32", train_global_batch_size=16, train_micro_batch_size=8, logprob_batch_size=8, max_total_sequence_length=96,
                          max_grad_norm=1.0, optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=1e-3, weight_decay=0.0)),
                          generation=dict(max_new_tokens=6, temperature=1.0, stop_token_ids=[], kv_cache_tokens=4096, block_size=8, max_running=32)),
           "logger": dict(log_dir=str(tmp_path)), "checkpointing": dict(enabled=False)}
    policy, gen, loader, _, loss_fn, logger, ck, ss, cfg = grpo.setup(cfg, tok, ds, None, env, model_cfg=_mc())
    hist = []
    grpo.grpo_train(policy, gen, loader, None, tok, loss_fn, env, env, logger, ck, ss, cfg, step_callback=lambda s, m: hist.append(m["train"]))
    assert len(hist) == 2
    assert all(abs(h["token_mult_prob_error"] - 1.0) < 1e-2 for h in hist)   # same images on both sides (the engine never samples the placeholder token: 1/512 of the mass here)


def test_vlm_checkpoint_round_trip(tmp_path):
    from rl_b200.models import hf_io
    from rl_b200.models.transformer import build_model

    m = build_model(_mc(), dtype=torch.float32, seed=3)
    hf_io.save_pretrained(m, str(tmp_path))
    m2 = hf_io.load_pretrained(str(tmp_path), dtype=torch.float32)
    a, b = dict(m.named_parameters()), dict(m2.named_parameters())
    assert type(m2).__name__ == "VLMCausalLM" and set(a) == set(b) and all(torch.equal(a[k], b[k]) for k in a)
    assert any(k.startswith("visual.") for k in a) and m2.cfg.image_token_id == IMG_TOK
