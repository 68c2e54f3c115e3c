"""NVFP4 / FP8 quantisation math and quantisation-aware training through the worker and the engine."""

import json
import os

import pytest
import torch

from rl_b200.models.config import preset


def test_nvfp4_rounding_pack_and_scales():
    from rl_b200.ops.nvfp4 import dequantize_nvfp4, fake_quant, quantize_nvfp4

    # one block whose scale is exactly 1: the grid and its ties (to the even mantissa)
    x = torch.tensor([[0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 0.24, 0.76, 5.1, -0.75, 0.0, -6.0, 2.9, -0.3]])
    assert fake_quant(x).tolist() == [[0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0, 0.0, 1.0, 6.0, -1.0, 0.0, -6.0, 3.0, -0.5]]
    torch.manual_seed(0)
    w = torch.randn(8, 64) * torch.logspace(-2, 1, 8)[:, None]
    packed, sb, s2 = quantize_nvfp4(w)
    assert packed.shape == (8, 32) and packed.dtype == torch.uint8 and sb.shape == (8, 4) and sb.dtype == torch.float8_e4m3fn
    assert float(s2) == pytest.approx(float(w.abs().max()) / (6 * 448), rel=1e-6)
    d = dequantize_nvfp4(packed, sb, s2)
    assert torch.equal(d, fake_quant(w))                    # the packed form carries exactly the fake-quantised values
    assert torch.equal(fake_quant(d), d)                    # quantising a representable tensor changes nothing
    # relative error per block is bounded by the coarsest step of the grid (2 of 6) over two, plus the scale's rounding
    blk = w.reshape(8, 4, 16)
    err = (d.reshape(8, 4, 16) - blk).abs().amax(-1) / blk.abs().amax(-1)
    assert float(err.max()) < 0.2
    assert float(fake_quant(torch.zeros(2, 16)).abs().max()) == 0.0
    # straight-through gradient; values beyond a static range get none
    xx = (torch.randn(4, 32) * 2).requires_grad_()
    fake_quant(xx).sum().backward()
    assert torch.equal(xx.grad, torch.ones_like(xx))
    xx.grad = None
    fake_quant(xx, "nvfp4", torch.tensor(1.0)).sum().backward()
    assert torch.equal(xx.grad, (xx.abs() <= 1.0).float())
    f8 = fake_quant(w, "fp8")
    assert float(((f8 - w).abs() / w.abs().clamp(min=float(w.abs().max()) / 448)).max()) < 0.07


def test_recipe_resolution_and_attachment(tmp_path):
    from rl_b200.models.transformer import build_model
    from rl_b200.policy import qat

    m = build_model(preset("tiny-llama-oracle", torch_dtype="float32"), dtype=torch.float32)
    q = qat.attach(m, qat.resolve_quant_cfg("NVFP4_DEFAULT_CFG"))
    assert "lm_head" not in q and "layers.0.self_attn.qkv_proj" in q and "layers.0.mlp.down_proj" in q and "embed_tokens" not in q
    assert q["layers.0.self_attn.qkv_proj"].weight == "nvfp4" and q["layers.0.self_attn.qkv_proj"].input == "nvfp4"
    assert q["layers.0.self_attn.qkv_proj"].pieces == [(0, 256), (256, 512), (512, 768)]      # q / k / v keep their own tensor scales
    qat.detach(m)
    q = qat.attach(m, qat.resolve_quant_cfg("nvfp4_a16"))
    assert all(v.input is None and v.weight == "nvfp4" for v in q.values())
    qat.detach(m)
    # a recipe file in the ModelOpt layout: ordered wildcards, later entries win
    y = tmp_path / "mlp_only.yaml"
    y.write_text("""
quantize:
  algorithm: max
  quant_cfg:
    - {quantizer_name: '*', enable: false}
    - quantizer_name: '*mlp*weight_quantizer'
      enable: true
      cfg: {num_bits: e2m1, block_sizes: {-1: 16, type: dynamic, scale_bits: e4m3}}
    - {quantizer_name: '*layers.3.*', enable: false}
""")
    q = qat.attach(m, qat.resolve_quant_cfg(str(y)))
    assert sorted(q) == sorted(f"layers.{i}.mlp.{n}" for i in range(3) for n in ("gate_up_proj", "down_proj"))
    qat.detach(m)
    bad = tmp_path / "bad.yaml"
    bad.write_text("quantize: {quant_cfg: [{quantizer_name: '*q_proj.weight_quantizer', enable: true}]}")
    with pytest.raises(ValueError, match="fused"):
        qat.attach(m, qat.resolve_quant_cfg(str(bad)))      # q without k / v: they share one fused parameter here
    with pytest.raises(ValueError, match="unknown quant_cfg"):
        qat.resolve_quant_cfg("NOT_A_RECIPE")
    # experts of a mixture model
    moe = build_model(preset("tiny-nemotron-h", torch_dtype="float32"), dtype=torch.float32)
    q = qat.attach(moe, qat.resolve_quant_cfg("NVFP4_EXPERTS"))
    assert sorted(q) == ["layers.5.mlp.down_proj", "layers.5.mlp.up_proj"]


def _data():
    from rl_b200.distributed.batched_data_dict import BatchedDataDict

    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 2048, (8, 20), generator=g)
    lens = torch.tensor([20, 13, 17, 20, 9, 20, 15, 11])
    return BatchedDataDict(input_ids=ids, input_lengths=lens, token_mask=(torch.arange(20)[None] < lens[:, None]).float(), sample_mask=torch.ones(8))


def _cfg(**over):
    c = dict(precision="float32", train_global_batch_size=8, train_micro_batch_size=4, max_total_sequence_length=64, max_grad_norm=1.0,
             optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=3e-3)),
             generation=dict(max_new_tokens=6, temperature=1.0, stop_token_ids=[], kv_cache_tokens=2048, block_size=16, max_running=8))
    c.update(over)
    return c


@pytest.mark.parametrize("recipe,model", [("NVFP4_DEFAULT_CFG", "tiny-llama-oracle"), ("NVFP4_EXPERTS", "tiny-nemotron-h")])
def test_quantisation_aware_training_through_worker_and_engine(tmp_path, recipe, model):
    """The quantised policy is what trains, scores and generates: log-probabilities differ from the bf16 / fp32 model's, equal
    those of a model whose weights were replaced by their quantised values (weights-only recipe), the engine's sampled
    log-probabilities agree with the trainer's, training lowers the loss, the export holds the packed tensors."""
    from rl_b200.algorithms.loss.loss_functions import NLLLossFn
    from rl_b200.policy import qat
    from rl_b200.policy.worker import PolicyWorker

    mc = preset(model, torch_dtype="float32")
    data = _data()
    plain = PolicyWorker(_cfg(), model_cfg=mc, device="cpu", init_reference_model=False, seed=5)
    w = PolicyWorker(_cfg(quant_cfg=recipe, quant_calib_size=8, quant_batch_size=4, quant_sequence_length=16), model_cfg=mc, device="cpu",
                     init_reference_model=True, seed=5)
    assert w.quantizers and all(q.input_amax is not None for q in w.quantizers.values() if q.input)
    lp_q, lp_p = w.get_logprobs(data)["logprobs"], plain.get_logprobs(data)["logprobs"]
    assert not torch.allclose(lp_q, lp_p, atol=1e-4) and (lp_q - lp_p).abs().max() < 1.0
    # the switch restores the unquantised model
    qat.QatState.enabled = False
    try:
        assert torch.allclose(w.get_logprobs(data)["logprobs"], lp_p, atol=1e-6)
    finally:
        qat.QatState.enabled = True
    # engine and trainer see the same quantised policy
    gen = w.build_generation()
    gen.prepare_for_generation()
    out = gen.generate(data)
    gen.finish_generation()
    from rl_b200.distributed.batched_data_dict import BatchedDataDict

    lp = w.get_logprobs(BatchedDataDict(input_ids=out["output_ids"], input_lengths=out["unpadded_sequence_lengths"]))["logprobs"]
    mask = out["logprobs"] != 0
    assert float((lp - out["logprobs"]).abs()[mask].max()) < 1e-3
    losses = [float(w.train(data, NLLLossFn())["loss"][0]) for _ in range(4)]
    assert losses[-1] < losses[0]
    assert not torch.allclose(w.get_logprobs(data)["logprobs"], lp_q, atol=1e-4)          # cached quantised weights were refreshed
    assert torch.allclose(w.get_reference_policy_logprobs(data)["reference_logprobs"], lp_q, atol=1e-5)   # the reference is quantised too
    meta = w.export_quantized(str(tmp_path / "q"))
    assert meta["quantization"]["quant_algo"] == "NVFP4" and meta["quantization"]["group_size"] == 16
    from safetensors.torch import load_file

    sd = load_file(str(tmp_path / "q" / "model.safetensors"))
    name = "model.layers.0.mlp.down_proj" if model == "tiny-llama-oracle" else "model.layers.5.mixer.experts.0.down_proj"
    assert sd[name + ".weight"].dtype == torch.uint8 and sd[name + ".weight_scale"].dtype == torch.float8_e4m3fn
    assert sd[name + ".weight_scale_2"].numel() == 1 and float(sd[name + ".input_scale"]) > 0
    assert "lm_head" in meta["quantization"]["exclude_modules"] and sd["lm_head.weight"].dtype == torch.float32
    assert json.load(open(tmp_path / "q" / "hf_quant_config.json"))["producer"]["name"] == "rl_b200"
    # calibrated ranges travel with checkpoints
    path = str(tmp_path / "step_1" / "policy" / "weights")
    w.save_checkpoint(path)
    w2 = PolicyWorker(_cfg(quant_cfg=recipe), model_cfg=mc, device="cpu", init_reference_model=False, seed=9)
    assert all(q.input_amax is None for q in w2.quantizers.values())
    w2.load_checkpoint(path)
    assert torch.allclose(w2.get_logprobs(data)["logprobs"], w.get_logprobs(data)["logprobs"], atol=1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_native_nvfp4_kernels_match_the_pytorch_statement(dtype, monkeypatch):
    """The streaming kernels produce the bits of the fp32 PyTorch statement: fake quantisation of a matrix (dynamic and static
    range), of stacked expert matrices with one range each, and the packed form with its block scales."""
    from rl_b200.ops import lib as L
    from rl_b200.ops import nvfp4 as N

    assert L.available()
    torch.manual_seed(0)
    x = (torch.randn(300, 4096, device="cuda") * torch.logspace(-3, 2, 300, device="cuda")[:, None]).to(dtype)
    x[5, :32] = 0
    w3 = (torch.randn(6, 64, 256, device="cuda") * torch.logspace(-2, 1, 6, device="cuda")[:, None, None]).to(dtype)
    a3 = w3.abs().amax(dim=(-2, -1), keepdim=True)
    got = [N.fake_quant(x), N.fake_quant(x, "nvfp4", torch.tensor(1.5, device="cuda")), N.fake_quant(w3, "nvfp4", a3, clip=False)]
    packed, sb, s2 = N.quantize_nvfp4(x)
    assert L.Counters.launches > 0
    monkeypatch.setenv("RLB_FORCE_REFERENCE_OPS", "1")
    ref = [N.fake_quant(x), N.fake_quant(x, "nvfp4", torch.tensor(1.5, device="cuda")), N.fake_quant(w3, "nvfp4", a3, clip=False)]
    rp, rsb, rs2 = N.quantize_nvfp4(x)
    for g, r in zip(got, ref):
        assert torch.equal(g, r)
    assert torch.equal(packed, rp) and torch.equal(sb.view(torch.uint8), rsb.view(torch.uint8)) and float(s2) == float(rs2)
    assert torch.equal(N.dequantize_nvfp4(packed, sb, s2, dtype), got[0])
    assert L.check_status() == 0


def test_export_script_from_a_checkpoint(tmp_path):
    import sys

    from rl_b200.models.hf_io import save_pretrained
    from rl_b200.models.transformer import build_model

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    from examples.converters import export_quantized_to_hf as ex

    m = build_model(preset("tiny-llama-oracle", torch_dtype="float32"), dtype=torch.float32, seed=2)
    save_pretrained(m, str(tmp_path / "w"))
    meta = ex.main(["--ckpt", str(tmp_path / "w"), "--quant-cfg", f"{root}/examples/configs/quant/nvfp4_a16_mlp_only.yaml", "--out", str(tmp_path / "q"),
                    "--device", "cpu"])
    assert meta["quantization"]["quant_algo"] == "W4A16_NVFP4"
    from safetensors.torch import load_file

    from rl_b200.ops.nvfp4 import dequantize_nvfp4, fake_quant

    sd = load_file(str(tmp_path / "q" / "model.safetensors"))
    w = dict(m.named_parameters())["layers.1.mlp.down_proj"].detach()
    got = dequantize_nvfp4(sd["model.layers.1.mlp.down_proj.weight"], sd["model.layers.1.mlp.down_proj.weight_scale"],
                           sd["model.layers.1.mlp.down_proj.weight_scale_2"])
    assert torch.equal(got, fake_quant(w)) and "model.layers.1.mlp.down_proj.input_scale" not in sd
    assert sd["model.layers.1.self_attn.q_proj.weight"].dtype == torch.float32
