"""FP8 block-wise and MXFP8 quantisation: CPU oracle properties and the native kernels against the oracle."""

import pytest
import torch

from rl_b200.ops.quant import (FP8_MAX, dequantize_fp8_blockwise, dequantize_mxfp8, quantize_fp8_blockwise, quantize_fp8_blockwise_ref,
                               quantize_mxfp8, quantize_mxfp8_ref)


def _w(R, C, seed=0, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(R, C, generator=g) * torch.rand(R, 1, generator=g) * 3
    w[0, :5] = 0
    return w.to(torch.bfloat16).to(device)


@pytest.mark.parametrize("pow2", [False, True])
def test_blockwise_oracle_properties(pow2):
    w = _w(300, 200)  # ragged in both dimensions: 3 x 2 blocks
    q, ds = quantize_fp8_blockwise_ref(w, 128, pow2)
    assert q.shape == w.shape and q.dtype == torch.float8_e4m3fn and ds.shape == (3, 2)
    back = dequantize_fp8_blockwise(q, ds).float()
    rel = (back - w.float()).abs().max() / w.float().abs().max()
    assert rel < 0.07  # e4m3 has 3 mantissa bits: relative step 2^-4 at the top of a block's range
    # full blocks use the whole fp8 range: max |q| is 448 without pow2 scales, within a factor 2 with them
    qmax = q.float()[:128, :128].abs().max()
    assert qmax == FP8_MAX if not pow2 else FP8_MAX / 2 < qmax <= FP8_MAX
    if pow2:
        assert torch.all(torch.log2(ds) == torch.log2(ds).round())
    # the ragged corner block is padded with the last element, which takes part in its amax
    w2 = w.clone()
    w2[-1, -1] = 1000.0
    _, ds2 = quantize_fp8_blockwise_ref(w2, 128, pow2)
    assert ds2[2, 0] > ds[2, 0] and ds2[0, 1] > ds[0, 1] and ds2[0, 0] == ds[0, 0]


def test_mxfp8_oracle_properties():
    w = _w(64, 256, seed=1)
    q, e = quantize_mxfp8_ref(w)
    assert e.dtype == torch.uint8 and e.shape == (64, 8)
    assert q.float().abs().max() <= FP8_MAX
    back = dequantize_mxfp8(q, e).float()
    assert ((back - w.float()).abs() <= 0.0625 * w.float().abs().reshape(64, 8, 32).amax(-1).repeat_interleave(32, 1) + 1e-9).all()
    assert e[0, 0] != 0 and quantize_mxfp8_ref(torch.zeros(1, 32, dtype=torch.bfloat16))[1].item() == 0  # all-zero group -> byte 0


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(256, 384), (300, 200), (4096, 1536)])
@pytest.mark.parametrize("pow2", [False, True])
def test_native_blockwise_matches_oracle(native_lib, shape, pow2):
    w = _w(*shape, seed=2, device="cuda")
    q, ds = quantize_fp8_blockwise(w, pow2)
    qr, dsr = quantize_fp8_blockwise_ref(w, 128, pow2)
    torch.cuda.synchronize()
    assert torch.allclose(ds, dsr, rtol=1e-6, atol=0)
    diff = (q.float() - qr.float()).abs()
    # identical up to a one-code difference where x * scale lands on a rounding tie computed in a different order
    assert (diff > 0).float().mean() < 1e-3 and (diff <= q.float().abs() * 0.13 + 2 ** -9).all()
    assert torch.equal(dequantize_fp8_blockwise(q, ds), (q.float() * dsr.repeat_interleave(128, 0)[: shape[0]].repeat_interleave(128, 1)[:, : shape[1]]).to(torch.bfloat16))


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(64, 256), (2048, 768), (777, 2048)])
def test_native_mxfp8_matches_oracle(native_lib, shape):
    w = _w(*shape, seed=3, device="cuda")
    q, e = quantize_mxfp8(w)
    qr, er = quantize_mxfp8_ref(w)
    torch.cuda.synchronize()
    assert torch.equal(e, er)
    assert torch.equal(q.view(torch.uint8), qr.view(torch.uint8))
    assert torch.equal(dequantize_mxfp8(q, e), dequantize_mxfp8(qr.cpu(), er.cpu()).cuda())


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(64, 256), (200, 1024), (777, 2048)])
def test_native_mxfp8_blocked_scales_match_the_swizzled_oracle(native_lib, shape):
    from rl_b200.ops.quant import quantize_mxfp8_blocked, swizzle_mx_scales

    w = _w(*shape, seed=5, device="cuda")
    q, sb = quantize_mxfp8_blocked(w)
    qr, er = quantize_mxfp8(w)
    torch.cuda.synchronize()
    assert torch.equal(q.view(torch.uint8), qr.view(torch.uint8))
    assert torch.equal(sb, swizzle_mx_scales(er))


def test_swizzled_scale_layout():
    from rl_b200.ops.quant import swizzle_mx_scales

    R, G = 200, 8  # two row blocks (second ragged), two K blocks
    sc = (torch.arange(R * G) % 251).to(torch.uint8).view(R, G)
    sw = swizzle_mx_scales(sc)
    assert sw.shape == (2, 2, 512)
    for r, g in [(0, 0), (33, 5), (127, 7), (128, 0), (199, 3)]:
        blk, rr, kb, j = r // 128, r % 128, g // 4, g % 4
        assert sw[blk, kb, (rr % 32) * 16 + (rr // 32) * 4 + j] == sc[r, g]
    assert sw[1, 0, (72 % 32) * 16 + (72 // 32) * 4] == 0  # row 200 does not exist


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(128, 128, 128), (256, 384, 512), (200, 264, 1024), (1024, 2048, 768)])
def test_mxfp8_gemm_matches_dequantised_reference(native_lib, shape):
    from rl_b200.ops.lib import check_status
    from rl_b200.ops.quant import gemm_mxfp8, swizzle_mx_scales

    M, N, K = shape
    a = _w(M, K, seed=5, device="cuda")
    b = _w(N, K, seed=6, device="cuda")
    aq, asf = quantize_mxfp8(a)
    bq, bsf = quantize_mxfp8(b)
    c = gemm_mxfp8(aq, swizzle_mx_scales(asf), bq, swizzle_mx_scales(bsf))
    torch.cuda.synchronize()
    assert check_status() == 0
    ref = dequantize_mxfp8(aq, asf).float() @ dequantize_mxfp8(bq, bsf).float().t()
    err = (c.float() - ref).abs().max().item()
    assert err <= 1e-2 * ref.abs().max().item() + 1e-3, (err, ref.abs().max().item())


@pytest.mark.gpu
def test_mxfp8_training_linear_matches_quantised_statement(native_lib):
    """Forward, input gradient and weight gradient of the MXFP8 training linear on the block-scaled tensor-core GEMM against
    the CPU statement (operands rounded to e4m3 with one E8M0 scale per 32 elements along each GEMM's contraction)."""
    from rl_b200.ops import functional as F
    from rl_b200.ops.lib import check_status

    torch.manual_seed(0)
    M, K, N = 200, 256, 384          # the token count is not a multiple of 128: the weight-gradient GEMM pads it
    x = torch.randn(M, K).to(torch.bfloat16)
    w = (torch.randn(N, K) * 0.05).to(torch.bfloat16)
    dy = torch.randn(M, N).to(torch.bfloat16)
    F.Fp8Training.configure(dict(enabled=True, fp8_recipe="mxfp8"))
    try:
        outs = {}
        for dev in ("cpu", "cuda"):
            xd, wd = x.detach().clone().to(dev).requires_grad_(), w.detach().clone().to(dev).requires_grad_()
            y = F.linear(xd, wd)
            y.backward(dy.to(dev))
            outs[dev] = (y.detach().float().cpu(), xd.grad.float().cpu(), wd.grad.float().cpu())
        for a, b, name in zip(outs["cpu"], outs["cuda"], ("y", "dx", "dw")):
            assert (a - b).abs().max().item() <= 2e-2 * a.abs().max().item() + 1e-3, name
        assert check_status() == 0
    finally:
        F.Fp8Training.configure(None)


@pytest.mark.gpu
def test_quantising_refit_on_one_gpu_matches_copy_then_quantise(native_lib):
    """The refit pass that quantises on the way (one kernel: bf16 block -> amax -> e4m3 + de-scale + fp8-rounded bf16) against
    the bf16 re-shard copy followed by the block-128 quantiser."""
    from rl_b200.models.config import ModelConfig
    from rl_b200.models.transformer import build_model
    from rl_b200.ops import quant as Q
    from rl_b200.ops.lib import check_status
    from rl_b200.parallel.tensor import TP
    from rl_b200.refit.synchronizer import WeightSynchronizer

    mc = ModelConfig(model_type="qwen3", vocab_size=1024, hidden_size=256, intermediate_size=640, num_hidden_layers=2,
                     num_attention_heads=4, num_key_value_heads=2, head_dim=128, qk_norm=True, tie_word_embeddings=False)
    train = build_model(mc, device="cuda", dtype=torch.bfloat16, seed=3, tp=TP(None, 0, 1))
    ws = WeightSynchronizer(train, mc, 1)
    ws.sync_weights()
    want = {n: Q.quantize_fp8_blockwise(p.data) for n, p in ws.serving_model.named_parameters()
            if p.dim() == 2 and n.rsplit(".", 1)[-1] in ("qkv_proj", "o_proj", "gate_up_proj", "down_proj")}
    plain = {n: p.data.clone() for n, p in ws.serving_model.named_parameters()}
    ws.arena.zero_()
    ws.sync_weights_fp8()
    torch.cuda.synchronize()
    assert check_status() == 0 and len(ws._fp8_fused) == len(want) == 8
    for n, p in ws.serving_model.named_parameters():
        if n in want:
            _, q, sc = p._rlb_q
            assert torch.equal(q.view(torch.uint8), want[n][0].view(torch.uint8)) and torch.equal(sc, want[n][1]), n
            assert torch.equal(p.data, Q.dequantize_fp8_blockwise(q, sc)), n      # the bf16 arena holds the fp8-rounded weights
        else:
            assert torch.equal(p.data, plain[n]), n                                # norms, embeddings, head: plain copies
    ws.close()
