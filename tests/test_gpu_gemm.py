"""tcgen05 GEMM against an fp32 PyTorch matmul of the same bf16 operands, all three operand layouts,
ragged edges, accumulate / bias / fp32-output epilogues, and the fused lm_head log-prob epilogues."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel_err(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-6)


SHAPES = [(128, 256, 64), (256, 512, 128), (300, 264, 200), (1000, 1024, 4096), (4096, 4096, 1024), (64, 8, 8)]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("layout", ["kk", "k_mn", "mn_mn", "mn_k"])
def test_gemm_layouts(native_lib, M, N, K, layout):
    from rl_b200.ops import functional as F
    from rl_b200.ops.lib import check_status

    if layout != "kk" and (M % 8 or N % 8):
        pytest.skip("MN-major operands need 16-byte aligned rows")
    torch.manual_seed(0)
    dev = "cuda"
    a_mn = layout.startswith("mn")
    b_mn = layout.endswith("mn")
    a = torch.randn((K, M) if a_mn else (M, K), device=dev, dtype=torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device=dev, dtype=torch.bfloat16)
    ref = (a.t() if a_mn else a).float() @ (b if b_mn else b.t()).float()
    out = F.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    torch.cuda.synchronize()
    assert check_status() == 0
    assert _rel_err(out, ref) < 1e-2


def test_gemm_epilogues(native_lib):
    from rl_b200.ops import functional as F

    torch.manual_seed(1)
    M, N, K = 384, 520, 256
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda")
    ref = a.float() @ b.float().t()
    out32 = F.gemm(a, b, out_dtype=torch.float32)
    assert _rel_err(out32, ref) < 2e-3
    outb = F.gemm(a, b, bias=bias)
    assert _rel_err(outb, ref + bias) < 1e-2
    acc = torch.ones(M, N, device="cuda", dtype=torch.float32)
    F.gemm(a, b, out=acc, accumulate=True)
    assert _rel_err(acc, ref + 1) < 2e-3
    accb = torch.ones(M, N, device="cuda", dtype=torch.bfloat16)
    F.gemm(a, b, out=accb, accumulate=True)
    assert _rel_err(accb, ref + 1) < 1e-2
    # strided views (slices of wider buffers)
    wide_a = torch.randn(M, K + 64, device="cuda", dtype=torch.bfloat16)
    wide_o = torch.zeros(M, N + 24, device="cuda", dtype=torch.bfloat16)
    F.gemm(wide_a[:, 64:], b, out=wide_o[:, 24:])
    assert _rel_err(wide_o[:, 24:], wide_a[:, 64:].float() @ b.float().t()) < 1e-2
    assert wide_o[:, :24].abs().max().item() == 0


def test_linear_autograd(native_lib):
    from rl_b200.ops import functional as F

    torch.manual_seed(2)
    x = torch.randn(3, 100, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(512, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = F.linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    yr = xr @ wr.t()
    yr.backward(g.float())
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 1e-2
    assert _rel_err(w.grad, wr.grad) < 1e-2


@pytest.mark.parametrize("M,V,K", [(200, 1000, 128), (1024, 32000, 512), (77, 128256, 256)])
def test_lm_head_logprob(native_lib, M, V, K):
    from rl_b200.ops import functional as F
    from rl_b200.ops.lib import check_status

    torch.manual_seed(3)
    h = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    w = (torch.randn(V, K, device="cuda") * 0.2).to(torch.bfloat16).requires_grad_()
    tg = torch.randint(0, V, (M,), device="cuda")
    temp = 0.8
    logp, ent = F.lm_head_logprobs(h, w, tg, temperature=temp, want_entropy=True)
    hr = h.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    lr, er = F._lm_head_ref(hr, wr, tg, 1.0 / temp, True)
    assert check_status() == 0
    assert (logp - lr).abs().max().item() < 2e-2
    assert (ent - er).abs().max().item() < 2e-2
    cl = torch.randn(M, device="cuda")
    ce = torch.randn(M, device="cuda") * 0.1
    (logp * cl + ent * ce).sum().backward()
    (lr * cl + er * ce).sum().backward()
    assert _rel_err(h.grad, hr.grad) < 3e-2
    assert _rel_err(w.grad, wr.grad) < 3e-2


@pytest.mark.parametrize("M", [1, 7, 32, 64, 100, 128, 200, 256])
@pytest.mark.parametrize("N,K", [(4096, 4096), (6144, 4096), (4096, 14336), (1000, 512), (128256, 1024)])
def test_skinny_gemm(native_lib, M, N, K):
    """Decode-sized GEMM (operands swapped, cluster split-K) against fp32 matmul, with bias / residual / fp32 output."""
    from rl_b200.ops import functional as F
    from rl_b200.ops.lib import check_status

    torch.manual_seed(M + N)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    ref = x.float() @ w.float().t()
    y = F.gemm(x, w)
    torch.cuda.synchronize()
    assert check_status() == 0
    assert _rel_err(y, ref) < 1e-2
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda")
    y2 = F.gemm(x, w, bias=bias, residual=res, out_dtype=torch.float32)
    assert _rel_err(y2, ref + bias + res.float()) < 2e-3


def test_skinny_split_values(native_lib):
    from rl_b200.ops.lib import call, lib, ptr, status_word, stream_ptr

    x = torch.randn(64, 4096, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(4096, 4096, device="cuda") * 0.05).to(torch.bfloat16)
    ref = x.float() @ w.float().t()
    outs = []
    for split in (1, 2, 3, 4, 8):
        y = torch.empty(64, 4096, device="cuda", dtype=torch.bfloat16)
        call("rlb_gemm_skinny", ptr(x), ptr(w), ptr(y), 64, 4096, 4096, 4096, 4096, 4096, 0, None, None, 0, split,
             ptr(status_word()), stream_ptr())
        assert _rel_err(y, ref) < 1e-2, split
        outs.append(y)
    assert lib().rlb_gemm_skinny_split(4096, 4096) in (1, 2, 4, 8)


@pytest.mark.parametrize("M", [5, 64, 130])
def test_skinny_gemm_epilogue_fusions_match_fp32_reference(native_lib, M):
    """RMSNorm folded into two projections (producer writes h * w and per-tile sums of squares, consumer scales its rows)
    and SwiGLU in the gate_up epilogue, against the fp32 statement of norm -> linear -> swiglu -> linear."""
    from rl_b200.ops.engine_ops import skinny_linear
    from rl_b200.ops.lib import check_status

    torch.manual_seed(M)
    d, f, eps = 512, 1408, 1e-5
    dev = "cuda"
    a = torch.randn(M, d, device=dev).to(torch.bfloat16)
    res = torch.randn(M, d, device=dev).to(torch.bfloat16)
    w_o = (torch.randn(d, d, device=dev) / d**0.5).to(torch.bfloat16)
    w_norm = (1 + 0.1 * torch.randn(d, device=dev)).to(torch.bfloat16)
    w_gu = (torch.randn(2 * f, d, device=dev) / d**0.5).to(torch.bfloat16)
    w_dn = (torch.randn(d, f, device=dev) / f**0.5).to(torch.bfloat16)
    tiles = d // 128
    ssq = torch.zeros((tiles, 256), device=dev)
    hw = torch.empty((M, d), device=dev, dtype=torch.bfloat16)
    # producer: h = a W_o^T + res, plus h * w_norm and the per-tile sums of squares
    h = skinny_linear(a, w_o, residual=res, ssq_out=ssq, norm_w=w_norm, out2=hw)
    h_ref = (a.float() @ w_o.float().t() + res.float())
    assert (h.float() - h_ref).abs().max().item() < 3e-2 * h_ref.abs().max().item()
    hb = h.float()
    assert torch.allclose(ssq[:, :M].sum(0), (hb * hb).sum(-1), rtol=1e-4)
    assert (hw.float() - hb * w_norm.float()).abs().max().item() < 2e-2 * hb.abs().max().item()
    # consumer with SwiGLU: silu(norm(h) Wg^T) * (norm(h) Wu^T)
    act = skinny_linear(hw, w_gu, ssq_in=ssq, eps=eps, swiglu=True)
    xn = hb * torch.rsqrt((hb * hb).mean(-1, keepdim=True) + eps) * w_norm.float()
    gu = xn @ w_gu.float().t()
    act_ref = torch.nn.functional.silu(gu[:, :f]) * gu[:, f:]
    assert act.shape == (M, f)
    assert (act.float() - act_ref).abs().max().item() < 3e-2 * act_ref.abs().max().item() + 1e-3
    # consumer without SwiGLU, fp32 output and a bias (lm_head / qkv form)
    bias = torch.randn(d, device=dev)
    y = skinny_linear(hw, w_o, ssq_in=ssq, eps=eps, bias=bias, out_dtype=torch.float32)
    y_ref = xn @ w_o.float().t() + bias
    assert (y - y_ref).abs().max().item() < 2e-2 * y_ref.abs().max().item()
    # and the down projection closes the loop with the next norm's hand-off
    h2 = skinny_linear(act, w_dn, residual=h, ssq_out=ssq, norm_w=w_norm, out2=hw)
    h2_ref = act.float() @ w_dn.float().t() + hb
    assert (h2.float() - h2_ref).abs().max().item() < 3e-2 * h2_ref.abs().max().item()
    assert check_status() == 0
