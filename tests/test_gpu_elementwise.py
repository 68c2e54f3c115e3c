"""Memory-bound kernels (RMSNorm, RoPE, SwiGLU, embedding, AdamW, ClippedPG, sampling, paged decode) against the
fp32 PyTorch restatement of each operator."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(a, b, tol):
    err = (a.float() - b.float()).abs().max().item()
    ref = b.float().abs().max().item() + 1e-6
    assert err / ref < tol, f"rel err {err / ref:.3e}"


def _ref_mode(fn, *args, **kw):
    """Runs an operator's PyTorch restatement on CPU copies of the arguments."""
    cpu = [a.detach().cpu() if isinstance(a, torch.Tensor) else a for a in args]
    return fn(*cpu, **kw)


@pytest.mark.parametrize("rows,d", [(7, 64), (513, 4096), (33, 5120), (100, 128)])
def test_rmsnorm_fwd_bwd(native_lib, rows, d):
    from rl_b200.ops import functional as F

    torch.manual_seed(0)
    x = torch.randn(rows, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(d, device="cuda")).to(torch.bfloat16).requires_grad_()
    y = F.rmsnorm(x, w, 1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    yr.backward(g.float())
    _close(y, yr, 1e-2)
    _close(x.grad, xr.grad, 2e-2)
    _close(w.grad, wr.grad, 2e-2)


def test_rmsnorm_residual(native_lib):
    from rl_b200.ops import functional as F

    x = torch.randn(65, 1024, device="cuda", dtype=torch.bfloat16)
    r = torch.randn(65, 1024, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(1024, device="cuda", dtype=torch.bfloat16)
    r_ref = (r.float() + x.float()).to(torch.bfloat16)
    y_ref = F._rmsnorm_ref(r_ref, w, 1e-6)
    y = F.rmsnorm_residual_(x, r, w, 1e-6)
    _close(r, r_ref, 1e-6)
    _close(y, y_ref, 1e-2)


def test_rope_and_inverse(native_lib):
    from rl_b200.ops import functional as F

    T, Hq, Hkv, D = 50, 8, 2, 128
    x = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16)
    pos = torch.randint(0, 4000, (T,), device="cuda", dtype=torch.int32)
    inv_freq = 1.0 / (500000.0 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    ref = F._rope_ref(x.clone(), pos, inv_freq, Hq + Hkv, D)
    x0 = x.clone()
    y = F.rope(x, pos, inv_freq, Hq + Hkv, D)
    _close(y, ref, 1e-2)
    assert torch.equal(y[:, (Hq + Hkv) * D :], x0[:, (Hq + Hkv) * D :])
    # autograd: gradient of sum(rope(x) * g) is the inverse rotation of g
    xg = x0.clone().requires_grad_()
    g = torch.randn_like(x0)
    (F.rope(xg * 1.0, pos, inv_freq, Hq + Hkv, D) * g).sum().backward()
    ref_g = F._rope_ref(g, pos, inv_freq, Hq + Hkv, D, sign=-1.0)
    _close(xg.grad, ref_g, 1e-2)


def test_head_rmsnorm(native_lib):
    from rl_b200.ops import functional as F

    T, Hq, Hkv, D = 40, 4, 2, 128
    buf = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(D, device="cuda")).to(torch.bfloat16).requires_grad_()
    out = F.head_rmsnorm(buf, w, 0, Hq, D, 1e-6)
    g = torch.randn_like(out)
    out.backward(g)
    bc = buf.detach().cpu().float().requires_grad_()
    wc = w.detach().cpu().float().requires_grad_()
    oc = F.head_rmsnorm(bc, wc, 0, Hq, D, 1e-6)
    oc.backward(g.cpu().float())
    _close(out.cpu(), oc, 1e-2)
    _close(buf.grad.cpu(), bc.grad, 2e-2)
    _close(w.grad.cpu(), wc.grad, 2e-2)


def test_swiglu(native_lib):
    from rl_b200.ops import functional as F

    gu = torch.randn(130, 2 * 688, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = F.swiglu(gu)
    g = torch.randn_like(y)
    y.backward(g)
    gr = gu.detach().float().requires_grad_()
    a, b = gr.chunk(2, -1)
    yr = torch.nn.functional.silu(a) * b
    yr.backward(g.float())
    _close(y, yr, 1e-2)
    _close(gu.grad, gr.grad, 2e-2)


def test_embedding(native_lib):
    from rl_b200.ops import functional as F

    table = torch.randn(1000, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    ids = torch.randint(0, 1000, (4, 33), device="cuda")
    y = F.embedding(ids, table)
    assert torch.equal(y, table.detach()[ids])
    g = torch.randn_like(y)
    y.backward(g)
    ref = torch.zeros(1000, 256, device="cuda")
    ref.index_add_(0, ids.reshape(-1), g.reshape(-1, 256).float())
    _close(table.grad, ref, 1e-2)


@pytest.mark.parametrize("split", [False, True])
@pytest.mark.parametrize("gdtype", [torch.bfloat16, torch.float32])
def test_adamw(native_lib, split, gdtype):
    from rl_b200.ops import functional as F

    torch.manual_seed(0)
    n = 100_003
    w0 = torch.randn(n, device="cuda")
    g = (torch.randn(n, device="cuda") * 0.1).to(gdtype)
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    ref = torch.nn.Parameter(w0.clone())
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    if split:
        hi, lo = F.split_master(w0)
        assert torch.equal(F.join_master(hi, lo), w0)
        p32 = None
    else:
        hi, lo, p32 = torch.empty(n, device="cuda", dtype=torch.bfloat16), None, w0.clone()
    for step in range(1, 4):
        ref.grad = g.float().clone()
        opt.step()
        F.adamw_step(hi, lo, p32, g, m, v, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
    got = F.join_master(hi, lo) if split else p32
    assert (got - ref.detach()).abs().max().item() < 1e-5
    if split:
        assert torch.equal(hi, F.split_master(got)[0])
    else:
        assert torch.equal(hi, got.to(torch.bfloat16))


def test_sumsq_clip(native_lib):
    from rl_b200.ops import functional as F

    x = torch.randn(1_000_001, device="cuda")
    acc = torch.zeros(1, device="cuda")
    F.sumsq_(x, acc)
    F.sumsq_(x.to(torch.bfloat16), acc)
    ref = x.pow(2).sum() + x.to(torch.bfloat16).float().pow(2).sum()
    assert abs(acc.item() - ref.item()) / ref.item() < 1e-4
    scale = torch.zeros(1, device="cuda")
    norm = torch.zeros(1, device="cuda")
    F.clip_scale(acc, 1.0, 0.5, scale, norm)
    assert abs(norm.item() - math.sqrt(ref.item())) / norm.item() < 1e-4
    assert abs(scale.item() - 0.5 / math.sqrt(ref.item())) < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sampling_greedy_and_logprob(native_lib, dtype):
    from rl_b200.ops.engine_ops import sample

    torch.manual_seed(0)
    B, V = 9, 128256
    logits = (torch.randn(B, V, device="cuda") * 3).to(dtype)
    tok, lp = sample(logits, greedy=True)
    ref = torch.log_softmax(logits.float(), -1)
    assert torch.equal(tok.long(), logits.float().argmax(-1))
    assert (lp - ref.gather(-1, tok.long()[:, None])[:, 0]).abs().max().item() < 1e-3
    # stochastic: logprob consistent with temperature-scaled distribution, tokens differ across steps
    t1, l1 = sample(logits, temperature=0.7, seed=5, step=1)
    t2, _ = sample(logits, temperature=0.7, seed=5, step=2)
    t1b, _ = sample(logits, temperature=0.7, seed=5, step=1)
    assert torch.equal(t1, t1b) and not torch.equal(t1, t2)
    ref7 = torch.log_softmax(logits.float() / 0.7, -1)
    assert (l1 - ref7.gather(-1, t1.long()[:, None])[:, 0]).abs().max().item() < 1e-3


def test_sampling_distribution_and_filters(native_lib):
    from rl_b200.ops.engine_ops import sample

    torch.manual_seed(1)
    V = 50
    base = torch.randn(V, device="cuda") * 2
    n = 20000
    logits = base[None].repeat(n, 1).contiguous()
    tok, lp = sample(logits, temperature=1.0, seed=11, step=0)
    freq = torch.bincount(tok.long(), minlength=V).float() / n
    p = torch.softmax(base, -1)
    assert (freq - p).abs().max().item() < 0.015
    # top-k = 5: only the 5 largest appear and logprobs renormalise over them
    tok, lp = sample(logits, top_k=5, seed=3, step=0)
    top5 = torch.topk(base, 5).indices
    assert set(tok.unique().tolist()) <= set(top5.tolist())
    ref = torch.log_softmax(base[top5], -1)
    idx = {int(t): i for i, t in enumerate(top5.tolist())}
    want = torch.tensor([ref[idx[int(t)]].item() for t in tok[:100].tolist()], device="cuda")
    assert (lp[:100] - want).abs().max().item() < 1e-3
    # top-p = 0.6: the kept set is the smallest prefix of the sorted probabilities reaching 0.6
    tok, lp = sample(logits, top_p=0.6, seed=4, step=0)
    sp, si = torch.sort(p, descending=True)
    keep = int(((sp.cumsum(0) - sp) < 0.6).sum().item())
    assert set(tok.unique().tolist()) <= set(si[:keep].tolist())
    assert len(tok.unique()) == keep


def test_sampling_top_k_then_top_p(native_lib):
    """Both filters on: top-k first, then the nucleus inside the renormalised top-k set (same kept set and the same
    log-probabilities as the CPU statement of the sampler)."""
    from rl_b200.ops.engine_ops import sample

    V, n = 64, 4000
    probs = torch.full((V,), 0.01 / (V - 3))
    probs[:3] = torch.tensor([0.95, 0.03, 0.01])
    peaked = probs.log()
    # a flatter row: top_k = 6 keeps 6 tokens, top_p = 0.7 of THEIR mass cuts further
    torch.manual_seed(5)
    flat = torch.randn(V)
    for base, k, p_ in ((peaked, 3, 0.9), (flat, 6, 0.7), (flat, 10, 0.5)):
        logits = base[None].repeat(n, 1).contiguous()
        tok_c, lp_c = sample(logits, top_k=k, top_p=p_, seed=1)           # CPU statement
        full = torch.log_softmax(base, -1)
        kth = torch.topk(base, k).values[-1]
        zk = base.masked_fill(base < kth, float("-inf"))
        sz, si = torch.sort(zk, descending=True)
        pr = torch.softmax(sz, -1)
        keep = si[((pr.cumsum(0) - pr) < p_)]
        ref_lp = torch.log_softmax(base[keep], -1)
        idx = {int(t): i for i, t in enumerate(keep.tolist())}
        tok, lp = sample(logits.cuda(), top_k=k, top_p=p_, seed=9, step=0)
        seen = set(tok.unique().tolist())
        assert seen <= set(keep.tolist()), (seen, keep.tolist())
        if len(keep) <= 4:
            assert seen == set(keep.tolist())
        want = torch.tensor([ref_lp[idx[int(t)]].item() for t in tok[:200].tolist()])
        assert (lp[:200].cpu() - want).abs().max().item() < 1e-3
        assert set(tok_c.unique().tolist()) <= set(keep.tolist())
        del full


@pytest.mark.parametrize("Hq,Hkv", [(32, 8), (8, 8), (16, 2)])
@pytest.mark.parametrize("splits", [1, 3])
@pytest.mark.parametrize("bs", [16, 64, 128, 48])
def test_paged_decode(native_lib, Hq, Hkv, splits, bs):
    from rl_b200.ops import engine_ops as E
    from rl_b200.ops.lib import check_status

    torch.manual_seed(0)
    D, nblocks, B = 128, 64, 5
    kc = torch.randn(nblocks, Hkv, bs, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn(nblocks, Hkv, bs, D, device="cuda", dtype=torch.bfloat16)
    lens = torch.tensor([1, 17, 100, 160, 333], device="cuda", dtype=torch.int32)
    perm = torch.randperm(nblocks, device="cuda").to(torch.int32)
    bt = torch.zeros(B, 24, device="cuda", dtype=torch.int32)
    c = 0
    for b in range(B):
        nb = (int(lens[b]) + bs - 1) // bs
        bt[b, :nb] = perm[c : c + nb]
        c += nb
    q = torch.randn(B, Hq * D, device="cuda", dtype=torch.bfloat16)
    out = E.paged_decode(q, kc, vc, bt, lens, Hq, Hkv, D, num_splits=splits)
    torch.cuda.synchronize()
    assert check_status() == 0
    ref = E.paged_decode(q.cpu(), kc.cpu(), vc.cpu(), bt.cpu(), lens.cpu(), Hq, Hkv, D)
    _close(out.cpu(), ref, 2e-2)


def test_kv_cache_write(native_lib):
    from rl_b200.ops import engine_ops as E

    Hq, Hkv, D, bs = 8, 2, 128, 16
    T = 37
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16)
    kc = torch.zeros(10, Hkv, bs, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    slots = torch.randperm(10 * bs, device="cuda")[:T].to(torch.int64)
    slots[3] = -1
    E.kv_cache_write(qkv, slots, kc, vc, Hq, Hkv, D)
    kr, vr = torch.zeros_like(kc).cpu(), torch.zeros_like(vc).cpu()
    E.kv_cache_write(qkv.cpu(), slots.cpu(), kr, vr, Hq, Hkv, D)
    assert torch.equal(kc.cpu(), kr) and torch.equal(vc.cpu(), vr)


@pytest.mark.parametrize("cfg", [
    dict(reference_policy_kl_penalty=0.05),
    dict(reference_policy_kl_penalty=0.05, reference_policy_kl_type="k2", ratio_clip_c=3.0),
    dict(reference_policy_kl_penalty=0.1, use_on_policy_kl_approximation=True, use_importance_sampling_correction=True,
         truncated_importance_sampling_ratio=2.0, truncated_importance_sampling_type="tis"),
    # custom clamps: the input clamp is active on some tokens (weight detached there), no output clamp
    dict(reference_policy_kl_penalty=0.1, kl_input_clamp_value=0.5, kl_output_clamp_value=None,
         use_on_policy_kl_approximation=True),
    dict(reference_policy_kl_penalty=0.1, kl_input_clamp_value=0.5, kl_output_clamp_value=None, reference_policy_kl_type="k1"),
    dict(reference_policy_kl_penalty=0.0, use_cispo=True),
])
def test_fused_clipped_pg_matches_pytorch_statement(native_lib, cfg):
    """Loss value, metrics and d loss / d logprob of the fused kernel against the PyTorch statement of the same loss."""
    from rl_b200.algorithms.loss.loss_functions import ClippedPGLossFn
    from rl_b200.distributed.batched_data_dict import BatchedDataDict

    g = torch.Generator().manual_seed(3)
    B, S = 6, 40
    tm = torch.ones(B, S)
    tm[:, :5] = 0
    prev = -torch.rand(B, S, generator=g) * 3
    data = BatchedDataDict(token_mask=tm, sample_mask=torch.tensor([1.0, 1, 1, 0, 1, 1]), advantages=torch.randn(B, S, generator=g),
                           prev_logprobs=prev, generation_logprobs=prev + 0.05 * torch.randn(B, S, generator=g),
                           reference_policy_logprobs=prev + 1.5 * torch.randn(B, S, generator=g)).to("cuda")
    fn = ClippedPGLossFn(cfg)
    base = (prev[:, 1:] + 0.4 * torch.randn(B, S - 1, generator=g)).cuda()
    mask = data["token_mask"][:, 1:] * data["sample_mask"][:, None]
    N = mask.sum()
    c1 = base.clone().requires_grad_()
    assert fn._can_fuse(c1, data)
    l1, m1 = fn(c1, data, torch.tensor(5.0), N)
    l1.backward()
    c2 = base.clone().requires_grad_()
    args = (c2, data["prev_logprobs"][:, 1:], data["generation_logprobs"][:, 1:],
            data["reference_policy_logprobs"][:, 1:] if fn.cfg["reference_policy_kl_penalty"] != 0 else None,
            data["advantages"][:, 1:], data["token_mask"][:, 1:], data["sample_mask"], mask, data, torch.tensor(5.0), N)
    l2, m2 = fn._reference(*args)
    l2.backward()
    assert l1.item() == pytest.approx(l2.item(), rel=2e-4, abs=1e-6)
    assert (c1.grad - c2.grad).abs().max().item() <= 2e-4 * c2.grad.abs().max().item() + 1e-8
    for k in ("probs_ratio", "kl_penalty", "token_mult_prob_error"):
        assert m1[k] == pytest.approx(m2[k], rel=1e-3, abs=1e-6), k
