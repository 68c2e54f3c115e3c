"""tcgen05 flash attention (varlen, causal, GQA) against fp32 PyTorch attention, forward and backward."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(lens, Hq, Hkv, seed=0, D=128):
    torch.manual_seed(seed)
    T = sum(lens)
    qkv = (torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda") * 0.7).to(torch.bfloat16)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    return qkv, cu, D


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("lens,Hq,Hkv", [([128], 2, 2), ([64], 4, 1), ([200, 57, 1, 333], 8, 2), ([1280] * 3, 32, 8), ([4096], 4, 4)])
def test_flash_fwd(native_lib, lens, Hq, Hkv, D):
    from rl_b200.ops import attention as A
    from rl_b200.ops import functional as F
    from rl_b200.ops.lib import check_status

    qkv, cu, D = _case(lens, Hq, Hkv, D=D)
    out, lse = A.flash_fwd(qkv, cu, Hq, Hkv, D, 1.0 / math.sqrt(D))
    torch.cuda.synchronize()
    assert check_status() == 0
    ref = F._attention_ref(qkv.float(), cu, Hq, Hkv, D, 1.0 / math.sqrt(D))
    err = (out.float() - ref).abs().max().item()
    assert err < 3e-2, f"max abs err {err}"
    # lse against the direct definition on the first sequence / head 0
    n = lens[0]
    q = qkv[:n, :D].float()
    k = qkv[:n, Hq * D : Hq * D + D].float()
    s = (q @ k.t()) / math.sqrt(D)
    s = s.masked_fill(torch.triu(torch.ones(n, n, device="cuda", dtype=torch.bool), 1), float("-inf"))
    assert (torch.logsumexp(s, -1) - lse[0, :n]).abs().max().item() < 2e-2


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("lens,Hq,Hkv", [([128], 2, 2), ([200, 57, 1, 333], 8, 2), ([1280, 700], 8, 2)])
def test_flash_autograd(native_lib, lens, Hq, Hkv, D):
    from rl_b200.ops import functional as F
    from rl_b200.ops.lib import check_status

    qkv, cu, D = _case(lens, Hq, Hkv, seed=1, D=D)
    x = qkv.clone().requires_grad_()
    y = F.attention_varlen(x, cu, max(lens), Hq, Hkv, D)
    g = torch.randn_like(y)
    y.backward(g)
    torch.cuda.synchronize()
    assert check_status() == 0
    xr = qkv.float().requires_grad_()
    yr = F._attention_ref(xr, cu, Hq, Hkv, D, 1.0 / math.sqrt(D))
    yr.backward(g.float())
    assert (y.float() - yr).abs().max().item() < 3e-2
    rel = (x.grad.float() - xr.grad).abs().max().item() / (xr.grad.abs().max().item() + 1e-6)
    assert rel < 3e-2, f"relative grad err {rel}"
