"""The bound on attention scores that follows from the q/k RMSNorm weights (host logic, CPU):
it must hold for adversarial inputs, and the sequence-parallel path's packed model must apply
it (pre-scaled query weights, bound in exp2 units) only where the bounded softmax accepts it."""
import math

import pytest
import torch

from conftest import load_binding
from oracle import mmdit_oracle as O


def _rms(t, w, eps=1e-6):
    return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) * w


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_bound_holds_for_random_and_adversarial_inputs(seed):
    s = load_binding()
    gen = torch.Generator().manual_seed(seed)
    wq = torch.randn(64, generator=gen) * 1.5
    wk = torch.randn(64, generator=gen) * 1.5
    bound = s.qk_norm_score_bound(wq, wk)
    # random rows
    q = _rms(torch.randn(4096, 64, generator=gen) * 10, wq)
    k = _rms(torch.randn(4096, 64, generator=gen) * 0.01, wk)
    assert (q @ k.t()).abs().max().item() <= bound
    # adversarial: all the energy in the dimension where |wq wk| is largest (both signs)
    d = int((wq.abs() * wk.abs()).argmax())
    e = torch.zeros(1, 64)
    e[0, d] = 1e4
    worst = (_rms(e, wq) @ _rms(-e, wk).t()).abs().item()
    assert worst <= bound
    assert worst >= bound / 1.02  # and the bound is tight there
    # the bf16 rounding of q and k is inside the 1 % margin
    qb, kb = _rms(e, wq).bfloat16().float(), _rms(e, wk).bfloat16().float()
    assert (qb @ kb.t()).abs().item() <= bound


def test_bound_takes_elementwise_maxima_over_streams():
    s = load_binding()
    a = torch.tensor([1.0, 3.0] + [0.5] * 62)
    b = torch.tensor([2.0, 0.1] + [0.5] * 62)
    k = torch.ones(64)
    # two query norms feed one attention: per dimension the larger weight counts
    assert math.isclose(s.qk_norm_score_bound([a, b], k), 1.01 * 64 * 3.0, rel_tol=1e-6)
    # the PRODUCT per dimension counts, not the product of the maxima
    kq = torch.tensor([0.1, 0.1] + [1.0] * 62)
    assert math.isclose(s.qk_norm_score_bound(a, kq), 1.01 * 64 * 0.5, rel_tol=1e-6)


def test_oracle_attention_is_shift_invariant():
    """What the bounded softmax relies on: softmax(s) = 2^(s c) / sum 2^(s c) for any constant
    shift, here checked on the oracle's attention against the unshifted closed form."""
    torch.manual_seed(3)
    q, k, v = (torch.randn(1, 50, 2, 64, dtype=torch.float64) for _ in range(3))
    ref = O.attention(q, k, v)
    c = 64 ** -0.5 * math.log2(math.e)
    sc = torch.einsum("bthd,bshd->bhts", q, k)
    p = torch.exp2(sc * c)
    out = torch.einsum("bhts,bshd->bthd", p, v) / p.sum(-1).permute(0, 2, 1)[..., None]
    assert torch.allclose(out.reshape(ref.shape), ref, atol=1e-10)
