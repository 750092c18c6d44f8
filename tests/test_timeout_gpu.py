"""The device-side timeout path, exercised without faulting or hanging anything: a
self-test kernel waits (1 ms limit) on a barrier that nobody arrives on, gives up,
records its code in the status word, raises the CTA abort flag, drains and returns.
No TMA, MMA or TMEM is involved, so the context stays healthy."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wait_that_runs_out_is_reported_once_and_leaves_the_device_usable(sd3):
    assert sd3.device_status() == 0
    sd3.check(sd3.lib().sd3_selftest_wait_timeout(1000, sd3.stream_ptr()), "selftest")
    torch.cuda.synchronize()
    assert sd3.device_status() == 199          # DEV_TIMEOUT_SELFTEST, read ...
    assert b"bounded wait" in sd3.lib().sd3_last_error()
    assert sd3.device_status() == 0            # ... and cleared by that read
    # the next product calls are unaffected (tcgen05 GEMM and attention)
    x = torch.randn(512, 256, device="cuda").bfloat16()
    w = (torch.randn(256, 256, device="cuda") * 0.05).bfloat16()
    y = sd3.linear(x, w)
    ref = x.float() @ w.float().t()
    assert ((y.float() - ref).norm() / ref.norm()).item() < 1e-2
    qkv = torch.randn(1, 200, 3 * 128, device="cuda").bfloat16()
    _, ox = sd3.attention(qkv, 1, 200, 2, 0, 0.125)
    q, k, v = [t.view(1, 200, 2, 64).transpose(1, 2).float() for t in qkv.split(128, dim=-1)]
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v, scale=0.125).transpose(1, 2).reshape(1, 200, 128)
    assert ((ox.float() - ref).norm() / ref.norm()).item() < 1e-2
    torch.cuda.synchronize()
    assert sd3.device_status() == 0


def test_selftest_rejects_bad_limits(sd3):
    assert sd3.lib().sd3_selftest_wait_timeout(0, sd3.stream_ptr()) == -1
    assert sd3.lib().sd3_selftest_wait_timeout(2000000, sd3.stream_ptr()) == -1
