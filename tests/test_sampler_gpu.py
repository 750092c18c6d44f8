"""Sampling loop (Euler flow matching + classifier-free guidance, in
miniature): the fused update kernel and the loop around the
denoiser against the CPU oracle's loop on the toy golden model."""
import pytest
import torch

from conftest import golden
from oracle import mmdit_oracle as O


def test_sigma_schedule_matches_oracle_and_is_monotone(sd3):
    for steps, shift in ((28, 3.0), (4, 1.0), (1, 3.0)):
        a, b = sd3.sigma_schedule(steps, shift), O.sigma_schedule(steps, shift)
        assert len(a) == steps + 1 and a[0] == pytest.approx(1.0) and a[-1] == 0.0
        assert all(x > y for x, y in zip(a, a[1:]))
        assert a == pytest.approx(b)


@pytest.mark.gpu
def test_cfg_euler_step_kernel(sd3):
    torch.manual_seed(0)
    n = 3 * 16 * 8 * 8
    for dtype in (torch.float32, torch.bfloat16):
        x = torch.randn(n, device="cuda")
        v = torch.randn(2 * n, device="cuda").to(dtype)
        x2 = torch.zeros(2 * n, device="cuda", dtype=dtype)
        ref = x + (-0.07) * (v[n:].float() + 4.5 * (v[:n].float() - v[n:].float()))
        sd3.check(sd3.lib().sd3_cfg_euler_step(sd3.ptr(x), sd3.ptr(x2), sd3.ptr(v), sd3.dtype_tag(x2), n,
                                               4.5, -0.07, sd3.stream_ptr()))
        assert (x - ref).abs().max().item() < 1e-5
        assert torch.equal(x2[:n], x.to(dtype)) and torch.equal(x2[n:], x.to(dtype))


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["f32", "bf16"])
def test_sampling_loop_matches_oracle(sd3, mode):
    g = golden("model_toy.pt")
    cfg = g["config"]
    dtype = torch.float32 if mode == "f32" else torch.bfloat16
    precision = sd3.PRECISION_F32 if mode == "f32" else sd3.PRECISION_BF16
    m = sd3.Model(cfg["num_layers"], cfg["dual_attention_layers"], cfg["pooled_dim"], cfg["captions_dim"],
                  cfg["in_channels"], cfg["emb_dim"], cfg["attn_heads"], cfg["mlp_expand"],
                  cfg["patch_size"], cfg["pos_embed_max_size"], cfg["base_height"], True, precision)
    m.load({k: v.to(dtype).cuda() for k, v in g["params"].items()})
    gen = torch.Generator().manual_seed(4)
    lat = g["latent"].float()
    un_caps = torch.randn(g["captions"].shape, generator=gen).bfloat16().float()
    un_pool = torch.randn(g["pooled"].shape, generator=gen).bfloat16().float()
    steps = 4
    out = sd3.sample(m, lat.to(dtype).cuda(), g["captions"].to(dtype).cuda(), g["pooled"].to(dtype).cuda(),
                     un_caps.to(dtype).cuda(), un_pool.to(dtype).cuda(), steps=steps, guidance=4.5, shift=3.0)
    torch.cuda.synchronize()
    assert sd3.device_status() == 0
    m.close()
    p = {k: v.float() for k, v in g["params"].items()}
    ref = O.sample_loop(lat, g["captions"].float(), g["pooled"].float(), un_caps, un_pool, p, cfg, steps)
    if mode == "f32":
        assert (out.cpu() - ref).abs().max().item() < 5e-4  # four chained model calls, guidance 4.5
    else:
        rel = ((out.cpu() - ref).norm() / ref.norm()).item()
        assert rel < 2e-2  # guidance amplifies the per-call bf16 error (~3e-3) by (2g - 1)


@pytest.mark.gpu
def test_sampling_loop_as_one_cuda_graph_gives_the_same_bits(sd3):
    g = golden("model_toy.pt")
    cfg = g["config"]
    m = sd3.Model(cfg["num_layers"], cfg["dual_attention_layers"], cfg["pooled_dim"], cfg["captions_dim"],
                  cfg["in_channels"], cfg["emb_dim"], cfg["attn_heads"], cfg["mlp_expand"],
                  cfg["patch_size"], cfg["pos_embed_max_size"], cfg["base_height"], True, sd3.PRECISION_BF16)
    m.load({k: v.bfloat16().cuda() for k, v in g["params"].items()})
    gen = torch.Generator().manual_seed(5)
    un_caps = torch.randn(g["captions"].shape, generator=gen).bfloat16().cuda()
    un_pool = torch.randn(g["pooled"].shape, generator=gen).bfloat16().cuda()
    args = (g["latent"].bfloat16().cuda(), g["captions"].bfloat16().cuda(), g["pooled"].bfloat16().cuda(),
            un_caps, un_pool)
    eager = sd3.sample(m, *args, steps=3, guidance=4.5, shift=3.0)
    graphed = sd3.sample(m, *args, steps=3, guidance=4.5, shift=3.0, use_graph=True)
    torch.cuda.synchronize()
    assert sd3.device_status() == 0
    assert torch.equal(eager, graphed)
    m.close()
