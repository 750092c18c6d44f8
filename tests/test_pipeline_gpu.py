"""HostPipeline: batches in pinned host memory, uploads and downloads on copy
streams that overlap the compute of neighbouring batches.  Each result must be
the bits a plain forward on that batch gives, whatever the overlap."""
import pytest
import torch

from conftest import golden


@pytest.mark.gpu
@pytest.mark.parametrize("depth,use_graph", [(1, True), (2, True), (3, True), (2, False)])
def test_pipelined_batches_equal_direct_forward(sd3, depth, use_graph):
    g = golden("model_toy.pt")
    cfg = g["config"]
    m = sd3.Model(cfg["num_layers"], cfg["dual_attention_layers"], cfg["pooled_dim"], cfg["captions_dim"],
                  cfg["in_channels"], cfg["emb_dim"], cfg["attn_heads"], cfg["mlp_expand"],
                  cfg["patch_size"], cfg["pos_embed_max_size"], cfg["base_height"], True, sd3.PRECISION_BF16)
    m.load({k: v.bfloat16().cuda() for k, v in g["params"].items()})
    B, C, H, W = g["latent"].shape
    Tc = g["captions"].shape[1]
    gen = torch.Generator().manual_seed(11)
    batches = []
    for i in range(5):
        batches.append(dict(
            pooled=torch.randn(g["pooled"].shape, generator=gen).bfloat16().pin_memory(),
            captions=torch.randn(g["captions"].shape, generator=gen).bfloat16().pin_memory(),
            latent=torch.randn(g["latent"].shape, generator=gen).bfloat16().pin_memory(),
            t=(torch.rand(B, generator=gen) * 1000).pin_memory(),
            out=torch.zeros(g["latent"].shape, dtype=torch.bfloat16).pin_memory()))
    pipe = sd3.HostPipeline(m, B, Tc, C, H, W, g["pooled"].shape[1], g["captions"].shape[2], torch.bfloat16,
                            depth=depth, use_graph=use_graph)
    for b in batches:
        pipe.submit(b["pooled"], b["captions"], b["latent"], b["t"], b["out"])
    pipe.flush()
    torch.cuda.synchronize()
    assert sd3.device_status() == 0
    for b in batches:
        ref = m.forward(b["pooled"].cuda(), b["captions"].cuda(), b["latent"].cuda(), b["t"].cuda())
        torch.cuda.synchronize()
        assert torch.equal(ref.cpu(), b["out"])
    m.close()
