"""Generates the golden fixtures in this directory by running the REFERENCE's
own PyTorch modules (module_tests/modules.py of MichelHUANGGit/SD3.c).

    python tests/golden/make_golden.py [/path/to/reference/checkout]

The reference checkout is only needed to (re)generate the fixtures; the tests
read the committed .pt files.  Every fixture stores the parameters in the
extension's boundary convention (2-D weights transposed to (in, out)), the
inputs and the reference outputs, all computed in float32 on CPU.  Parameter
and input values are rounded to bfloat16-representable numbers first, so the
same fixture serves the bf16 GPU path without a second rounding step.
"""
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bf16_round(t):
    return t.to(torch.bfloat16).to(torch.float32)


def export_params(module):
    out = {}
    for name, p in module.named_parameters():
        out[name] = p.data.clone() if p.dim() != 2 else p.data.T.contiguous()
    return out


def randomize(module, gen, std=0.05):
    """Non-trivial values everywhere (biases and RMSNorm weights included)."""
    with torch.no_grad():
        for name, p in module.named_parameters():
            if "rmsnorm" in name:
                p.copy_(bf16_round(1.0 + 0.2 * torch.randn(p.shape, generator=gen)))
            elif p.dim() >= 2:
                p.copy_(bf16_round(std * torch.randn(p.shape, generator=gen)))
            else:
                p.copy_(bf16_round(0.1 * torch.randn(p.shape, generator=gen)))


def make_block(ref, name, seed, E, heads, mlp_expand, dual, discard, qk_norm, B, Tc, Tx):
    gen = torch.Generator().manual_seed(seed)
    blk = ref.MM_DiT_Block(E, heads, mlp_expand, discard, dual, qk_norm)
    randomize(blk, gen)
    x = bf16_round(torch.randn(B, Tx, E, generator=gen))
    c = bf16_round(torch.randn(B, Tc, E, generator=gen))
    y = bf16_round(torch.nn.functional.silu(torch.randn(B, E, generator=gen)))
    with torch.no_grad():
        c_out, x_out = blk(x, c, y)
    torch.save({
        "kind": "block",
        "config": dict(emb_dim=E, attn_heads=heads, mlp_expand=mlp_expand, use_dual_attention=dual,
                       discard_context=discard, use_qk_norm=qk_norm, B=B, Tc=Tc, Tx=Tx),
        "params": {k: v.to(torch.bfloat16) for k, v in export_params(blk).items()},
        "x": x.to(torch.bfloat16), "c": c.to(torch.bfloat16), "y": y.to(torch.bfloat16),
        "c_out": c_out, "x_out": x_out,
    }, os.path.join(HERE, name))


def make_model(ref, name, seed, num_layers, dual_layers, in_dim, E, pooled_dim, captions_dim, patch,
               heads, mlp_expand, pos_max, base_height, B, Tc, H, W):
    gen = torch.Generator().manual_seed(seed)
    model = ref.MMDiT(num_layers, dual_layers, in_dim, E, pooled_dim, captions_dim, patch, heads,
                      mlp_expand, pos_max, base_height, True)
    randomize(model, gen)
    latent = bf16_round(torch.randn(B, in_dim, H, W, generator=gen))
    captions = bf16_round(torch.randn(B, Tc, captions_dim, generator=gen))
    pooled = bf16_round(torch.randn(B, pooled_dim, generator=gen))
    timesteps = bf16_round(torch.rand(B, generator=gen) * 1000.0)
    with torch.no_grad():
        out = model(latent, captions, pooled, timesteps)
        # intermediate pins: conditioning vector, embedded streams
        temb = model.timestep_mlp(ref.get_sinusoidal_embedding(timesteps, 256))
        y = torch.nn.functional.silu(temb + model.pooled_mlp(pooled))
        x0 = model.to_patch(latent)
        c0 = model.captions_linear(captions)
    torch.save({
        "kind": "model",
        "config": dict(num_layers=num_layers, dual_attention_layers=list(dual_layers), in_channels=in_dim,
                       emb_dim=E, pooled_dim=pooled_dim, captions_dim=captions_dim, patch_size=patch,
                       attn_heads=heads, mlp_expand=mlp_expand, pos_embed_max_size=pos_max,
                       base_height=base_height, B=B, Tc=Tc, H=H, W=W),
        "params": {k: v.to(torch.bfloat16) for k, v in export_params(model).items()},
        "latent": latent.to(torch.bfloat16), "captions": captions.to(torch.bfloat16),
        "pooled": pooled.to(torch.bfloat16), "timesteps": timesteps,
        "out": out, "y": y, "x0": x0, "c0": c0,
    }, os.path.join(HERE, name))


def main():
    # the reference checkout: first argument, else a directory "reference" next to this repository
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.path.join(
        os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference")
    sys.path.insert(0, os.path.join(ref_root, "module_tests"))
    import modules as ref  # the reference's PyTorch modules

    torch.set_num_threads(max(1, os.cpu_count() or 1))
    # dual block with context kept (the MMDiT-X block of layers 0-12), head_dim 64
    make_block(ref, "block_dual.pt", 11, 128, 2, 2, True, False, True, B=2, Tc=21, Tx=150)
    # last block: context discarded after attention, (scale, shift) AdaLN order
    make_block(ref, "block_last.pt", 12, 128, 2, 2, False, True, True, B=2, Tc=21, Tx=70)
    # plain block, head_dim 32, no qk norm (generic kernels)
    make_block(ref, "block_plain_hd32.pt", 13, 64, 2, 2, False, False, False, B=1, Tc=9, Tx=40)
    # full model, toy size, non-square latent, layer 0 dual
    make_model(ref, "model_toy.pt", 21, 3, (0,), 16, 128, 80, 96, 2, 2, 2, 24, 16, B=2, Tc=19, H=12, W=20)


if __name__ == "__main__":
    main()
