"""CPU oracle for the SD3.5-medium MMDiT-X denoiser forward.

TEST INFRASTRUCTURE ONLY.  This file is a plain-PyTorch restatement of the
reference's own PyTorch modules (module_tests/modules.py of
MichelHUANGGit/SD3.c), written as free functions over the reference's
parameter-dict boundary convention (named_parameters() keys, every 2-D weight
transposed to (in, out); module_tests/DiT.py:25-31).  It is imported by
tests/, by __graft_entry__.smoke() and by bench.py's CPU-baseline legs as the
checker / CPU baseline; the product (the CUDA library) never calls it.

Parity pin: tests/golden/*.pt were produced by running the reference modules
themselves (tests/golden/make_golden.py imports them from the reference
checkout); tests/test_oracle.py checks this file against those fixtures.

Each function names the reference lines it restates.
"""
import math

import torch
import torch.nn.functional as F


def linear(x, w_in_out, b=None):
    """nn.Linear with the boundary weight layout (in, out): y = x W + b
    (modules.cpp:475-490; module_tests/DiT.py:31)."""
    y = x @ w_in_out
    return y if b is None else y + b


def sinusoidal_embedding(t, dim=256):
    """get_sinusoidal_embedding, module_tests/modules.py:70-77 (cos first)."""
    half = dim // 2
    freqs = torch.exp(-9.2103403719761836 * torch.arange(half, dtype=torch.float32) / half)[None, :]
    a = t.to(torch.float32)[:, None] * freqs.to(t.device)
    return torch.cat([torch.cos(a), torch.sin(a)], dim=1)


def pos_embed_cropped(emb_dim, h, w, pos_max, base_size):
    """positional_encoding_2D_HF + PatchEmbedding.crop_pos_enc,
    module_tests/modules.py:79-99 and 43-53, evaluated only on the cropped
    (h, w) window: token (r, s) uses column position S = s + (pos_max - w)//2 for
    the first half of the channels and row position R = r + (pos_max - h)//2 for
    the second half (the reference's meshgrid(..., indexing="xy") makes its
    `pos_h` vary along columns).  float64 math, cast to float32."""
    oh, ow = (pos_max - h) // 2, (pos_max - w) // 2
    grid = torch.arange(pos_max, dtype=torch.float64) / (pos_max / base_size)
    div = 1.0 / (10000.0 ** (torch.arange(emb_dim // 4, dtype=torch.float64) / (emb_dim / 4.0)))
    col = grid[ow:ow + w]  # (w,)
    row = grid[oh:oh + h]  # (h,)
    pc = col[None, :, None] * div  # (1, w, q)
    pr = row[:, None, None] * div  # (h, 1, q)
    pc = pc.expand(h, w, -1)
    pr = pr.expand(h, w, -1)
    out = torch.cat([torch.sin(pc), torch.cos(pc), torch.sin(pr), torch.cos(pr)], dim=-1)
    return out.reshape(h * w, emb_dim).to(torch.float32)


def patch_embed(latent, conv_w, conv_b, pos_max, base_height, patch):
    """PatchEmbedding.forward, module_tests/modules.py:56-68: conv with
    kernel = stride = patch, tokens row-major over (h, w), plus the cropped
    position table."""
    x = F.conv2d(latent, conv_w, conv_b, stride=patch)
    B, E, h, w = x.shape
    x = x.flatten(2).transpose(1, 2)
    pe = pos_embed_cropped(E, h, w, pos_max, base_height // patch).to(device=x.device, dtype=x.dtype)
    return x + pe


def layer_norm(x, eps):
    """nn.LayerNorm(elementwise_affine=False), module_tests/modules.py:221,232,393."""
    mean = x.mean(-1, keepdim=True)
    var = (x - mean).pow(2).mean(-1, keepdim=True)
    return (x - mean) * torch.rsqrt(var + eps)


def rms_norm(x, weight, eps=1e-6):
    """RMSNorm.forward, module_tests/modules.py:188-203 (fp32 statistics)."""
    var = x.to(torch.float32).pow(2).mean(-1, keepdim=True)
    y = x * torch.rsqrt(var + eps)
    if weight is not None:
        y = y.to(weight.dtype) * weight
    return y


def attention(q, k, v):
    """F.scaled_dot_product_attention on (B, T, NH, D) inputs, no mask
    (module_tests/modules.py:302-307, 330-331).  Returns (B, T, NH*D)."""
    o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
    return o.transpose(1, 2).flatten(2, -1)


def mlp(x, p, prefix):
    """MLP.forward, module_tests/modules.py:166-170 (GELU tanh)."""
    h = linear(x, p[prefix + ".lin1.weight"], p[prefix + ".lin1.bias"])
    h = F.gelu(h, approximate="tanh")
    return linear(h, p[prefix + ".lin2.weight"], p[prefix + ".lin2.bias"])


def dit_block(x, c, y, p, attn_heads, use_dual_attention, use_qk_norm, discard_context, prefix=""):
    """MM_DiT_Block.forward, module_tests/modules.py:255-355.  `p` holds the
    block's parameters under `prefix`.  Returns (c_out or None, x_out)."""
    g = lambda n: p[prefix + n]
    B, Tc, C = c.shape
    Tx = x.shape[1]
    D = C // attn_heads

    ada_c = linear(y, g("context_ada_lnorm.linear.weight"), g("context_ada_lnorm.linear.bias"))[:, None, :]
    if not discard_context:
        shift_a_c, scale_a_c, gate_a_c, shift_m_c, scale_m_c, gate_m_c = ada_c.chunk(6, dim=-1)
    else:
        scale_a_c, shift_a_c = ada_c.chunk(2, dim=-1)  # swapped order, modules.py:267-268
    c_h = (1.0 + scale_a_c) * layer_norm(c, 1e-6) + shift_a_c
    qc, kc, vc = linear(c_h, g("context_to_qkv.weight"), g("context_to_qkv.bias")).chunk(3, dim=-1)
    qc, kc, vc = (t.reshape(B, Tc, attn_heads, D) for t in (qc, kc, vc))

    ada_x = linear(y, g("latent_ada_lnorm.linear.weight"), g("latent_ada_lnorm.linear.bias"))[:, None, :]
    if use_dual_attention:
        (shift_a_x, scale_a_x, gate_a_x, shift_m_x, scale_m_x, gate_m_x,
         shift_a_x2, scale_a_x2, gate_a_x2) = ada_x.chunk(9, dim=-1)
    else:
        shift_a_x, scale_a_x, gate_a_x, shift_m_x, scale_m_x, gate_m_x = ada_x.chunk(6, dim=-1)
    x_ln = layer_norm(x, 1e-6)
    x1 = (1.0 + scale_a_x) * x_ln + shift_a_x
    qx, kx, vx = linear(x1, g("latent_to_qkv.weight"), g("latent_to_qkv.bias")).chunk(3, dim=-1)
    qx, kx, vx = (t.reshape(B, Tx, attn_heads, D) for t in (qx, kx, vx))

    if use_qk_norm:
        kc = rms_norm(kc, g("context_rmsnorm_key.weight"))
        qc = rms_norm(qc, g("context_rmsnorm_query.weight"))
        kx = rms_norm(kx, g("latent_rmsnorm_key.weight"))
        qx = rms_norm(qx, g("latent_rmsnorm_query.weight"))

    # context tokens first, then image tokens (modules.py:302-304)
    o = attention(torch.cat([qc, qx], 1), torch.cat([kc, kx], 1), torch.cat([vc, vx], 1))

    if not discard_context:
        c = c + gate_a_c * linear(o[:, :Tc], g("context_attn_Wout.weight"), g("context_attn_Wout.bias"))
    x = x + gate_a_x * linear(o[:, Tc:], g("latent_attn_Wout.weight"), g("latent_attn_Wout.bias"))

    if use_dual_attention:
        x2 = (1.0 + scale_a_x2) * x_ln + shift_a_x2  # same LayerNorm of the block input
        q2, k2, v2 = linear(x2, g("latent_dual_to_qkv.weight"), g("latent_dual_to_qkv.bias")).chunk(3, dim=-1)
        q2, k2, v2 = (t.reshape(B, Tx, attn_heads, D) for t in (q2, k2, v2))
        if use_qk_norm:
            q2 = rms_norm(q2, g("latent_dual_rmsnorm_query.weight"))
            k2 = rms_norm(k2, g("latent_dual_rmsnorm_key.weight"))
        o2 = attention(q2, k2, v2)
        x = x + gate_a_x2 * linear(o2, g("latent_dual_attn_Wout.weight"), g("latent_dual_attn_Wout.bias"))

    x_h = layer_norm(x, 1e-6) * (1.0 + scale_m_x) + shift_m_x
    x = x + gate_m_x * mlp(x_h, p, prefix + "latent_mlp")

    if not discard_context:
        c_h = layer_norm(c, 1e-6) * (1.0 + scale_m_c) + shift_m_c
        c = c + gate_m_c * mlp(c_h, p, prefix + "context_mlp")
    else:
        c = None
    return c, x


def conditioning(pooled, timesteps, p):
    """y of MMDiT.forward, module_tests/modules.py:403-407."""
    emb = sinusoidal_embedding(timesteps, 256).to(pooled.dtype)
    t = linear(F.silu(linear(emb, p["timestep_mlp.0.weight"], p["timestep_mlp.0.bias"])),
               p["timestep_mlp.2.weight"], p["timestep_mlp.2.bias"])
    q = linear(F.silu(linear(pooled, p["pooled_mlp.0.weight"], p["pooled_mlp.0.bias"])),
               p["pooled_mlp.2.weight"], p["pooled_mlp.2.bias"])
    return F.silu(t + q)


def dit_forward(pooled, captions, latent, timesteps, p, num_layers, dual_attention_layers,
                attn_heads, patch_size, pos_embed_max_size, base_height, use_qk_norm=True):
    """MMDiT.forward, module_tests/modules.py:397-425, with the argument order of
    the extension's DiT entry point (modules.cpp:1605-1613)."""
    B, C_in, H, W = latent.shape
    y = conditioning(pooled, timesteps, p)
    c = linear(captions, p["captions_linear.weight"], p["captions_linear.bias"])
    x = patch_embed(latent, p["to_patch.conv.weight"], p["to_patch.conv.bias"], pos_embed_max_size,
                    base_height, patch_size)
    dual = set(int(l) for l in dual_attention_layers)
    for l in range(num_layers):
        last = l == num_layers - 1
        c, x = dit_block(x, c, y, p, attn_heads, (l in dual) and not last, use_qk_norm, last,
                         prefix="transformer.%d." % l)
    ada = linear(y, p["ada_ln_out.linear.weight"], p["ada_ln_out.linear.bias"])[:, None, :]
    scale, shift = ada.chunk(2, dim=-1)  # (scale, shift) order, modules.py:414
    h = layer_norm(x, 1e-5) * (1.0 + scale) + shift
    o = linear(h, p["linear_out.weight"], p["linear_out.bias"])
    hp, wp = H // patch_size, W // patch_size
    o = o.view(B, hp, wp, patch_size, patch_size, C_in)
    o = torch.einsum("bhwpqc->bchpwq", o)
    return o.flatten(2, 3).flatten(3, 4)


# ---------------------------------------------------------------------------
# seeded synthetic parameters / inputs (SD3.5-medium shapes)
# ---------------------------------------------------------------------------
def block_param_shapes(E, mlp_expand, head_dim, dual, discard_context, qk_norm=True):
    """name -> shape in the boundary layout ((in, out) for 2-D weights)."""
    Fh = E * mlp_expand
    s = {}

    def lin(name, i, o):
        s[name + ".weight"] = (i, o)
        s[name + ".bias"] = (o,)

    lin("context_ada_lnorm.linear", E, (2 if discard_context else 6) * E)
    lin("context_to_qkv", E, 3 * E)
    if qk_norm:
        s["context_rmsnorm_key.weight"] = (head_dim,)
        s["context_rmsnorm_query.weight"] = (head_dim,)
    if not discard_context:
        lin("context_attn_Wout", E, E)
        lin("context_mlp.lin1", E, Fh)
        lin("context_mlp.lin2", Fh, E)
    lin("latent_ada_lnorm.linear", E, (9 if dual else 6) * E)
    lin("latent_to_qkv", E, 3 * E)
    if qk_norm:
        s["latent_rmsnorm_key.weight"] = (head_dim,)
        s["latent_rmsnorm_query.weight"] = (head_dim,)
    lin("latent_attn_Wout", E, E)
    lin("latent_mlp.lin1", E, Fh)
    lin("latent_mlp.lin2", Fh, E)
    if dual:
        lin("latent_dual_to_qkv", E, 3 * E)
        if qk_norm:
            s["latent_dual_rmsnorm_key.weight"] = (head_dim,)
            s["latent_dual_rmsnorm_query.weight"] = (head_dim,)
        lin("latent_dual_attn_Wout", E, E)
    return s


def model_param_shapes(num_layers, dual_layers, in_dim, E, pooled_dim, captions_dim, patch,
                       attn_heads, mlp_expand, qk_norm=True):
    s = {}

    def lin(name, i, o):
        s[name + ".weight"] = (i, o)
        s[name + ".bias"] = (o,)

    lin("timestep_mlp.0", 256, E)
    lin("timestep_mlp.2", E, E)
    lin("pooled_mlp.0", pooled_dim, E)
    lin("pooled_mlp.2", E, E)
    lin("captions_linear", captions_dim, E)
    s["to_patch.conv.weight"] = (E, in_dim, patch, patch)
    s["to_patch.conv.bias"] = (E,)
    dual = set(dual_layers)
    for l in range(num_layers):
        last = l == num_layers - 1
        for k, v in block_param_shapes(E, mlp_expand, E // attn_heads, (l in dual) and not last, last,
                                       qk_norm).items():
            s["transformer.%d.%s" % (l, k)] = v
    lin("ada_ln_out.linear", E, 2 * E)
    lin("linear_out", E, patch * patch * in_dim)
    return s


def random_params(shapes, seed, std=0.02, dtype=torch.float32, device="cpu", bias_std=0.0,
                  norm_std=0.0):
    """Weights N(0, std) for dim >= 2; biases N(0, bias_std) (0 -> zeros);
    RMSNorm weights 1 + N(0, norm_std)."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    out = {}
    for name, shp in shapes.items():
        if len(shp) >= 2:
            t = torch.randn(shp, generator=gen) * std
        elif "rmsnorm" in name:
            t = 1.0 + torch.randn(shp, generator=gen) * norm_std
        else:
            t = torch.randn(shp, generator=gen) * bias_std
        out[name] = t.to(dtype).to(device)
    return out


SD35_MEDIUM = dict(num_layers=24, dual_layers=tuple(range(13)), in_dim=16, E=1536, pooled_dim=2048,
                   captions_dim=4096, patch=2, attn_heads=24, mlp_expand=4, pos_max=384,
                   base_height=128)


def sigma_schedule(steps, shift=3.0):
    """Shifted flow-matching sigmas used by the sampling-loop checks:
    s = shift*u/(1+(shift-1)*u), u = 1 - i/steps, then a final 0.  The reference
    has no sampler, so this schedule is pinned by nothing in the reference; the
    loop is checked step for step against this restatement only."""
    sig = [shift * (1.0 - i / steps) / (1.0 + (shift - 1.0) * (1.0 - i / steps)) for i in range(steps)]
    return sig + [0.0]


def sample_loop(latents, cond_captions, cond_pooled, uncond_captions, uncond_pooled, p, cfg, steps,
                guidance=4.5, shift=3.0):
    """Euler flow-matching sampling with classifier-free guidance around
    dit_forward: x <- x + (s_{i+1} - s_i) (v_u + g (v_c - v_u)), t = 1000 s_i."""
    x = latents.clone()
    sig = sigma_schedule(steps, shift)
    n = x.shape[0]
    for i in range(steps):
        t = torch.full((n,), 1000.0 * sig[i])
        args = (p, cfg["num_layers"], cfg["dual_attention_layers"], cfg["attn_heads"], cfg["patch_size"],
                cfg["pos_embed_max_size"], cfg["base_height"], True)
        vc = dit_forward(cond_pooled, cond_captions, x, t, *args)
        vu = dit_forward(uncond_pooled, uncond_captions, x, t, *args)
        x = x + (sig[i + 1] - sig[i]) * (vu + guidance * (vc - vu))
    return x
