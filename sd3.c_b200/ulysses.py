"""Ulysses-style sequence parallelism for ONE long image sequence (batch 1):
the image tokens are split into contiguous row blocks across P ranks, every
token-local operator (LayerNorm+modulate, QKV / out-proj / MLP GEMMs) runs on
the local rows only, and around each attention an all-to-all turns
"my tokens x all heads" into "all tokens x my heads" and back.  The 333
context tokens are replicated on every rank (their linear work is ~2 % of the
image stream's), so only their attention output needs an all-gather over heads.

All arithmetic goes through the library's C ABI (sd3_b200.py); this file only
orchestrates launches, re-lays tensors for the exchange and calls
torch.distributed (NCCL over NVLink on GPUs; the layout helpers are plain
tensor code and are also exercised on CPU with emulated ranks).  Received
data always lands in local memory first and is then read by local kernels.

The reference has no distributed code at all; the math per block is
MM_DiT_Block.forward (module_tests/modules.py:255-355).
"""
import os


def _torch():
    import torch
    return torch


# ---------------------------------------------------------------------------
# layout helpers (pure tensor code; no communication)
# ---------------------------------------------------------------------------
def split_heads_for_send(qkv_rows, P):
    """(Tl, 3E) local image rows with q|k|v column blocks -> (P, Tl, 3, E/P):
    slab d holds the q, k and v columns of the heads owned by rank d."""
    Tl, threeE = qkv_rows.shape
    E = threeE // 3
    return qkv_rows.view(Tl, 3, P, E // P).permute(2, 0, 1, 3).contiguous()


def assemble_attention_input(ctx_qkv, recv, rank, P):
    """ctx_qkv (Tc, 3E): replicated context rows (all heads); recv (P, Tl, 3, E/P):
    slab s = image rows of rank s, my heads.  Returns (1, Tc + P*Tl, 3E/P) packed
    q|k|v for the local heads, context rows first."""
    torch = _torch()
    Tc, threeE = ctx_qkv.shape
    E = threeE // 3
    Eh = E // P
    ctx = ctx_qkv.view(Tc, 3, P, Eh)[:, :, rank, :]  # (Tc, 3, Eh)
    img = recv.reshape(-1, 3, Eh)                   # (P*Tl, 3, Eh), rank-major == token order
    return torch.cat([ctx, img], 0).reshape(1, -1, 3 * Eh).contiguous()


def split_tokens_for_send(o_x, P):
    """(Tx, E/P) attention output for my heads over all image rows -> (P, Tl, E/P)."""
    Tx, Eh = o_x.shape
    return o_x.view(P, Tx // P, Eh).contiguous()


def assemble_rows(recv):
    """(P, Tl, E/P): slab s = my rows, heads of rank s -> (Tl, E)."""
    P, Tl, Eh = recv.shape
    return recv.permute(1, 0, 2).reshape(Tl, P * Eh).contiguous()


# ---------------------------------------------------------------------------
# communicator abstraction: torch.distributed, or emulated ranks for CPU tests
# ---------------------------------------------------------------------------
class DistComm:
    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)

    def all_to_all(self, send):
        out = _torch().empty_like(send)
        self.dist.all_to_all_single(out, send, group=self.group)
        return out

    def all_gather(self, t):
        out = _torch().empty((self.world,) + tuple(t.shape), device=t.device, dtype=t.dtype)
        self.dist.all_gather_into_tensor(out, t.contiguous(), group=self.group)
        return out


# ---------------------------------------------------------------------------
# packed weights of one model, kept as torch tensors (device memory plumbing)
# ---------------------------------------------------------------------------
class PackedModel:
    """bf16 packed (out, in) weights for the op-level ABI, from the reference
    params dict (2-D weights (in, out); module_tests/DiT.py:25-31)."""

    def __init__(self, sd3, params, cfg):
        torch = _torch()
        self.sd3 = sd3
        self.cfg = dict(cfg)
        self.w = {}
        for name, t in params.items():
            t = t.cuda().contiguous()
            if t.dim() == 2:
                self.w[name] = sd3.pack_weight(t, torch.bfloat16)
            elif t.dim() == 4:
                self.w[name] = t.reshape(t.shape[0], -1).to(torch.bfloat16).contiguous()
            else:
                self.w[name] = t.to(torch.float32).contiguous()
        torch.cuda.synchronize()

    def lin(self, name):
        return self.w[name + ".weight"], self.w[name + ".bias"]


def _gate_resid(sd3, x_bf16, w, b, gate_row, resid):
    """resid (rows, E) f32 += gate * (x W^T + b); one sample, so one gate row."""
    sd3.check(sd3.lib().sd3_linear_gate_residual(
        sd3.ptr(x_bf16), sd3.ptr(w), sd3.ptr(b), gate_row.data_ptr(), 0, resid.shape[0], sd3.ptr(resid),
        x_bf16.shape[0], w.shape[0], x_bf16.shape[1], sd3.stream_ptr()), "sd3_linear_gate_residual")


def _ln_mod(sd3, x, E, eps, shift, scale, shift2=None, scale2=None):
    return sd3.layernorm_modulate(x, 1, x.shape[0], E, eps, shift, scale, shift2, scale2, mod_stride=0)


def block_forward(pm, l, y, c, x_loc, comm, last, dual):
    """One MMDiT(-X) block with the image rows sharded: c (Tc, E) f32 replicated,
    x_loc (Tl, E) f32 local rows; both updated in place."""
    torch = _torch()
    sd3 = pm.sd3
    cfg = pm.cfg
    E, NH = cfg["emb_dim"], cfg["attn_heads"]
    P, rank = comm.world, comm.rank
    Eh = E // P
    pre = "transformer.%d." % l
    Tc, Tl = c.shape[0], x_loc.shape[0]
    scale = (E // NH) ** -0.5

    wa, ba = pm.lin(pre + "context_ada_lnorm.linear")
    cm = sd3.skinny_linear(y, wa, ba)[0]
    wa, ba = pm.lin(pre + "latent_ada_lnorm.linear")
    xm = sd3.skinny_linear(y, wa, ba)[0]
    ch = lambda v, i: v[i * E:(i + 1) * E]
    if last:
        c_scale_a, c_shift_a = ch(cm, 0), ch(cm, 1)
    else:
        c_shift_a, c_scale_a, c_gate_a, c_shift_m, c_scale_m, c_gate_m = (ch(cm, i) for i in range(6))
    x_shift_a, x_scale_a, x_gate_a, x_shift_m, x_scale_m, x_gate_m = (ch(xm, i) for i in range(6))

    h_c, _ = _ln_mod(sd3, c, E, 1e-6, c_shift_a, c_scale_a)
    if dual:
        h_x, h_x2 = _ln_mod(sd3, x_loc, E, 1e-6, x_shift_a, x_scale_a, ch(xm, 6), ch(xm, 7))
    else:
        h_x, h_x2 = _ln_mod(sd3, x_loc, E, 1e-6, x_shift_a, x_scale_a)

    def rms(n):
        return pm.w.get(pre + n + "_rmsnorm_query.weight"), pm.w.get(pre + n + "_rmsnorm_key.weight")

    # local QKV (context rows first), then tokens x all heads -> all tokens x my heads
    qkv = torch.empty((1, Tc + Tl, 3 * E), device=c.device, dtype=torch.bfloat16)
    w, b = pm.lin(pre + "context_to_qkv")
    wq, wk = rms("context")
    sd3.qkv_project(h_c, w, b, wq, wk, 1e-6, qkv, 1, Tc, Tc + Tl, 0, E)
    w, b = pm.lin(pre + "latent_to_qkv")
    wq, wk = rms("latent")
    sd3.qkv_project(h_x, w, b, wq, wk, 1e-6, qkv, 1, Tl, Tc + Tl, Tc, E)
    recv = comm.all_to_all(split_heads_for_send(qkv[0, Tc:], P))
    att_in = assemble_attention_input(qkv[0, :Tc], recv, rank, P)
    o_c, o_x = sd3.attention(att_in, 1, Tc + P * Tl, NH // P, Tc, scale, want_context=not last)
    o_rows = assemble_rows(comm.all_to_all(split_tokens_for_send(o_x[0], P)))
    if not last:
        o_ctx = assemble_rows(comm.all_gather(o_c[0]))  # (P, Tc, Eh) -> (Tc, E)
        w, b = pm.lin(pre + "context_attn_Wout")
        _gate_resid(sd3, o_ctx, w, b, c_gate_a, c)
    w, b = pm.lin(pre + "latent_attn_Wout")
    _gate_resid(sd3, o_rows, w, b, x_gate_a, x_loc)

    if dual:
        qkv2 = torch.empty((1, Tl, 3 * E), device=c.device, dtype=torch.bfloat16)
        w, b = pm.lin(pre + "latent_dual_to_qkv")
        wq, wk = rms("latent_dual")
        sd3.qkv_project(h_x2, w, b, wq, wk, 1e-6, qkv2, 1, Tl, Tl, 0, E)
        recv = comm.all_to_all(split_heads_for_send(qkv2[0], P))
        att_in = recv.reshape(1, P * Tl, 3 * Eh).contiguous()
        _, o_x = sd3.attention(att_in, 1, P * Tl, NH // P, 0, scale)
        o_rows = assemble_rows(comm.all_to_all(split_tokens_for_send(o_x[0], P)))
        w, b = pm.lin(pre + "latent_dual_attn_Wout")
        _gate_resid(sd3, o_rows, w, b, ch(xm, 8), x_loc)

    h_x, _ = _ln_mod(sd3, x_loc, E, 1e-6, x_shift_m, x_scale_m)
    w, b = pm.lin(pre + "latent_mlp.lin1")
    hid = sd3.linear(h_x, w, b, act=sd3.ACT_GELU_TANH)
    w, b = pm.lin(pre + "latent_mlp.lin2")
    _gate_resid(sd3, hid, w, b, x_gate_m, x_loc)
    if not last:
        h_c, _ = _ln_mod(sd3, c, E, 1e-6, c_shift_m, c_scale_m)
        w, b = pm.lin(pre + "context_mlp.lin1")
        hid = sd3.linear(h_c, w, b, act=sd3.ACT_GELU_TANH)
        w, b = pm.lin(pre + "context_mlp.lin2")
        _gate_resid(sd3, hid, w, b, c_gate_m, c)


def dit_forward_sharded(pm, pooled, captions, latent, timesteps, comm):
    """Full denoiser forward for ONE sample (batch 1) with the image tokens
    sharded over comm.world ranks.  Inputs are the full (replicated) tensors in
    bf16; returns the full (1, C, H, W) float32 output on every rank.
    Math: MMDiT.forward (module_tests/modules.py:397-425)."""
    torch = _torch()
    sd3 = pm.sd3
    cfg = pm.cfg
    E, NH, p = cfg["emb_dim"], cfg["attn_heads"], cfg["patch_size"]
    P, rank = comm.world, comm.rank
    B, C, H, W = latent.shape
    if B != 1:
        raise sd3.Sd3Error("sequence sharding handles one sample at a time")
    hp, wp = H // p, W // p
    Tx = hp * wp
    if Tx % P or NH % P:
        raise sd3.Sd3Error("image tokens (%d) and heads (%d) must divide by the number of ranks (%d)" % (Tx, NH, P))
    Tl = Tx // P
    # conditioning vector (replicated)
    emb = sd3.sinusoidal_embedding(timesteps.float().contiguous(), 256)
    w, b = pm.lin("timestep_mlp.0")
    th = sd3.skinny_linear(emb, w, b, None, act=1)
    w, b = pm.lin("timestep_mlp.2")
    tout = sd3.skinny_linear(th, w, b)
    w, b = pm.lin("pooled_mlp.0")
    ph = sd3.skinny_linear(pooled.float().contiguous(), w, b, None, act=1)
    w, b = pm.lin("pooled_mlp.2")
    y = sd3.skinny_linear(ph, w, b, tout, act=1)
    # context stream (replicated) and the local slice of the image stream
    w, b = pm.lin("captions_linear")
    c = sd3.linear(captions[0].to(torch.bfloat16).contiguous(), w, b, out_dtype=torch.float32)
    pos = sd3.pos_embed_table(hp, wp, E, cfg["pos_embed_max_size"], cfg["base_height"] // p)
    w, b = pm.lin("to_patch.conv")
    x_full = sd3.patch_embed(latent.to(torch.bfloat16).contiguous(), w, b, pos, p, E)
    x_loc = x_full[rank * Tl:(rank + 1) * Tl].contiguous()
    del x_full
    dual = set(int(l) for l in cfg["dual_attention_layers"])
    L = cfg["num_layers"]
    for l in range(L):
        last = l == L - 1
        block_forward(pm, l, y, c, x_loc, comm, last, (l in dual) and not last)
    # final layer on the local rows, then gather the rows and undo the patching
    w, b = pm.lin("ada_ln_out.linear")
    fm = sd3.skinny_linear(y, w, b)[0]
    h, _ = sd3.layernorm_modulate(x_loc, 1, Tl, E, 1e-5, fm[E:2 * E], fm[0:E], mod_stride=0)
    w, b = pm.lin("linear_out")
    o_loc = sd3.linear(h, w, b, out_dtype=torch.float32)          # (Tl, p*p*C)
    o = comm.all_gather(o_loc).reshape(Tx, p * p * C)             # rank-major == token order
    o = o.view(1, hp, wp, p, p, C)
    o = torch.einsum("bhwpqc->bchpwq", o).reshape(1, C, H, W).contiguous()
    return o
