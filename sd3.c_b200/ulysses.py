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

    # variants into preallocated (contiguous) outputs: chunk d of `send` goes to rank d,
    # chunk s of `out` comes from rank s
    def all_to_all_into(self, out, send):
        self.dist.all_to_all_single(out.reshape(-1), send.reshape(-1), group=self.group)

    def all_gather_into(self, out, t):
        self.dist.all_gather_into_tensor(out.reshape(-1), t.reshape(-1), group=self.group)

    def all_to_all_start(self, out, send):
        """all_to_all_into that returns at once with a handle: the exchange runs on the
        communicator's stream behind the work already queued on the current stream, and the
        current stream only waits for it at handle.wait().  Neither buffer may be touched
        between the two calls."""
        return self.dist.all_to_all_single(out.reshape(-1), send.reshape(-1), group=self.group, async_op=True)


class _Done:
    def wait(self):
        return True


class LocalComm:
    """The one-rank communicator: every exchange is a copy.  Lets the sharded forward run
    (and be tested) on a single GPU without a process group."""
    rank = 0
    world = 1

    def all_to_all(self, send):
        return send.clone()

    def all_gather(self, t):
        return t.unsqueeze(0).clone()

    def all_to_all_into(self, out, send):
        out.reshape(-1).copy_(send.reshape(-1))

    def all_gather_into(self, out, t):
        out.reshape(-1).copy_(t.reshape(-1))

    def all_to_all_start(self, out, send):
        out.reshape(-1).copy_(send.reshape(-1))
        return _Done()


# ---------------------------------------------------------------------------
# packed weights of one model, kept as torch tensors (device memory plumbing)
# ---------------------------------------------------------------------------
class PackedModel:
    """bf16 packed (out, in) weights for the op-level ABI, from the reference
    params dict (2-D weights (in, out); module_tests/DiT.py:25-31).

    Two things are prepared once per model so that the forward needs no glue:
    the AdaLN matrices of all blocks and of the final layer are concatenated
    (one GEMM with M = 1 yields every modulation vector of the step), and, once
    the rank is known (`for_rank`), the context QKV weights are sliced to the
    heads this rank owns (the context rows are replicated, so each rank projects
    them onto its own heads only)."""

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
        # all AdaLN vectors of the step from one GEMM: rows [off, off + n) per (layer, stream)
        L = cfg["num_layers"]
        ws, bs, self.ada_off, off = [], [], {}, 0
        names = []
        for l in range(L):
            names += ["transformer.%d.context_ada_lnorm.linear" % l, "transformer.%d.latent_ada_lnorm.linear" % l]
        names.append("ada_ln_out.linear")
        for n in names:
            w, b = self.w.pop(n + ".weight"), self.w.pop(n + ".bias")
            self.ada_off[n] = (off, w.shape[0])
            off += w.shape[0]
            ws.append(w)
            bs.append(b)
        self.ada_w = torch.cat(ws, 0).contiguous()
        self.ada_b = torch.cat(bs, 0).contiguous()
        self.ada_total = off
        # Bounds on the scores of each block's joint and image-only attention, from the q/k RMSNorm
        # weights.  Where a bound is small enough for the kernel's bounded softmax (exp2 arguments
        # of at most 80), the query norm weights are replaced by copies that carry
        # softmax_scale * log2(e): q leaves the QKV epilogue pre-scaled, the attention is called
        # with scale 0 and the bound in those units.  Otherwise (0.0, plain scale) nothing changes.
        self.score_bound = {}
        c = 1.4426950408889634 * (cfg["emb_dim"] // cfg["attn_heads"]) ** -0.5
        for l in range(L):
            pre = "transformer.%d." % l
            def names(kind, streams):
                return [pre + s_ + "_rmsnorm_" + kind + ".weight" for s_ in streams
                        if pre + s_ + "_rmsnorm_" + kind + ".weight" in self.w]
            def bound(qn, kn, want):
                if len(qn) != want or len(kn) != want:
                    return 0.0
                b = sd3.qk_norm_score_bound([self.w[n] for n in qn], [self.w[n] for n in kn]) * c
                if not 0.0 < b <= 80.0:
                    return 0.0
                for n in qn:
                    self.w[n] = (self.w[n] * c).contiguous()
                return b
            joint = bound(names("query", ("context", "latent")), names("key", ("context", "latent")), 2)
            dual = bound(names("query", ("latent_dual",)), names("key", ("latent_dual",)), 1)
            self.score_bound[l] = (joint, dual)
        self.local = None
        self.ws = {}
        torch.cuda.synchronize()

    def lin(self, name):
        return self.w[name + ".weight"], self.w[name + ".bias"]

    def for_rank(self, rank, P):
        """Context QKV weights restricted to the heads of `rank` (q, k and v rows of that
        head group), as (3 E/P, E) matrices."""
        if self.local is not None and self.local[0] == (rank, P):
            return self.local[1]
        torch = _torch()
        E = self.cfg["emb_dim"]
        Eh = E // P
        out = {}
        for l in range(self.cfg["num_layers"]):
            w, b = self.lin("transformer.%d.context_to_qkv" % l)
            rows = torch.cat([torch.arange(part * E + rank * Eh, part * E + (rank + 1) * Eh) for part in range(3)]).to(w.device)
            out[l] = (w.index_select(0, rows).contiguous(), b.index_select(0, rows).contiguous())
        self.local = ((rank, P), out)
        return out

    def buffers(self, Tc, Tl, P, dual_any):
        """Activation buffers of the sharded forward, allocated once per shape."""
        key = (Tc, Tl, P)
        if key in self.ws:
            return self.ws[key]
        torch = _torch()
        E = self.cfg["emb_dim"]
        F = E * self.cfg["mlp_expand"]
        Eh = E // P
        bf, dev = torch.bfloat16, "cuda"
        e = lambda *shape: torch.empty(shape, device=dev, dtype=bf)
        b = dict(h_c=e(Tc, E), h_x=e(Tl, E), h_x2=e(Tl, E), send=e(P, Tl, 3, Eh), att_in=e(1, Tc + P * Tl, 3 * Eh),
                 att2=e(1, P * Tl, 3 * Eh), o_c=e(1, Tc, Eh), o_x=e(1, P * Tl, Eh), recv_o=e(P, Tl, Eh),
                 send2=e(P, Tl, 3, Eh), o_x2=e(1, P * Tl, Eh), recv_o2=e(P, Tl, Eh),  # dual attention's own set
                 o_rows=e(Tl, E), gath_c=e(P, Tc, Eh), o_ctx=e(Tc, E), hid_x=e(Tl, F), hid_c=e(Tc, F),
                 mod=torch.empty((1, self.ada_total), device=dev, dtype=torch.float32))
        NHl = self.cfg["attn_heads"] // P
        sc1 = self.sd3.attention_scratch(1, Tc + P * Tl, NHl)
        sc2 = self.sd3.attention_scratch(1, P * Tl, NHl)
        b["attn_scratch"] = sc1 if (sc2 is None or (sc1 is not None and sc1.numel() >= sc2.numel())) else sc2
        self.ws[key] = b
        return b


def _gate_resid(sd3, x_bf16, w, b, gate_row, resid):
    """resid (rows, E) f32 += gate * (x W^T + b); one sample, so one gate row."""
    sd3.check(sd3.lib().sd3_linear_gate_residual(
        sd3.ptr(x_bf16), sd3.ptr(w), sd3.ptr(b), gate_row.data_ptr(), 0, resid.shape[0], sd3.ptr(resid),
        x_bf16.shape[0], w.shape[0], x_bf16.shape[1], sd3.stream_ptr()), "sd3_linear_gate_residual")


# The context rows' GEMMs ride in the launches of the image rows' GEMMs of the same kind
# (sd3_linear_pair, sd3_linear_gate_residual_pair); False launches them separately.
PAIR_LAUNCHES = True


def _gate_resid_pair(sd3, x0, w0, b0, gate0, resid0, x1, w1, b1, gate1, resid1):
    """Two gate+residual GEMMs of one shape class (image rows and context rows of a block) as
    one launch; one sample each, so one gate row each."""
    if not PAIR_LAUNCHES:
        _gate_resid(sd3, x0, w0, b0, gate0, resid0)
        _gate_resid(sd3, x1, w1, b1, gate1, resid1)
        return
    sd3.check(sd3.lib().sd3_linear_gate_residual_pair(
        sd3.ptr(x0), sd3.ptr(w0), sd3.ptr(b0), gate0.data_ptr(), resid0.shape[0], sd3.ptr(resid0), x0.shape[0],
        sd3.ptr(x1), sd3.ptr(w1), sd3.ptr(b1), gate1.data_ptr(), resid1.shape[0], sd3.ptr(resid1), x1.shape[0],
        0, w0.shape[0], x0.shape[1], sd3.stream_ptr()), "sd3_linear_gate_residual_pair")


def _linear_pair_into(sd3, x0, w0, b0, out0, x1, w1, b1, out1, act=0):
    if not PAIR_LAUNCHES:
        _linear_into(sd3, x0, w0, b0, out0, act=act)
        _linear_into(sd3, x1, w1, b1, out1, act=act)
        return
    sd3.check(sd3.lib().sd3_linear_pair(sd3.ptr(x0), sd3.ptr(w0), sd3.ptr(b0), sd3.ptr(out0), x0.shape[0],
                                        sd3.ptr(x1), sd3.ptr(w1), sd3.ptr(b1), sd3.ptr(out1), x1.shape[0],
                                        sd3.dtype_tag(out0), w0.shape[0], x0.shape[1], act, sd3.stream_ptr()),
              "sd3_linear_pair")


def _ln_mod(sd3, x, E, eps, shift, scale, out1, shift2=None, scale2=None, out2=None):
    """LayerNorm + modulate of (rows, E) f32 rows of one sample into preallocated bf16 outputs."""
    from ctypes import c_void_p
    sd3.check(sd3.lib().sd3_layernorm_modulate(
        sd3.ptr(x), 1, x.shape[0], E, eps, c_void_p(shift.data_ptr()), c_void_p(scale.data_ptr()), sd3.ptr(out1),
        c_void_p(shift2.data_ptr()) if shift2 is not None else None,
        c_void_p(scale2.data_ptr()) if scale2 is not None else None,
        sd3.ptr(out2) if shift2 is not None else None, 0, sd3.DTYPE_BF16, sd3.stream_ptr()), "sd3_layernorm_modulate")


def _linear_into(sd3, x, w, b, out, act=0):
    sd3.check(sd3.lib().sd3_linear(sd3.ptr(x), sd3.ptr(w), sd3.ptr(b), sd3.ptr(out), sd3.dtype_tag(out),
                                   x.shape[0], w.shape[0], x.shape[1], act, sd3.stream_ptr()), "sd3_linear")
    return out


def _attention_into(sd3, att_in, T, heads, Tc, scale, o_c, o_x, scratch=None, score_bound=0.0):
    """Attention over the local heads.  With few heads per rank a launch has too few CTAs for
    the GPU; the scratch buffer lets the kernel split the keys of each query tile.  score_bound:
    the block's bound on |q . k| (0.0 if unknown)."""
    sd3.check(sd3.lib().sd3_attention_bounded(sd3.ptr(att_in), 1, T, heads, Tc,
                                              sd3.ptr(o_c) if o_c is not None else None, sd3.ptr(o_x), scale,
                                              score_bound, sd3.ptr(scratch),
                                              scratch.numel() * scratch.element_size() if scratch is not None else 0,
                                              sd3.stream_ptr()), "sd3_attention_bounded")


def block_forward(pm, l, mod, c, x_loc, comm, last, dual):
    """One MMDiT(-X) block with the image rows sharded: c (Tc, E) f32 replicated,
    x_loc (Tl, E) f32 local rows; both updated in place.  mod: the (ada_total,) f32
    vector of all AdaLN outputs of the step.

    No tensor is re-laid between kernels: the image QKV GEMM writes the all-to-all send
    buffer (head-group layout) directly, the context rows are projected onto the local
    heads with a sliced weight straight into the attention input, the all-to-all delivers
    the image rows behind them in token order, and the attention output is already
    partitioned by destination rank.  The one copy left per attention turns the returned
    (source rank, row, head-group columns) slabs into (row, all columns) rows."""
    sd3 = pm.sd3
    cfg = pm.cfg
    E, NH = cfg["emb_dim"], cfg["attn_heads"]
    P, rank = comm.world, comm.rank
    Eh = E // P
    pre = "transformer.%d." % l
    Tc, Tl = c.shape[0], x_loc.shape[0]
    Tx = P * Tl
    scale = (E // NH) ** -0.5
    B = pm.buffers(Tc, Tl, P, True)
    ctx_local = pm.for_rank(rank, P)

    oc, nc = pm.ada_off[pre + "context_ada_lnorm.linear"]
    ox, nx = pm.ada_off[pre + "latent_ada_lnorm.linear"]
    cm, xm = mod[oc:oc + nc], mod[ox:ox + nx]
    ch = lambda v, i: v[i * E:(i + 1) * E]
    if last:
        c_scale_a, c_shift_a = ch(cm, 0), ch(cm, 1)
    else:
        c_shift_a, c_scale_a, c_gate_a, c_shift_m, c_scale_m, c_gate_m = (ch(cm, i) for i in range(6))
    x_shift_a, x_scale_a, x_gate_a, x_shift_m, x_scale_m, x_gate_m = (ch(xm, i) for i in range(6))

    _ln_mod(sd3, c, E, 1e-6, c_shift_a, c_scale_a, B["h_c"])
    if dual:
        _ln_mod(sd3, x_loc, E, 1e-6, x_shift_a, x_scale_a, B["h_x"], ch(xm, 6), ch(xm, 7), B["h_x2"])
    else:
        _ln_mod(sd3, x_loc, E, 1e-6, x_shift_a, x_scale_a, B["h_x"])

    def rms(n):
        return pm.w.get(pre + n + "_rmsnorm_query.weight"), pm.w.get(pre + n + "_rmsnorm_key.weight")

    # joint attention: context rows (my heads) | image rows of every rank (my heads)
    att_in = B["att_in"]
    w, b = pm.lin(pre + "latent_to_qkv")
    wq, wk = rms("latent")
    sd3.qkv_project_groups(B["h_x"], w, b, wq, wk, 1e-6, B["send"], E, P)
    jb, db = pm.score_bound[l]
    # The exchanges of a dual block are pipelined: each all-to-all runs on the communicator's
    # stream under the next kernel of the other attention (the image-only QKV under the first
    # exchange, the joint attention under the second, the image-only attention under the third,
    # the joint out-projection under the fourth).  A plain block has nothing to put under its
    # two exchanges but the small context projection.
    h_in = comm.all_to_all_start(att_in[0, Tc:], B["send"])
    h_in2 = None
    if dual:
        w, b = pm.lin(pre + "latent_dual_to_qkv")
        wq, wk = rms("latent_dual")
        sd3.qkv_project_groups(B["h_x2"], w, b, wq, wk, 1e-6, B["send2"], E, P)
        h_in2 = comm.all_to_all_start(B["att2"][0], B["send2"])
    wl, bl = ctx_local[l]
    wq, wk = rms("context")
    sd3.qkv_project_groups(B["h_c"], wl, bl, wq, wk, 1e-6, att_in, Eh, 1)  # rows [0, Tc) of att_in
    h_in.wait()
    _attention_into(sd3, att_in, Tc + Tx, NH // P, Tc, 0.0 if jb > 0.0 else scale, None if last else B["o_c"], B["o_x"],
                    B["attn_scratch"], jb)
    h_out = comm.all_to_all_start(B["recv_o"], B["o_x"])
    h_out2 = None
    if dual:  # image-only attention of the dual blocks
        h_in2.wait()
        _attention_into(sd3, B["att2"], Tx, NH // P, 0, 0.0 if db > 0.0 else scale, None, B["o_x2"], B["attn_scratch"], db)
        h_out2 = comm.all_to_all_start(B["recv_o2"], B["o_x2"])
    h_out.wait()
    B["o_rows"].view(Tl, P, Eh).copy_(B["recv_o"].permute(1, 0, 2))
    w, b = pm.lin(pre + "latent_attn_Wout")
    if not last:
        comm.all_gather_into(B["gath_c"], B["o_c"])
        B["o_ctx"].view(Tc, P, Eh).copy_(B["gath_c"].permute(1, 0, 2))
        wc_, bc_ = pm.lin(pre + "context_attn_Wout")
        # the replicated context rows ride in the tail of the image rows' launch
        _gate_resid_pair(sd3, B["o_rows"], w, b, x_gate_a, x_loc, B["o_ctx"], wc_, bc_, c_gate_a, c)
    else:
        _gate_resid(sd3, B["o_rows"], w, b, x_gate_a, x_loc)
    if dual:
        h_out2.wait()
        B["o_rows"].view(Tl, P, Eh).copy_(B["recv_o2"].permute(1, 0, 2))
        w, b = pm.lin(pre + "latent_dual_attn_Wout")
        _gate_resid(sd3, B["o_rows"], w, b, ch(xm, 8), x_loc)

    _ln_mod(sd3, x_loc, E, 1e-6, x_shift_m, x_scale_m, B["h_x"])
    w1, b1 = pm.lin(pre + "latent_mlp.lin1")
    w2, b2 = pm.lin(pre + "latent_mlp.lin2")
    if not last:  # both streams' MLPs: each linear of the pair as one launch
        _ln_mod(sd3, c, E, 1e-6, c_shift_m, c_scale_m, B["h_c"])
        wc1, bc1 = pm.lin(pre + "context_mlp.lin1")
        wc2, bc2 = pm.lin(pre + "context_mlp.lin2")
        _linear_pair_into(sd3, B["h_x"], w1, b1, B["hid_x"], B["h_c"], wc1, bc1, B["hid_c"], act=sd3.ACT_GELU_TANH)
        _gate_resid_pair(sd3, B["hid_x"], w2, b2, x_gate_m, x_loc, B["hid_c"], wc2, bc2, c_gate_m, c)
    else:
        _linear_into(sd3, B["h_x"], w1, b1, B["hid_x"], act=sd3.ACT_GELU_TANH)
        _gate_resid(sd3, B["hid_x"], w2, b2, x_gate_m, x_loc)


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
    if Tx % P or NH % P or hp % P:
        raise sd3.Sd3Error("image rows (%d), tokens (%d) and heads (%d) must divide by the number of ranks (%d)"
                           % (hp, Tx, NH, P))
    Tl = Tx // P
    Tc = captions.shape[1]
    bufs = pm.buffers(Tc, Tl, P, True)
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
    # every AdaLN vector of the step from one GEMM with M = 1 over the concatenated matrices
    if pm.ada_total % 64 == 0 and E % 64 == 0:
        _linear_into(sd3, sd3.cast(y, torch.bfloat16), pm.ada_w, pm.ada_b, bufs["mod"])
        mod = bufs["mod"][0]
    else:
        mod = sd3.skinny_linear(y, pm.ada_w, pm.ada_b)[0]
    # context stream (replicated) and the local rows of the image stream: rank r owns the
    # patch rows [r * hp / P, (r + 1) * hp / P), i.e. a contiguous block of latent rows
    w, b = pm.lin("captions_linear")
    c = sd3.linear(captions[0].to(torch.bfloat16).contiguous(), w, b, out_dtype=torch.float32)
    pos = sd3.pos_embed_table(hp, wp, E, cfg["pos_embed_max_size"], cfg["base_height"] // p)
    hl = hp // P
    lat_loc = latent[:, :, rank * hl * p:(rank + 1) * hl * p, :].to(torch.bfloat16).contiguous()
    w, b = pm.lin("to_patch.conv")
    x_loc = sd3.patch_embed(lat_loc, w, b, pos[rank * Tl:(rank + 1) * Tl].contiguous(), p, E)
    dual = set(int(l) for l in cfg["dual_attention_layers"])
    L = cfg["num_layers"]
    for l in range(L):
        last = l == L - 1
        block_forward(pm, l, mod, c, x_loc, comm, last, (l in dual) and not last)
    # final layer on the local rows, then gather the rows and undo the patching
    off, n = pm.ada_off["ada_ln_out.linear"]
    fm = mod[off:off + n]
    _ln_mod(sd3, x_loc, E, 1e-5, fm[E:2 * E], fm[0:E], bufs["h_x"])
    w, b = pm.lin("linear_out")
    o_loc = sd3.linear(bufs["h_x"], w, b, out_dtype=torch.float32)  # (Tl, p*p*C)
    o = comm.all_gather(o_loc).reshape(Tx, p * p * C)               # rank-major == token order
    o = o.view(1, hp, wp, p, p, C)
    o = torch.einsum("bhwpqc->bchpwq", o).reshape(1, C, H, W).contiguous()
    return o
