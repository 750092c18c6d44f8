"""ctypes binding of libsd3_b200.so plus torch-tensor conveniences.

PyTorch is used here for device memory and streams only; every computation
goes through the C ABI declared in include/sd3_b200.h.  There is no CPU or
PyTorch fallback: if the library is missing or a call fails, an exception is
raised.

The directory name of this package contains a dot, so it is loaded by path:

    import importlib.util, os
    spec = importlib.util.spec_from_file_location(
        "sd3_b200", os.path.join(repo, "sd3.c_b200", "sd3_b200.py"))
"""
import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_long, c_uint64, c_void_p, POINTER

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("SD3_B200_LIB") or os.path.join(HERE, "libsd3_b200.so")

DTYPE_F32 = 0
DTYPE_BF16 = 1
PRECISION_BF16 = 0
PRECISION_F32 = 1
PRECISION_FP8 = 2
ACT_NONE = 0
ACT_GELU_TANH = 1


class Sd3Error(RuntimeError):
    pass


class Config(ctypes.Structure):
    _fields_ = [
        ("num_layers", c_int),
        ("dual_attention_mask", c_uint64),
        ("pooled_dim", c_int),
        ("captions_dim", c_int),
        ("in_channels", c_int),
        ("emb_dim", c_int),
        ("attn_heads", c_int),
        ("mlp_expand", c_int),
        ("patch_size", c_int),
        ("pos_embed_max_size", c_int),
        ("base_height", c_int),
        ("use_qk_norm", c_int),
        ("last_discards_context", c_int),
        ("precision", c_int),
        ("block_only", c_int),
    ]


# name -> (restype, argtypes); must list every function include/sd3_b200.h declares
PROTOTYPES = {
    "sd3_abi_version": (c_int, []),
    "sd3_last_error": (c_char_p, []),
    "sd3_device_status": (c_int, [POINTER(c_int)]),
    "sd3_linear": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "sd3_linear_f32": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "sd3_linear_e4m3": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p]),
    "sd3_quantize_e4m3": (c_int, [c_void_p, c_int, c_void_p, c_long, c_float, c_void_p]),
    "sd3_linear_gate_residual": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_int, c_void_p, c_int, c_int, c_int, c_void_p]),
    "sd3_qkv_project": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "sd3_linear_pair": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "sd3_linear_gate_residual_pair": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_long, c_int, c_int, c_void_p]),
    "sd3_qkv_project_groups": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "sd3_attention": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p]),
    "sd3_attention_scratch_bytes": (c_long, [c_int, c_int, c_int]),
    "sd3_attention_ws": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p, c_long, c_void_p]),
    "sd3_attention_bounded": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_float, c_void_p, c_long, c_void_p]),
    "sd3_attention_generic": (c_int, [c_void_p, c_void_p, c_void_p, c_long, c_int, c_int, c_int, c_int, c_int, c_void_p, c_long, c_int, c_float, c_void_p]),
    "sd3_cross_attention": (c_int, [c_void_p, c_void_p, c_void_p, c_long, c_long, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_long, c_int, c_float, c_void_p]),
    "sd3_conv2d": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "sd3_layernorm_modulate": (c_int, [c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_int, c_void_p]),
    "sd3_skinny_linear": (c_int, [c_void_p, c_long, c_void_p, c_int, c_void_p, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int, c_int, c_void_p]),
    "sd3_sinusoidal_embedding": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "sd3_pos_embed_table": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "sd3_patch_embed": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "sd3_patch_embed_static": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "sd3_pack_weight": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p]),
    "sd3_cast": (c_int, [c_void_p, c_int, c_void_p, c_int, c_long, c_void_p]),
    "sd3_rmsnorm_heads": (c_int, [c_void_p, c_int, c_long, c_long, c_int, c_int, c_int, c_void_p, c_float, c_void_p]),
    "sd3_model_create": (c_int, [POINTER(Config), POINTER(c_void_p)]),
    "sd3_model_destroy": (None, [c_void_p]),
    "sd3_model_set_param": (c_int, [c_void_p, c_char_p, c_void_p, c_int, c_int, POINTER(c_int64), c_void_p]),
    "sd3_model_finalize": (c_int, [c_void_p, POINTER(c_int)]),
    "sd3_model_reserve": (c_int, [c_void_p, c_int, c_int, c_int, c_int]),
    "sd3_dit_forward": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "sd3_block_forward": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "sd3_cfg_euler_step": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_long, c_float, c_float, c_void_p]),
    "sd3_launch_count": (c_long, [c_int]),
    "sd3_selftest_wait_timeout": (c_int, [c_int, c_void_p]),
}

_lib = None


def lib():
    """Loads the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise Sd3Error(
                "libsd3_b200.so not found at %s: run `python sd3.c_b200/build.py` "
                "(there is no fallback path)" % LIB_PATH)
        l = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(l, name)
            fn.restype = res
            fn.argtypes = args
        _lib = l
    return _lib


def check(rc, what=""):
    if rc != 0:
        msg = lib().sd3_last_error()
        raise Sd3Error("%s failed (%d): %s" % (what or "sd3 call", rc, (msg or b"").decode()))


def device_status():
    st = c_int(0)
    check(lib().sd3_device_status(ctypes.byref(st)), "sd3_device_status")
    return st.value


def assert_healthy():
    st = device_status()
    if st != 0:
        raise Sd3Error("device status %d: a kernel gave up a bounded wait" % st)


# ---------------------------------------------------------------------------
# torch helpers
# ---------------------------------------------------------------------------
def _torch():
    import torch
    return torch


def dtype_tag(t):
    torch = _torch()
    if t.dtype == torch.float32:
        return DTYPE_F32
    if t.dtype == torch.bfloat16:
        return DTYPE_BF16
    raise Sd3Error("unsupported dtype %s (float32 or bfloat16 expected)" % t.dtype)


def ptr(t):
    if t is None:
        return None
    if not t.is_cuda:
        raise Sd3Error("CUDA tensor expected")
    if not t.is_contiguous():
        raise Sd3Error("contiguous tensor expected")
    return c_void_p(t.data_ptr())


def stream_ptr():
    return c_void_p(_torch().cuda.current_stream().cuda_stream)


def pack_weight(w_in_out, out_dtype=None):
    """(in, out) boundary weight -> packed (out, in) tensor of out_dtype (default bf16)."""
    torch = _torch()
    out_dtype = out_dtype or torch.bfloat16
    K, N = w_in_out.shape
    out = torch.empty((N, K), device=w_in_out.device, dtype=out_dtype)
    check(lib().sd3_pack_weight(ptr(w_in_out), dtype_tag(w_in_out), ptr(out), dtype_tag(out), K, N,
                                stream_ptr()), "sd3_pack_weight")
    return out


def cast(t, dtype):
    torch = _torch()
    out = torch.empty(t.shape, device=t.device, dtype=dtype)
    check(lib().sd3_cast(ptr(t), dtype_tag(t), ptr(out), dtype_tag(out), t.numel(), stream_ptr()),
          "sd3_cast")
    return out


def linear(x_bf16, w_nk_bf16, bias=None, act=ACT_NONE, out_dtype=None):
    torch = _torch()
    M, K = x_bf16.shape
    N = w_nk_bf16.shape[0]
    out = torch.empty((M, N), device=x_bf16.device, dtype=out_dtype or torch.bfloat16)
    check(lib().sd3_linear(ptr(x_bf16), ptr(w_nk_bf16), ptr(bias), ptr(out), dtype_tag(out), M, N, K,
                           act, stream_ptr()), "sd3_linear")
    return out


def linear_f32(x, w_nk, bias=None, act=ACT_NONE):
    torch = _torch()
    M, K = x.shape
    N = w_nk.shape[0]
    out = torch.empty((M, N), device=x.device, dtype=torch.float32)
    check(lib().sd3_linear_f32(ptr(x), ptr(w_nk), ptr(bias), ptr(out), M, N, K, act, stream_ptr()),
          "sd3_linear_f32")
    return out


def linear_gate_residual(x_bf16, w_nk_bf16, bias, gate, rows_per_sample, resid):
    M, K = x_bf16.shape
    N = w_nk_bf16.shape[0]
    check(lib().sd3_linear_gate_residual(ptr(x_bf16), ptr(w_nk_bf16), ptr(bias), ptr(gate),
                                         gate.stride(0), rows_per_sample, ptr(resid), M, N, K,
                                         stream_ptr()), "sd3_linear_gate_residual")
    return resid


def qkv_project(x_bf16, w_nk_bf16, bias, wq, wk, eps, qkv_out, B, T_in, T_total, row_offset, E):
    check(lib().sd3_qkv_project(ptr(x_bf16), ptr(w_nk_bf16), ptr(bias), ptr(wq), ptr(wk), eps,
                                ptr(qkv_out), B, T_in, T_total, row_offset, E, stream_ptr()),
          "sd3_qkv_project")
    return qkv_out


def qkv_project_groups(x_bf16, w_nk_bf16, bias, wq, wk, eps, out, E_out, head_groups):
    """out (head_groups, rows, 3, E_out/head_groups) bf16: see sd3_qkv_project_groups."""
    rows, K = x_bf16.shape
    check(lib().sd3_qkv_project_groups(ptr(x_bf16), ptr(w_nk_bf16), ptr(bias), ptr(wq), ptr(wk), eps, ptr(out),
                                       rows, E_out, K, head_groups, stream_ptr()), "sd3_qkv_project_groups")
    return out


def qk_norm_score_bound(wq, wk, head_dim=64):
    """Upper bound on |q . k| after the per-head RMSNorm with weights wq, wk (tensors, or lists of
    tensors when several norms feed one attention): a normed head vector is x_hat * w with
    |x_hat|^2 <= head_dim, so |q . k| <= head_dim * max_d |wq_d wk_d| (element-wise maxima over
    the listed weights); 1 % on top for the bf16 rounding of q and k."""
    torch = _torch()
    def absmax(w):
        ws = w if isinstance(w, (list, tuple)) else [w]
        return torch.stack([t.detach().float().abs().reshape(-1) for t in ws]).amax(0)
    return 1.01 * head_dim * float((absmax(wq) * absmax(wk)).max())


def attention(qkv_bf16, B, T, num_heads, Tc, scale, want_context=True, scratch=None, score_bound=0.0):
    """scratch: optional uint8/float tensor of sd3_attention_scratch_bytes(B, T, num_heads) bytes;
    with it, shapes that would not fill the GPU split the keys over several CTAs.
    score_bound: optional upper bound on |q . k| (see qk_norm_score_bound, sd3_attention_bounded)."""
    torch = _torch()
    E = num_heads * 64
    out_c = torch.empty((B, Tc, E), device=qkv_bf16.device, dtype=torch.bfloat16) if (want_context and Tc > 0) else None
    out_x = torch.empty((B, T - Tc, E), device=qkv_bf16.device, dtype=torch.bfloat16)
    if score_bound > 0.0:
        nbytes = scratch.numel() * scratch.element_size() if scratch is not None else 0
        check(lib().sd3_attention_bounded(ptr(qkv_bf16), B, T, num_heads, Tc, ptr(out_c), ptr(out_x), scale,
                                          score_bound, ptr(scratch), nbytes, stream_ptr()), "sd3_attention_bounded")
    elif scratch is None:
        check(lib().sd3_attention(ptr(qkv_bf16), B, T, num_heads, Tc, ptr(out_c), ptr(out_x), scale,
                                  stream_ptr()), "sd3_attention")
    else:
        check(lib().sd3_attention_ws(ptr(qkv_bf16), B, T, num_heads, Tc, ptr(out_c), ptr(out_x), scale,
                                     ptr(scratch), scratch.numel() * scratch.element_size(), stream_ptr()),
              "sd3_attention_ws")
    return out_c, out_x


def attention_scratch(B, T, num_heads, device="cuda"):
    """Scratch tensor for attention(..., scratch=...) / sd3_attention_ws, or None if this shape
    fills the GPU without a key split."""
    n = lib().sd3_attention_scratch_bytes(B, T, num_heads)
    return _torch().empty(n, device=device, dtype=_torch().uint8) if n > 0 else None


def attention_generic(q, k, v, num_heads, scale=None, out_dtype=None):
    torch = _torch()
    B, T, C = q.shape
    D = C // num_heads
    scale = scale if scale is not None else D ** -0.5
    out = torch.empty((B, T, C), device=q.device, dtype=out_dtype or q.dtype)
    check(lib().sd3_attention_generic(ptr(q), ptr(k), ptr(v), C, dtype_tag(q), B, T, num_heads, D,
                                      ptr(out), C, dtype_tag(out), scale, stream_ptr()),
          "sd3_attention_generic")
    return out


def layernorm_modulate(x, B, T, E, eps, shift1, scale1, shift2=None, scale2=None, mod_stride=None,
                       out_dtype=None):
    torch = _torch()
    out_dtype = out_dtype or torch.bfloat16
    out1 = torch.empty((B * T, E), device=x.device, dtype=out_dtype)
    out2 = torch.empty((B * T, E), device=x.device, dtype=out_dtype) if shift2 is not None else None
    ms = mod_stride if mod_stride is not None else shift1.stride(0)
    check(lib().sd3_layernorm_modulate(ptr(x), B, T, E, eps, c_void_p(shift1.data_ptr()),
                                       c_void_p(scale1.data_ptr()), ptr(out1),
                                       c_void_p(shift2.data_ptr()) if shift2 is not None else None,
                                       c_void_p(scale2.data_ptr()) if scale2 is not None else None,
                                       ptr(out2), ms, dtype_tag(out1), stream_ptr()),
          "sd3_layernorm_modulate")
    return out1, out2


def skinny_linear(inp, w_nk, bias=None, add=None, act=0):
    torch = _torch()
    B, K = inp.shape
    N = w_nk.shape[0]
    out = torch.empty((B, N), device=inp.device, dtype=torch.float32)
    check(lib().sd3_skinny_linear(ptr(inp), K, ptr(w_nk), dtype_tag(w_nk), ptr(bias), ptr(add),
                                  N if add is not None else 0, ptr(out), N, B, N, K, act,
                                  stream_ptr()), "sd3_skinny_linear")
    return out


def sinusoidal_embedding(t, dim):
    torch = _torch()
    out = torch.empty((t.shape[0], dim), device=t.device, dtype=torch.float32)
    check(lib().sd3_sinusoidal_embedding(ptr(t), ptr(out), t.shape[0], dim, stream_ptr()),
          "sd3_sinusoidal_embedding")
    return out


def pos_embed_table(h, w, E, pos_max, base_size, device="cuda"):
    torch = _torch()
    out = torch.empty((h * w, E), device=device, dtype=torch.float32)
    check(lib().sd3_pos_embed_table(ptr(out), h, w, E, pos_max, base_size, stream_ptr()),
          "sd3_pos_embed_table")
    return out


def patch_embed(latent, w_nk_bf16, bias, pos_table, patch, E):
    torch = _torch()
    B, C, H, W = latent.shape
    hp, wp = H // patch, W // patch
    out = torch.empty((B * hp * wp, E), device=latent.device, dtype=torch.float32)
    scratch = torch.empty((B * hp * wp, C * patch * patch), device=latent.device, dtype=torch.bfloat16)
    check(lib().sd3_patch_embed(ptr(latent), dtype_tag(latent), ptr(w_nk_bf16), ptr(bias),
                                ptr(pos_table), ptr(out), ptr(scratch), B, C, H, W, patch, E,
                                stream_ptr()), "sd3_patch_embed")
    return out


STATIC_PATCH_ELEMS = 4 * 1024 * 1024


def patch_embed_static(latent, w_nk_bf16, bias, pos_table, patch, E, out=None):
    """sd3_patch_embed_static: same result as patch_embed, scratch inside the library.
    `out` may be preallocated so that the call itself allocates nothing at all."""
    torch = _torch()
    B, C, H, W = latent.shape
    hp, wp = H // patch, W // patch
    if out is None:
        out = torch.empty((B * hp * wp, E), device=latent.device, dtype=torch.float32)
    # the C side only sees pointers: shapes, dtypes and devices are checked here
    if (out.dtype != torch.float32 or out.numel() != B * hp * wp * E or not out.is_contiguous()
            or out.device != latent.device):
        raise Sd3Error("patch_embed_static: out must be a contiguous float32 tensor of %d elements on %s"
                       % (B * hp * wp * E, latent.device))
    if tuple(w_nk_bf16.shape) != (E, C * patch * patch) or w_nk_bf16.dtype != torch.bfloat16:
        raise Sd3Error("patch_embed_static: weight must be bfloat16 of shape (%d, %d)" % (E, C * patch * patch))
    if tuple(pos_table.shape) != (hp * wp, E) or pos_table.dtype != torch.float32:
        raise Sd3Error("patch_embed_static: pos_table must be float32 of shape (%d, %d)" % (hp * wp, E))
    if bias is not None and (bias.numel() != E or bias.dtype != torch.float32):
        raise Sd3Error("patch_embed_static: bias must be float32 with %d elements" % E)
    check(lib().sd3_patch_embed_static(ptr(latent), dtype_tag(latent), ptr(w_nk_bf16), ptr(bias),
                                       ptr(pos_table), ptr(out), B, C, H, W, patch, E,
                                       stream_ptr()), "sd3_patch_embed_static")
    return out


def rmsnorm_heads(x, col0, nheads, head_dim, w, eps):
    rows = x.numel() // x.shape[-1]
    check(lib().sd3_rmsnorm_heads(ptr(x), dtype_tag(x), x.shape[-1], rows, col0, nheads, head_dim,
                                  ptr(w), eps, stream_ptr()), "sd3_rmsnorm_heads")
    return x


# ---------------------------------------------------------------------------
# model-level wrapper
# ---------------------------------------------------------------------------
class Model:
    """Owns an sd3_model handle.  `params` follows the reference convention:
    named_parameters() keys, 2-D weights transposed to (in, out)
    (module_tests/DiT.py:25-31)."""

    def __init__(self, num_layers, dual_attention_layers, pooled_dim, captions_dim, in_channels,
                 emb_dim, attn_heads, mlp_expand, patch_size, pos_embed_max_size, base_height,
                 use_qk_norm=True, precision=PRECISION_BF16, last_discards_context=True,
                 block_only=False):
        mask = 0
        for l in dual_attention_layers:
            mask |= 1 << int(l)
        self.cfg = Config(num_layers, mask, pooled_dim, captions_dim, in_channels, emb_dim,
                          attn_heads, mlp_expand, patch_size, pos_embed_max_size, base_height,
                          int(bool(use_qk_norm)), int(bool(last_discards_context)), precision,
                          int(bool(block_only)))
        self.handle = c_void_p()
        check(lib().sd3_model_create(ctypes.byref(self.cfg), ctypes.byref(self.handle)),
              "sd3_model_create")

    def close(self):
        self._graphs = {}
        if self.handle:
            lib().sd3_model_destroy(self.handle)
            self.handle = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_param(self, name, tensor):
        self._graphs = {}  # captured forwards refer to the parameters as they were
        shape = (c_int64 * tensor.dim())(*tensor.shape)
        check(lib().sd3_model_set_param(self.handle, name.encode(), ptr(tensor), dtype_tag(tensor),
                                        tensor.dim(), shape, stream_ptr()),
              "sd3_model_set_param(%s)" % name)

    def load(self, params, prefix=""):
        for name, t in params.items():
            self.set_param(prefix + name, t.contiguous())
        missing = c_int(0)
        check(lib().sd3_model_finalize(self.handle, ctypes.byref(missing)), "sd3_model_finalize")
        return self

    def reserve(self, B, Tc, H, W):
        self._graphs = {}  # the workspace may move
        check(lib().sd3_model_reserve(self.handle, B, Tc, H, W), "sd3_model_reserve")

    def forward(self, pooled, captions, latent, timesteps, out=None):
        torch = _torch()
        B, C, H, W = latent.shape
        Tc = captions.shape[1]
        if out is None:
            out = torch.empty_like(latent)
        t32 = timesteps.to(torch.float32).contiguous()
        check(lib().sd3_dit_forward(self.handle, ptr(pooled), ptr(captions), ptr(latent), ptr(t32),
                                    ptr(out), dtype_tag(latent), B, Tc, H, W, stream_ptr()),
              "sd3_dit_forward")
        return out

    def forward_graphed(self, pooled, captions, latent, timesteps, out):
        """forward() on exactly these tensors, replayed as one CUDA graph: the first call for a
        set of tensor addresses and shapes runs the forward once eagerly (which reserves the
        workspace), captures it on the current stream and replays it; later calls only replay.
        For loops that call the denoiser on fixed device buffers (a sampler's latent buffer, a
        serving slot): at one sample per GPU the ~270 launches of a step otherwise cost about
        2 % of it.  The tensors must stay alive and in place; a larger problem, set_param and
        reserve drop the captured graphs.  Returns `out`."""
        torch = _torch()
        args = (pooled, captions, latent, timesteps, out)
        key = tuple((t.data_ptr(), tuple(t.shape), str(t.dtype)) for t in args)
        graphs = self.__dict__.setdefault("_graphs", {})
        entry = graphs.get(key)
        if entry is None:
            if len(graphs) >= 8:
                graphs.clear()
            self.forward(pooled, captions, latent, timesteps, out)
            torch.cuda.synchronize()
            n0 = lib().sd3_launch_count(0)
            g = torch.cuda.CUDAGraph()
            # thread-local capture mode: other host threads (a communicator's watchdog, a data
            # loader) may keep calling the CUDA runtime while this thread captures
            with torch.cuda.graph(g, capture_error_mode="thread_local"):
                self.forward(pooled, captions, latent, timesteps, out)
            launches = int(lib().sd3_launch_count(0) - n0)
            entry = graphs[key] = (g, launches, args)
        entry[0].replay()
        return out

    def graph_launches(self, pooled, captions, latent, timesteps, out):
        """Kernel launches inside the graph forward_graphed replays for these tensors (0 if none
        has been captured)."""
        key = tuple((t.data_ptr(), tuple(t.shape), str(t.dtype)) for t in (pooled, captions, latent, timesteps, out))
        entry = self.__dict__.get("_graphs", {}).get(key)
        return entry[1] if entry else 0

    def block_forward(self, layer, y, c, x):
        B, Tc, E = c.shape
        Tx = x.shape[1]
        check(lib().sd3_block_forward(self.handle, layer, ptr(y), ptr(c), ptr(x), B, Tc, Tx,
                                      stream_ptr()), "sd3_block_forward")
        return c, x


class HostPipeline:
    """Runs the denoiser on batches that live in pinned host memory.

    Every `submit` uploads one batch, runs `model.forward` on it and downloads the
    result into the caller's host buffer.  Uploads go through a copy stream of
    their own into one of `depth` device input sets, downloads through a second
    one, so the upload of batch i+1 and the download of batch i-1 overlap the
    compute of batch i; the order of work on a set is kept by events.  Nothing
    is allocated after construction.  `flush()` makes the current stream wait
    for the last download (call it before reading the host buffers or timing).
    With use_graph (the default) the forward on each device input set is captured
    once as a CUDA graph and replayed (Model.forward_graphed): the sets are fixed
    device buffers, which is what that needs."""

    def __init__(self, model, B, Tc, C, H, W, pooled_dim, captions_dim, dtype=None, depth=2, use_graph=True):
        torch = _torch()
        dtype = dtype or torch.bfloat16
        self.model = model
        self.h2d = torch.cuda.Stream()
        self.d2h = torch.cuda.Stream()
        self.sets = []
        for _ in range(max(1, depth)):
            self.sets.append(dict(
                latent=torch.empty(B, C, H, W, device="cuda", dtype=dtype),
                captions=torch.empty(B, Tc, captions_dim, device="cuda", dtype=dtype),
                pooled=torch.empty(B, pooled_dim, device="cuda", dtype=dtype),
                t=torch.empty(B, device="cuda", dtype=torch.float32),
                out=torch.empty(B, C, H, W, device="cuda", dtype=dtype),
                uploaded=torch.cuda.Event(), computed=torch.cuda.Event(), drained=torch.cuda.Event()))
        self.count = 0
        self.last = None
        self.use_graph = use_graph
        model.reserve(B, Tc, H, W)

    def submit(self, h_pooled, h_captions, h_latent, h_timesteps, h_out):
        torch = _torch()
        st = self.sets[self.count % len(self.sets)]
        self.count += 1
        cur = torch.cuda.current_stream()
        with torch.cuda.stream(self.h2d):
            self.h2d.wait_event(st["computed"])  # the compute that last read this set is over
            st["latent"].copy_(h_latent, non_blocking=True)
            st["captions"].copy_(h_captions, non_blocking=True)
            st["pooled"].copy_(h_pooled, non_blocking=True)
            st["t"].copy_(h_timesteps, non_blocking=True)
            st["uploaded"].record(self.h2d)
        cur.wait_event(st["uploaded"])
        cur.wait_event(st["drained"])  # the download that last read this set's output is over
        fwd = self.model.forward_graphed if self.use_graph else self.model.forward
        fwd(st["pooled"], st["captions"], st["latent"], st["t"], st["out"])
        st["computed"].record(cur)
        with torch.cuda.stream(self.d2h):
            self.d2h.wait_event(st["computed"])
            h_out.copy_(st["out"], non_blocking=True)
            st["drained"].record(self.d2h)
        self.last = st

    def flush(self):
        if self.last is not None:
            _torch().cuda.current_stream().wait_event(self.last["drained"])


def shard_range(n, world, rank):
    """Contiguous slice [lo, hi) of n independent samples owned by `rank` of
    `world` ranks (sizes differ by at most one).  Samples never interact in the
    denoiser, so batch sharding needs no collective on the data path."""
    base, rem = divmod(n, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


# ---------------------------------------------------------------------------
# sampling loop (the caller next to the denoiser; the reference has none)
# ---------------------------------------------------------------------------
def sigma_schedule(steps, shift=3.0):
    """Flow-matching sigmas: s_i = shift * u / (1 + (shift - 1) * u) with
    u = 1 - i/steps for i = 0..steps-1, followed by a final 0.
    The model is called at timestep t = 1000 * sigma."""
    out = []
    for i in range(steps):
        u = 1.0 - i / steps
        out.append(shift * u / (1.0 + (shift - 1.0) * u))
    out.append(0.0)
    return out


def sample(model, latents, cond_captions, cond_pooled, uncond_captions, uncond_pooled, steps=28,
           guidance=4.5, shift=3.0, use_graph=False):
    """Euler flow-matching sampling with classifier-free guidance.  Conditional
    and unconditional branches run stacked in one denoiser call per step
    (effective batch 2n); the update and the refresh of the stacked input are
    one fused kernel (sd3_cfg_euler_step).  Returns the final latents (n, C, H, W)
    in float32.

    use_graph: record all `steps` denoiser calls and updates into one CUDA graph
    and launch that (one untimed denoiser call first sizes the workspace, which
    a stream capture must not do).  The result is bit-identical to the eager
    loop; what it saves is the host's share of ~360 launches per step."""
    torch = _torch()
    n = latents.shape[0]
    dt = latents.dtype
    x_state = latents.to(torch.float32).contiguous().clone()
    x2 = torch.cat([latents, latents], 0).contiguous()
    caps = torch.cat([cond_captions, uncond_captions], 0).to(dt).contiguous()
    pooled = torch.cat([cond_pooled, uncond_pooled], 0).to(dt).contiguous()
    v = torch.empty_like(x2)
    sig = sigma_schedule(steps, shift)
    tvec = torch.empty(2 * n, device=latents.device, dtype=torch.float32)
    half = x_state.numel()

    def loop():
        for i in range(steps):
            tvec.fill_(1000.0 * sig[i])
            model.forward(pooled, caps, x2, tvec, v)
            check(lib().sd3_cfg_euler_step(ptr(x_state), ptr(x2), ptr(v), dtype_tag(x2), half, guidance,
                                           sig[i + 1] - sig[i], stream_ptr()), "sd3_cfg_euler_step")

    if not use_graph:
        loop()
        return x_state
    tvec.fill_(1000.0 * sig[0])
    model.forward(pooled, caps, x2, tvec, v)  # warm-up: x_state and x2 are not touched
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        loop()
    graph.replay()
    return x_state
