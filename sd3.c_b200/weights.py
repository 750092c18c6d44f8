"""Checkpoint loading for the denoiser: a safetensors reader/writer and the
name mapping from a Hugging Face `SD3Transformer2DModel` state dict to the
parameter names of the reference project.

The reference has no loader; it only spells the correspondence out when it
copies its own weights INTO a diffusers model to compare the two
(module_tests/modules.py:534-612).  `hf_to_reference` is that correspondence
run the other way: q/k/v projections are stacked along the output dimension
into one `*_to_qkv` matrix (order q, k, v, the order the reference slices in
modules.py:566-571), everything else is a rename.  The QK-RMSNorm weights are
not touched by the reference's comparison (both sides keep their initial
ones); they are mapped here by the diffusers attribute names `norm_q`,
`norm_k`, `norm_added_q`, `norm_added_k`.

Layouts: a state dict in "oracle layout" keeps 2-D weights as (out, in), the
way `nn.Linear` stores them; `to_extension_layout` transposes them to the
(in, out) form the extension entry points take (module_tests/DiT.py:25-31).

The safetensors format: 8 bytes little-endian header length N, N bytes of JSON
mapping each tensor name to {"dtype", "shape", "data_offsets": [begin, end]}
relative to the byte after the header (plus an optional "__metadata__" entry),
then the raw little-endian tensor bytes.
"""
import json
import mmap
import os
import struct

_DTYPES = {
    "F64": ("float64", 8),
    "F32": ("float32", 4),
    "F16": ("float16", 2),
    "BF16": ("bfloat16", 2),
    "I64": ("int64", 8),
    "I32": ("int32", 4),
    "U8": ("uint8", 1),
    "BOOL": ("bool", 1),
}


class CheckpointError(ValueError):
    pass


def _torch():
    import torch
    return torch


def read_safetensors_header(path):
    """Returns (header dict without "__metadata__", metadata dict, data start offset)."""
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        raw = f.read(8)
        if len(raw) != 8:
            raise CheckpointError("%s: shorter than a safetensors header" % path)
        (n,) = struct.unpack("<Q", raw)
        if n < 2 or 8 + n > size:
            raise CheckpointError("%s: header length %d exceeds the file" % (path, n))
        try:
            header = json.loads(f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise CheckpointError("%s: header is not JSON (%s)" % (path, e))
    if not isinstance(header, dict):
        raise CheckpointError("%s: header is not a JSON object" % path)
    meta = header.pop("__metadata__", {}) or {}
    start = 8 + n
    for name, ent in header.items():
        try:
            dt, shape, (lo, hi) = ent["dtype"], ent["shape"], ent["data_offsets"]
        except (KeyError, TypeError, ValueError):
            raise CheckpointError("%s: malformed entry for %r" % (path, name))
        if dt not in _DTYPES:
            raise CheckpointError("%s: unsupported dtype %s for %r" % (path, dt, name))
        count = 1
        for d in shape:
            count *= int(d)
        if lo < 0 or hi < lo or start + hi > size or hi - lo != count * _DTYPES[dt][1]:
            raise CheckpointError("%s: byte range of %r does not match its shape" % (path, name))
    return header, meta, start


def read_safetensors(path, names=None):
    """Reads tensors (all, or those in `names`) as CPU torch tensors.  The data is
    copied out of a read-only memory map, so the result owns its storage."""
    torch = _torch()
    header, _, start = read_safetensors_header(path)
    want = list(header) if names is None else list(names)
    out = {}
    with open(path, "rb") as f:
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        try:
            for name in want:
                if name not in header:
                    raise CheckpointError("%s: no tensor named %r" % (path, name))
                ent = header[name]
                lo, hi = ent["data_offsets"]
                dt = getattr(torch, _DTYPES[ent["dtype"]][0])
                shape = [int(d) for d in ent["shape"]]
                if hi == lo:
                    out[name] = torch.empty(shape, dtype=dt)
                    continue
                buf = bytearray(mm[start + lo:start + hi])
                out[name] = torch.frombuffer(buf, dtype=dt).reshape(shape)
        finally:
            mm.close()
    return out


def write_safetensors(path, tensors, metadata=None):
    """Writes CPU-convertible torch tensors in safetensors layout (names sorted,
    data packed in that order, header padded with spaces to 8 bytes)."""
    torch = _torch()
    rev = {getattr(torch, v[0]): k for k, v in _DTYPES.items()}
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blobs = []
    off = 0
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in rev:
            raise CheckpointError("cannot store dtype %s (%r)" % (t.dtype, name))
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": rev[t.dtype], "shape": list(t.shape),
                        "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for raw in blobs:
            f.write(raw)


def read_checkpoint(path):
    """`path` is a .safetensors file, a diffusers index json
    (`*.safetensors.index.json`, whose "weight_map" names the shard of every
    tensor), or a directory holding either."""
    if os.path.isdir(path):
        idx = [f for f in sorted(os.listdir(path)) if f.endswith(".safetensors.index.json")]
        if idx:
            path = os.path.join(path, idx[0])
        else:
            files = [f for f in sorted(os.listdir(path)) if f.endswith(".safetensors")]
            if not files:
                raise CheckpointError("%s: no safetensors file" % path)
            state = {}
            for f in files:
                state.update(read_safetensors(os.path.join(path, f)))
            return state
    if path.endswith(".json"):
        with open(path) as f:
            wm = json.load(f).get("weight_map")
        if not isinstance(wm, dict):
            raise CheckpointError("%s: no weight_map" % path)
        by_file = {}
        for name, fn in wm.items():
            by_file.setdefault(fn, []).append(name)
        state = {}
        for fn, names in by_file.items():
            state.update(read_safetensors(os.path.join(os.path.dirname(path), fn), names))
        return state
    return read_safetensors(path)


# ---------------------------------------------------------------------------
# name mapping
# ---------------------------------------------------------------------------
_MODEL_LEVEL = [  # (diffusers module, reference module)
    ("pos_embed.proj", "to_patch.conv"),
    ("time_text_embed.timestep_embedder.linear_1", "timestep_mlp.0"),
    ("time_text_embed.timestep_embedder.linear_2", "timestep_mlp.2"),
    ("time_text_embed.text_embedder.linear_1", "pooled_mlp.0"),
    ("time_text_embed.text_embedder.linear_2", "pooled_mlp.2"),
    ("context_embedder", "captions_linear"),
    ("norm_out.linear", "ada_ln_out.linear"),
    ("proj_out", "linear_out"),
]
_BLOCK_RENAMES = [  # weight + bias pairs inside transformer_blocks.{l}
    ("norm1.linear", "latent_ada_lnorm.linear"),
    ("norm1_context.linear", "context_ada_lnorm.linear"),
    ("attn.to_out.0", "latent_attn_Wout"),
    ("attn.to_add_out", "context_attn_Wout"),
    ("attn2.to_out.0", "latent_dual_attn_Wout"),
    ("ff.net.0.proj", "latent_mlp.lin1"),
    ("ff.net.2", "latent_mlp.lin2"),
    ("ff_context.net.0.proj", "context_mlp.lin1"),
    ("ff_context.net.2", "context_mlp.lin2"),
]
_BLOCK_STACKS = [  # (q, k, v) projections stacked into one matrix
    (("attn.to_q", "attn.to_k", "attn.to_v"), "latent_to_qkv"),
    (("attn.add_q_proj", "attn.add_k_proj", "attn.add_v_proj"), "context_to_qkv"),
    (("attn2.to_q", "attn2.to_k", "attn2.to_v"), "latent_dual_to_qkv"),
]
_BLOCK_NORMS = [  # RMSNorm weights (no bias)
    ("attn.norm_q.weight", "latent_rmsnorm_query.weight"),
    ("attn.norm_k.weight", "latent_rmsnorm_key.weight"),
    ("attn.norm_added_q.weight", "context_rmsnorm_query.weight"),
    ("attn.norm_added_k.weight", "context_rmsnorm_key.weight"),
    ("attn2.norm_q.weight", "latent_dual_rmsnorm_query.weight"),
    ("attn2.norm_k.weight", "latent_dual_rmsnorm_key.weight"),
]
_IGNORED = ("pos_embed.pos_embed",)  # a buffer; the position table is computed on the device


def num_layers_of(hf_state):
    ls = [int(k.split(".")[1]) for k in hf_state if k.startswith("transformer_blocks.")]
    return max(ls) + 1 if ls else 0


def dual_layers_of(hf_state):
    return sorted({int(k.split(".")[1]) for k in hf_state
                   if k.startswith("transformer_blocks.") and ".attn2." in k})


def hf_to_reference(hf_state, strict=True):
    """diffusers SD3Transformer2DModel state dict -> reference names, oracle layout
    ((out, in) weights).  With `strict`, a tensor of the checkpoint that has no
    place in the reference's parameter set raises."""
    torch = _torch()
    out = {}
    used = set()

    def take(name):
        used.add(name)
        return hf_state[name]

    for hf, ref in _MODEL_LEVEL:
        for suffix in ("weight", "bias"):
            k = "%s.%s" % (hf, suffix)
            if k in hf_state:
                out["%s.%s" % (ref, suffix)] = take(k)
    for l in range(num_layers_of(hf_state)):
        pre_h = "transformer_blocks.%d." % l
        pre_r = "transformer.%d." % l
        for hf, ref in _BLOCK_RENAMES:
            for suffix in ("weight", "bias"):
                k = "%s%s.%s" % (pre_h, hf, suffix)
                if k in hf_state:
                    out["%s%s.%s" % (pre_r, ref, suffix)] = take(k)
        for hfs, ref in _BLOCK_STACKS:
            for suffix in ("weight", "bias"):
                ks = ["%s%s.%s" % (pre_h, h, suffix) for h in hfs]
                have = [k in hf_state for k in ks]
                if all(have):
                    out["%s%s.%s" % (pre_r, ref, suffix)] = torch.cat([take(k) for k in ks], dim=0)
                elif any(have):
                    raise CheckpointError("layer %d: incomplete q/k/v set for %s.%s" % (l, ref, suffix))
        for hf, ref in _BLOCK_NORMS:
            k = pre_h + hf
            if k in hf_state:
                out[pre_r + ref] = take(k)
    if strict:
        extra = [k for k in hf_state if k not in used and k not in _IGNORED]
        if extra:
            raise CheckpointError("no reference parameter for %d tensors, e.g. %s" % (len(extra), extra[:3]))
    return out


def reference_to_hf(ref_state):
    """The inverse of `hf_to_reference` (oracle layout in, diffusers names out)."""
    out = {}
    inv_model = {r: h for h, r in _MODEL_LEVEL}
    inv_block = {r: h for h, r in _BLOCK_RENAMES}
    inv_stack = {r: hs for hs, r in _BLOCK_STACKS}
    inv_norm = {r: h for h, r in _BLOCK_NORMS}
    for name, t in ref_state.items():
        if name.startswith("transformer."):
            _, l, rest = name.split(".", 2)
            pre_h = "transformer_blocks.%s." % l
            if rest in inv_norm:
                out[pre_h + inv_norm[rest]] = t
                continue
            mod, suffix = rest.rsplit(".", 1)
            if mod in inv_block:
                out["%s%s.%s" % (pre_h, inv_block[mod], suffix)] = t
            elif mod in inv_stack:
                if t.shape[0] % 3:
                    raise CheckpointError("%s: leading size %d is not 3 x E" % (name, t.shape[0]))
                for h, part in zip(inv_stack[mod], t.chunk(3, dim=0)):
                    out["%s%s.%s" % (pre_h, h, suffix)] = part.contiguous()
            else:
                raise CheckpointError("unknown reference parameter %s" % name)
        else:
            mod, suffix = name.rsplit(".", 1)
            if mod not in inv_model:
                raise CheckpointError("unknown reference parameter %s" % name)
            out["%s.%s" % (inv_model[mod], suffix)] = t
    return out


def to_extension_layout(ref_state):
    """Oracle layout -> what the extension entry points take: 2-D weights
    transposed to (in, out) and contiguous, the rest as is."""
    return {k: (v.t().contiguous() if v.dim() == 2 else v.contiguous()) for k, v in ref_state.items()}


def config_from_state(ref_state, attn_heads=None, patch_size=2, pos_embed_max_size=384, base_height=128):
    """Model hyper-parameters that can be read off the tensor shapes (oracle
    layout).  head_dim comes from the RMSNorm weights, else 64."""
    conv = ref_state["to_patch.conv.weight"]
    E = conv.shape[0]
    nl = 1 + max(int(k.split(".")[1]) for k in ref_state if k.startswith("transformer."))
    hd = 64
    for k, v in ref_state.items():
        if k.endswith("rmsnorm_query.weight"):
            hd = v.shape[0]
            break
    return dict(
        num_layers=nl,
        dual_attention_layers=sorted({int(k.split(".")[1]) for k in ref_state if ".latent_dual_to_qkv." in k}),
        pooled_dim=ref_state["pooled_mlp.0.weight"].shape[1],
        captions_dim=ref_state["captions_linear.weight"].shape[1],
        in_channels=conv.shape[1],
        emb_dim=E,
        attn_heads=attn_heads or E // hd,
        mlp_expand=ref_state["transformer.0.latent_mlp.lin1.weight"].shape[0] // E,
        patch_size=conv.shape[2] if conv.dim() == 4 else patch_size,
        pos_embed_max_size=pos_embed_max_size,
        base_height=base_height,
        use_qk_norm=any(k.endswith("rmsnorm_query.weight") for k in ref_state),
    )


def load_hf_checkpoint(path, device="cuda", precision=None, **overrides):
    """Reads a diffusers SD3 transformer checkpoint and returns a packed
    `sd3_b200.Model` on `device`.  Hyper-parameters come from the shapes;
    `overrides` replaces any of them (e.g. pos_embed_max_size, base_height)."""
    import importlib.util
    import sys
    s = sys.modules.get("sd3_b200")
    if s is None:  # the package directory name has a dot, so it is loaded by path
        here = os.path.dirname(os.path.abspath(__file__))
        spec = importlib.util.spec_from_file_location("sd3_b200", os.path.join(here, "sd3_b200.py"))
        s = importlib.util.module_from_spec(spec)
        sys.modules["sd3_b200"] = s
        spec.loader.exec_module(s)
    ref = hf_to_reference(read_checkpoint(path))
    cfg = config_from_state(ref)
    cfg.update(overrides)
    if precision is not None:
        cfg["precision"] = precision
    model = s.Model(**cfg)
    # One tensor at a time: the host copy of a 2.2 B parameter model is 4.5 GB in
    # bf16, and no second full copy is made on the device.
    for name in list(ref):
        t = ref.pop(name).to(device)
        model.set_param(name, t.t().contiguous() if t.dim() == 2 else t.contiguous())
    model.load({})
    return model
