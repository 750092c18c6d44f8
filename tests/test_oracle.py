"""The CPU oracle against the golden fixtures produced by the reference's own
PyTorch modules (tests/golden/make_golden.py).  No GPU needed."""
import os
import sys

import pytest
import torch

from conftest import REPO, golden
from oracle import mmdit_oracle as O


def f32(d):
    return {k: v.to(torch.float32) for k, v in d.items()}


@pytest.mark.parametrize("name", ["block_dual.pt", "block_last.pt", "block_plain_hd32.pt"])
def test_block_matches_reference(name):
    g = golden(name)
    cfg = g["config"]
    p = f32(g["params"])
    c, x = O.dit_block(g["x"].float(), g["c"].float(), g["y"].float(), p, cfg["attn_heads"],
                       cfg["use_dual_attention"], cfg["use_qk_norm"], cfg["discard_context"])
    assert (x - g["x_out"]).abs().max().item() < 1e-5
    if cfg["discard_context"]:
        assert c is None and g["c_out"] is None
    else:
        assert (c - g["c_out"]).abs().max().item() < 1e-5


def test_model_matches_reference():
    g = golden("model_toy.pt")
    cfg = g["config"]
    p = f32(g["params"])
    out = O.dit_forward(g["pooled"].float(), g["captions"].float(), g["latent"].float(),
                        g["timesteps"], p, cfg["num_layers"], cfg["dual_attention_layers"],
                        cfg["attn_heads"], cfg["patch_size"], cfg["pos_embed_max_size"],
                        cfg["base_height"], True)
    # the reference's own full-model check uses 1e-5 (module_tests/DiT.py:51)
    assert (out - g["out"]).abs().max().item() < 1e-5
    y = O.conditioning(g["pooled"].float(), g["timesteps"], p)
    assert (y - g["y"]).abs().max().item() < 1e-5
    x0 = O.patch_embed(g["latent"].float(), p["to_patch.conv.weight"], p["to_patch.conv.bias"],
                       cfg["pos_embed_max_size"], cfg["base_height"], cfg["patch_size"])
    assert (x0 - g["x0"]).abs().max().item() < 1e-5


def test_pos_embed_closed_form_equals_full_table():
    # full-table construction exactly as the reference builds it
    # (module_tests/modules.py:79-99 and 43-53), against the cropped closed form
    E, P, base = 32, 12, 4
    hh = torch.arange(P, dtype=torch.float64) / (P / base)
    ww = torch.arange(P, dtype=torch.float64) / (P / base)
    ph, pw = torch.meshgrid(hh, ww, indexing="xy")
    ph, pw = ph.reshape(-1), pw.reshape(-1)
    div = 1.0 / (10000.0 ** (torch.arange(E // 4, dtype=torch.float64) / (E / 4.0)))
    full = torch.cat([torch.sin(ph.outer(div)), torch.cos(ph.outer(div)),
                      torch.sin(pw.outer(div)), torch.cos(pw.outer(div))], -1).to(torch.float32)
    for (h, w) in [(12, 12), (5, 8), (3, 3), (1, 12)]:
        oh, ow = (P - h) // 2, (P - w) // 2
        crop = full.view(P, P, E)[oh:oh + h, ow:ow + w].flatten(0, 1)
        assert torch.equal(crop, O.pos_embed_cropped(E, h, w, P, base))


def test_param_shapes_cover_reference_names():
    g = golden("model_toy.pt")
    cfg = g["config"]
    shapes = O.model_param_shapes(cfg["num_layers"], cfg["dual_attention_layers"], cfg["in_channels"],
                                  cfg["emb_dim"], cfg["pooled_dim"], cfg["captions_dim"],
                                  cfg["patch_size"], cfg["attn_heads"], cfg["mlp_expand"])
    assert set(shapes) == set(g["params"])
    for k, v in g["params"].items():
        assert tuple(v.shape) == tuple(shapes[k]), k
    gb = golden("block_dual.pt")
    cb = gb["config"]
    bs = O.block_param_shapes(cb["emb_dim"], cb["mlp_expand"], cb["emb_dim"] // cb["attn_heads"],
                              cb["use_dual_attention"], cb["discard_context"], cb["use_qk_norm"])
    assert set(bs) == set(gb["params"])


def test_sd35_medium_parameter_count():
    c = O.SD35_MEDIUM
    shapes = O.model_param_shapes(c["num_layers"], c["dual_layers"], c["in_dim"], c["E"],
                                  c["pooled_dim"], c["captions_dim"], c["patch"], c["attn_heads"],
                                  c["mlp_expand"])
    n = 0
    for s in shapes.values():
        k = 1
        for d in s:
            k *= d
        n += k
    assert n == 2243171520


def _load_reference_cpu_extension():
    """oracle/_ref/custom_modules_ref.so: the reference's own modules.cpp compiled
    CPU-only by oracle/build_ref.py (present when a reference checkout was
    available at build time)."""
    import importlib.util
    path = os.path.join(REPO, "oracle", "_ref", "custom_modules_ref.so")
    if not os.path.exists(path):
        return None
    spec = importlib.util.spec_from_file_location("custom_modules_ref", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_oracle_matches_reference_cpp_extension():
    """Runs in a fresh interpreter: the reference's C++ forward works on
    `new float[]` scratch buffers it never initialises (modules.cpp:1635-1658),
    so its result can depend on what the process heap held before the call."""
    import subprocess
    if not os.path.exists(os.path.join(REPO, "oracle", "_ref", "custom_modules_ref.so")):
        pytest.skip("oracle/_ref not built (no reference checkout at build time)")
    code = ("import sys; sys.path.insert(0, %r); sys.path.insert(0, %r); import test_oracle as t; "
            "t._check_against_reference_cpp()" % (os.path.join(REPO, "tests"), REPO))
    last = None
    for _ in range(3):
        last = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
        if last.returncode == 0:
            return
    raise AssertionError(last.stdout[-2000:] + last.stderr[-2000:])


def _check_against_reference_cpp():
    ref = _load_reference_cpu_extension()
    assert ref is not None
    g = golden("model_toy.pt")
    cfg = g["config"]
    p = f32(g["params"])
    out_ref = ref.DiT(g["pooled"].float(), g["captions"].float(), g["latent"].float(), g["timesteps"],
                      {k: v.clone() for k, v in p.items()}, cfg["num_layers"],
                      set(cfg["dual_attention_layers"]), cfg["pooled_dim"], cfg["captions_dim"],
                      cfg["in_channels"], cfg["emb_dim"], cfg["attn_heads"], cfg["mlp_expand"],
                      cfg["patch_size"], cfg["pos_embed_max_size"], cfg["base_height"], True)
    out = O.dit_forward(g["pooled"].float(), g["captions"].float(), g["latent"].float(), g["timesteps"],
                        p, cfg["num_layers"], cfg["dual_attention_layers"], cfg["attn_heads"],
                        cfg["patch_size"], cfg["pos_embed_max_size"], cfg["base_height"], True)
    assert (out - out_ref).abs().max().item() < 1e-5
    gb = golden("block_dual.pt")
    cb = gb["config"]
    pb = f32(gb["params"])
    c, x = gb["c"].float().clone(), gb["x"].float().clone()
    ref.Dit_block(gb["y"].float(), c, x, pb, cb["B"], cb["Tc"], cb["Tx"], cb["emb_dim"], cb["attn_heads"],
                  cb["mlp_expand"], cb["use_dual_attention"], cb["use_qk_norm"], cb["discard_context"])
    co, xo = O.dit_block(gb["x"].float(), gb["c"].float(), gb["y"].float(), pb, cb["attn_heads"],
                         cb["use_dual_attention"], cb["use_qk_norm"], cb["discard_context"])
    assert (x - xo).abs().max().item() < 1e-5
    assert (c - co).abs().max().item() < 1e-5
