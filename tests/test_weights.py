"""Checkpoint reader and the diffusers -> reference name mapping
(sd3.c_b200/weights.py).  The mapping follows the copy the reference makes the
other way round in module_tests/modules.py:534-612."""
import importlib.util
import json
import os
import struct
import sys

import pytest
import torch

from conftest import REPO, golden

sys.path.insert(0, os.path.join(REPO, "oracle"))
import mmdit_oracle as O  # noqa: E402


def _weights():
    name = "sd3_weights"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, os.path.join(REPO, "sd3.c_b200", "weights.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


W = _weights()


def test_safetensors_round_trip(tmp_path):
    g = torch.Generator().manual_seed(0)
    tensors = {
        "a.weight": torch.randn(5, 7, generator=g),
        "b.bias": torch.randn(9, generator=g).to(torch.bfloat16),
        "c.half": torch.randn(2, 3, 4, generator=g).to(torch.float16),
        "d.idx": torch.arange(6, dtype=torch.int64).reshape(2, 3),
        "e.empty": torch.empty(0, 4),
    }
    path = str(tmp_path / "t.safetensors")
    W.write_safetensors(path, tensors, metadata={"format": "pt"})
    header, meta, start = W.read_safetensors_header(path)
    assert meta == {"format": "pt"} and start % 8 == 0
    assert header["b.bias"]["dtype"] == "BF16" and header["a.weight"]["shape"] == [5, 7]
    back = W.read_safetensors(path)
    assert set(back) == set(tensors)
    for k, v in tensors.items():
        assert back[k].dtype == v.dtype and back[k].shape == v.shape
        assert torch.equal(back[k], v)
    only = W.read_safetensors(path, names=["c.half"])
    assert list(only) == ["c.half"]
    with pytest.raises(W.CheckpointError):
        W.read_safetensors(path, names=["nope"])


def test_safetensors_rejects_malformed_files(tmp_path):
    p = tmp_path / "short.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(W.CheckpointError):
        W.read_safetensors(str(p))
    p = tmp_path / "hdr.safetensors"
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(W.CheckpointError):
        W.read_safetensors(str(p))
    p = tmp_path / "json.safetensors"
    p.write_bytes(struct.pack("<Q", 8) + b"not json")
    with pytest.raises(W.CheckpointError):
        W.read_safetensors(str(p))
    # byte range that does not match the shape
    hdr = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p = tmp_path / "range.safetensors"
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(W.CheckpointError):
        W.read_safetensors(str(p))
    # byte range past the end of the file
    hdr = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p = tmp_path / "eof.safetensors"
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(W.CheckpointError):
        W.read_safetensors(str(p))


def _toy_reference_state(seed=3):
    """Oracle-layout ((out, in)) state of a 3-layer toy model: layer 0 dual,
    layer 2 last (no context output path)."""
    shapes = O.model_param_shapes(3, (0,), 4, 128, 48, 96, 2, 2, 4)
    boundary = O.random_params(shapes, seed, bias_std=0.02, norm_std=0.1)
    return {k: (v.t().contiguous() if v.dim() == 2 else v) for k, v in boundary.items()}, boundary


def test_name_mapping_round_trip():
    ref, boundary = _toy_reference_state()
    hf = W.reference_to_hf(ref)
    # the diffusers names a real checkpoint uses
    for k in ["pos_embed.proj.weight", "time_text_embed.timestep_embedder.linear_1.weight",
              "time_text_embed.text_embedder.linear_2.bias", "context_embedder.weight",
              "transformer_blocks.0.norm1.linear.weight", "transformer_blocks.0.norm1_context.linear.bias",
              "transformer_blocks.0.attn.to_q.weight", "transformer_blocks.0.attn.add_v_proj.bias",
              "transformer_blocks.0.attn.to_out.0.weight", "transformer_blocks.0.attn.to_add_out.weight",
              "transformer_blocks.0.attn2.to_k.weight", "transformer_blocks.0.attn2.to_out.0.bias",
              "transformer_blocks.0.attn.norm_added_q.weight", "transformer_blocks.0.attn2.norm_k.weight",
              "transformer_blocks.1.ff.net.0.proj.weight", "transformer_blocks.1.ff_context.net.2.bias",
              "norm_out.linear.weight", "proj_out.bias"]:
        assert k in hf, k
    # plain layers have no second attention; the last block has no context output path
    assert not any(k.startswith("transformer_blocks.1.attn2.") for k in hf)
    assert not any(k.startswith("transformer_blocks.2.ff_context.") for k in hf)
    assert "transformer_blocks.2.attn.to_add_out.weight" not in hf
    assert "transformer_blocks.2.attn.add_q_proj.weight" in hf
    E = 128
    assert hf["transformer_blocks.0.attn.to_q.weight"].shape == (E, E)
    # q, k, v are the three row blocks of the stacked matrix, in that order
    qkv = ref["transformer.0.latent_to_qkv.weight"]
    assert torch.equal(hf["transformer_blocks.0.attn.to_k.weight"], qkv[E:2 * E])
    assert W.num_layers_of(hf) == 3 and W.dual_layers_of(hf) == [0]
    back = W.hf_to_reference(hf)
    assert set(back) == set(ref)
    for k in ref:
        assert torch.equal(back[k], ref[k]), k
    ext = W.to_extension_layout(back)
    for k in boundary:
        assert torch.equal(ext[k], boundary[k]), k
    cfg = W.config_from_state(back, pos_embed_max_size=16, base_height=8)
    assert cfg["num_layers"] == 3 and cfg["dual_attention_layers"] == [0]
    assert (cfg["emb_dim"], cfg["attn_heads"], cfg["mlp_expand"]) == (128, 2, 4)
    assert (cfg["pooled_dim"], cfg["captions_dim"], cfg["in_channels"], cfg["patch_size"]) == (48, 96, 4, 2)
    assert cfg["use_qk_norm"] is True


def test_mapping_is_strict_and_ignores_the_position_buffer():
    ref, _ = _toy_reference_state()
    hf = W.reference_to_hf(ref)
    hf["pos_embed.pos_embed"] = torch.zeros(1, 4, 128)  # a buffer, recomputed on the device
    assert set(W.hf_to_reference(hf)) == set(ref)
    hf["transformer_blocks.0.attn.to_q_extra.weight"] = torch.zeros(2)
    with pytest.raises(W.CheckpointError):
        W.hf_to_reference(hf)
    assert set(W.hf_to_reference(hf, strict=False)) == set(ref)
    del hf["transformer_blocks.0.attn.to_q_extra.weight"]
    del hf["transformer_blocks.1.attn.to_v.weight"]
    with pytest.raises(W.CheckpointError):
        W.hf_to_reference(hf)
    with pytest.raises(W.CheckpointError):
        W.reference_to_hf({"transformer.0.bogus.weight": torch.zeros(1)})


def test_sharded_checkpoint_with_index(tmp_path):
    ref, _ = _toy_reference_state()
    hf = W.reference_to_hf(ref)
    names = sorted(hf)
    half = len(names) // 2
    shards = {"diffusion_pytorch_model-00001-of-00002.safetensors": names[:half],
              "diffusion_pytorch_model-00002-of-00002.safetensors": names[half:]}
    wm = {}
    for fn, ns in shards.items():
        W.write_safetensors(str(tmp_path / fn), {n: hf[n] for n in ns})
        wm.update({n: fn for n in ns})
    (tmp_path / "diffusion_pytorch_model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    for target in (str(tmp_path), str(tmp_path / "diffusion_pytorch_model.safetensors.index.json")):
        state = W.read_checkpoint(target)
        assert set(state) == set(hf)
        assert all(torch.equal(state[k], hf[k]) for k in hf)


@pytest.mark.gpu
@pytest.mark.parametrize("store", ["f32", "bf16"])
def test_model_loaded_from_checkpoint_matches_direct_parameters(sd3, tmp_path, store):
    """Golden toy model -> diffusers names -> safetensors -> loader gives the same
    output bits as handing the parameters over directly."""
    g = golden("model_toy.pt")
    cfg = g["config"]
    sdt = torch.float32 if store == "f32" else torch.bfloat16
    ref = {k: (v.t().contiguous() if v.dim() == 2 else v).to(sdt) for k, v in g["params"].items()}
    path = str(tmp_path / "toy.safetensors")
    W.write_safetensors(path, W.reference_to_hf(ref))
    m1 = W.load_hf_checkpoint(path, precision=sd3.PRECISION_BF16,
                              pos_embed_max_size=cfg["pos_embed_max_size"], base_height=cfg["base_height"])
    m2 = sd3.Model(cfg["num_layers"], cfg["dual_attention_layers"], cfg["pooled_dim"], cfg["captions_dim"],
                   cfg["in_channels"], cfg["emb_dim"], cfg["attn_heads"], cfg["mlp_expand"],
                   cfg["patch_size"], cfg["pos_embed_max_size"], cfg["base_height"], True,
                   sd3.PRECISION_BF16)
    m2.load({k: v.to(sdt).cuda() for k, v in g["params"].items()})
    args = (g["pooled"].bfloat16().cuda(), g["captions"].bfloat16().cuda(), g["latent"].bfloat16().cuda(),
            g["timesteps"].cuda())
    o1 = m1.forward(*args)
    o2 = m2.forward(*args)
    torch.cuda.synchronize()
    assert sd3.device_status() == 0
    assert torch.equal(o1, o2)
    rel = ((o1.float().cpu() - g["out"]).norm() / g["out"].norm()).item()
    assert rel < 1e-2
    m1.close()
    m2.close()
