"""The `custom_modules` torch extension used the way the reference's own test
scripts use it (module_tests/DiT.py, module_tests/dit_block.py and the per-op
scripts), on CUDA tensors, checked against the golden fixtures and the oracle."""
import os
import sys

import pytest
import torch

from conftest import REPO, golden
from oracle import mmdit_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def F():
    pkg = os.path.join(REPO, "sd3.c_b200")
    if pkg not in sys.path:
        sys.path.insert(0, pkg)
    import custom_modules
    return custom_modules


def rel_l2(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return ((a - b).norm() / (b.norm() + 1e-30)).item()


def test_DiT_like_reference_script(F):
    # same call as module_tests/DiT.py:40-47, on CUDA tensors
    g = golden("model_toy.pt")
    c = g["config"]
    for dtype, tol_abs, tol_rel in ((torch.float32, 1e-4, None), (torch.bfloat16, None, 1e-2)):
        params = {k: v.to(dtype).cuda() for k, v in g["params"].items()}
        out = F.DiT(g["pooled"].to(dtype).cuda(), g["captions"].to(dtype).cuda(),
                    g["latent"].to(dtype).cuda(), g["timesteps"].cuda(), params,
                    c["num_layers"], set(c["dual_attention_layers"]), c["pooled_dim"], c["captions_dim"],
                    c["in_channels"], c["emb_dim"], c["attn_heads"], c["mlp_expand"], c["patch_size"],
                    c["pos_embed_max_size"], c["base_height"], True)
        assert out.shape == g["latent"].shape and out.dtype == dtype
        if tol_abs:
            assert (out.cpu() - g["out"]).abs().max().item() < tol_abs
        else:
            assert rel_l2(out, g["out"]) < tol_rel
        # second call reuses the packed weights and gives identical bits
        out2 = F.DiT(g["pooled"].to(dtype).cuda(), g["captions"].to(dtype).cuda(),
                     g["latent"].to(dtype).cuda(), g["timesteps"].cuda(), params,
                     c["num_layers"], set(c["dual_attention_layers"]), c["pooled_dim"], c["captions_dim"],
                     c["in_channels"], c["emb_dim"], c["attn_heads"], c["mlp_expand"], c["patch_size"],
                     c["pos_embed_max_size"], c["base_height"], True)
        assert torch.equal(out, out2)


@pytest.mark.parametrize("name", ["block_dual.pt", "block_last.pt"])
def test_Dit_block_in_place_like_reference_script(F, name):
    # same call as module_tests/dit_block.py:60-66; c and x are updated in place
    g = golden(name)
    c = g["config"]
    params = {k: v.float().cuda() for k, v in g["params"].items()}
    y, cc, xx = g["y"].float().cuda(), g["c"].float().cuda(), g["x"].float().cuda()
    res = F.DiT_block_cuda(y, cc, xx, params, c["B"], c["Tc"], c["Tx"], c["emb_dim"], c["attn_heads"],
                           c["mlp_expand"], c["use_dual_attention"], c["use_qk_norm"], c["discard_context"])
    assert res[1].data_ptr() == xx.data_ptr() and res[0].data_ptr() == cc.data_ptr()
    assert (xx.cpu() - g["x_out"]).abs().max().item() < 1e-4
    if not c["discard_context"]:
        assert (cc.cpu() - g["c_out"]).abs().max().item() < 1e-4
    # bf16 tensors select the tensor-core path
    params16 = {k: v.cuda() for k, v in g["params"].items()}
    y, cc, xx = g["y"].cuda(), g["c"].cuda(), g["x"].cuda()
    F.Dit_block(y, cc, xx, params16, c["B"], c["Tc"], c["Tx"], c["emb_dim"], c["attn_heads"],
                c["mlp_expand"], c["use_dual_attention"], c["use_qk_norm"], c["discard_context"])
    assert rel_l2(xx, g["x_out"]) < 1.5e-2  # the in/out streams themselves are bf16 here


def test_cpu_tensors_are_rejected(F):
    x = torch.randn(4, 8)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        F.linear(x, torch.randn(8, 8), torch.zeros(8))


def test_per_op_entry_points(F):
    torch.manual_seed(0)
    # linear (module_tests/linear.py: W given as (C_in, C_out))
    x = torch.randn(2, 4, 512, device="cuda")
    W = torch.randn(512, 128, device="cuda") * 0.05
    b = torch.randn(128, device="cuda")
    assert (F.linear(x, W, b) - (x @ W + b)).abs().max().item() < 1e-4
    assert rel_l2(F.linear(x.bfloat16(), W.bfloat16(), b), x.bfloat16().float() @ W.bfloat16().float() + b) < 1e-2
    # layer_norm with affine parameters (module_tests/ln.py)
    x = torch.randn(2, 3, 64, device="cuda")
    w, bb = torch.randn(64, device="cuda"), torch.randn(64, device="cuda")
    ref = torch.nn.functional.layer_norm(x, (64,), w, bb, 1e-5)
    assert (F.layer_norm(x, w, bb, 1e-5, False)[0] - ref).abs().max().item() < 1e-4
    # rms_norm (module_tests/rmsnorm.py)
    ref = torch.nn.functional.rms_norm(x, (64,), w, 1e-5)
    assert (F.rms_norm(x, w, 1e-5, False)[0] - ref).abs().max().item() < 1e-4
    # sinusoidal / positional embeddings (module_tests/sinusoidal_embeddings.py)
    t = torch.rand(16, device="cuda") * 1000
    assert (F.sinusoidal_embedding(t, 256).cpu() - O.sinusoidal_embedding(t.cpu(), 256)).abs().max().item() < 1e-4
    pe = F.positional_embedding(256, 96, 96, 64)
    assert (pe.cpu() - O.pos_embed_cropped(256, 96, 96, 96, 64)).abs().max().item() < 1e-6
    # conv2d in the patch-embedding form (kernel == stride)
    lat = torch.randn(2, 16, 8, 12, device="cuda").bfloat16().float()
    k = (torch.randn(64, 16, 2, 2, device="cuda") * 0.1).bfloat16().float()
    cb = torch.randn(64, device="cuda")
    assert (F.conv2d(lat, k, cb, 2, 0) - torch.nn.functional.conv2d(lat, k, cb, stride=2)).abs().max().item() < 1e-4
    # conv2d with other strides / padding (module_tests/conv2d.py), fp32 and bf16
    xin = torch.randn(2, 3, 17, 19, device="cuda")
    k3 = torch.randn(5, 3, 3, 3, device="cuda") * 0.2
    b3 = torch.randn(5, device="cuda")
    for stride, pad in ((1, 1), (2, 1), (1, 0), (3, 2)):
        ref = torch.nn.functional.conv2d(xin, k3, b3, stride=stride, padding=pad)
        got = F.conv2d(xin, k3, b3, stride, pad)
        assert got.shape == ref.shape and (got - ref).abs().max().item() < 1e-4
    got = F.conv2d(xin.bfloat16(), k3.bfloat16(), b3, 2, 1)
    ref = torch.nn.functional.conv2d(xin.bfloat16().float(), k3.bfloat16().float(), b3, stride=2, padding=1)
    assert got.dtype == torch.bfloat16 and rel_l2(got, ref) < 1e-2
    # mha (module_tests/attention.py shapes: B2 T128 C512 H8 -> head_dim 64)
    q, kk, v = [torch.randn(2, 128, 512, device="cuda") for _ in range(3)]
    ref = O.attention(q.view(2, 128, 8, 64), kk.view(2, 128, 8, 64), v.view(2, 128, 8, 64))
    assert (F.mha(q, kk, v, 8) - ref).abs().max().item() < 1e-4
    assert rel_l2(F.mha(q.bfloat16(), kk.bfloat16(), v.bfloat16(), 8), ref) < 1e-2
    # mha with a key length other than the query length (module_tests/attention.py: T 128, L 96)
    k96, v96 = torch.randn(2, 96, 512, device="cuda"), torch.randn(2, 96, 512, device="cuda")
    ref = torch.nn.functional.scaled_dot_product_attention(
        q.view(2, 128, 8, 64).transpose(1, 2), k96.view(2, 96, 8, 64).transpose(1, 2),
        v96.view(2, 96, 8, 64).transpose(1, 2)).transpose(1, 2).reshape(2, 128, 512)
    assert (F.mha(q, k96, v96, 8) - ref).abs().max().item() < 1e-4
    assert rel_l2(F.mha(q.bfloat16(), k96.bfloat16(), v96.bfloat16(), 8), ref) < 1e-2
    # mlp with GELU-tanh (the block's MLP)
    x = torch.randn(6, 64, device="cuda")
    W1, b1 = torch.randn(64, 256, device="cuda") * 0.1, torch.randn(256, device="cuda")
    W2, b2 = torch.randn(256, 64, device="cuda") * 0.1, torch.randn(64, device="cuda")
    ref = torch.nn.functional.gelu(x @ W1 + b1, approximate="tanh") @ W2 + b2
    assert (F.mlp(x, W1, b1, W2, b2, "gelu_tanh", 6, 64, 256, 64) - ref).abs().max().item() < 1e-4
