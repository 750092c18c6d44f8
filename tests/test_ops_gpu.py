"""Per-operator parity on the GPU through the C ABI, each op against a plain
PyTorch fp32 evaluation of the same formula on the same seeded inputs.
Tolerances: fp32 kernels max-abs <= 1e-4 (north-star per-module bound);
bf16-operand kernels rel-L2 <= 1e-2 (they are far tighter in practice because
accumulation is fp32 and the inputs here are already bf16-representable)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def rel_l2(a, b):
    a, b = a.double(), b.double()
    return ((a - b).norm() / (b.norm() + 1e-30)).item()


@pytest.fixture(autouse=True)
def _healthy(sd3):
    yield
    assert sd3.device_status() == 0


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (77, 1536, 1536), (333, 4608, 1536),
                                   (4096, 1536, 1536), (1000, 6144, 1536), (1000, 1536, 6144),
                                   (200, 384, 192), (500, 64, 1536), (130, 1000, 72), (1, 8, 8)])
def test_linear_bf16(sd3, M, N, K):
    torch.manual_seed(M + N + K)
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    b = torch.randn(N, device="cuda")
    out = sd3.linear(x, w, b, out_dtype=torch.float32)
    ref = x.float() @ w.float().t() + b
    assert rel_l2(out, ref) < 1e-4
    out16 = sd3.linear(x, w, b)
    assert rel_l2(out16, ref) < 1e-2
    g = sd3.linear(x, w, b, act=sd3.ACT_GELU_TANH, out_dtype=torch.float32)
    assert rel_l2(g, torch.nn.functional.gelu(ref, approximate="tanh")) < 1e-4


def test_linear_rejects_bad_shapes(sd3):
    x = torch.zeros(16, 12, device="cuda", dtype=torch.bfloat16)  # K = 12: pitch not 16-byte multiple
    w = torch.zeros(8, 12, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(sd3.Sd3Error):
        sd3.linear(x, w)


@pytest.mark.parametrize("M,N,K", [(77, 1536, 1536), (130, 100, 70), (5, 3, 2)])
def test_linear_f32_exact(sd3, M, N, K):
    torch.manual_seed(1)
    x = torch.randn(M, K, device="cuda")
    w = torch.randn(N, K, device="cuda") * 0.05
    b = torch.randn(N, device="cuda")
    ref = (x.double() @ w.double().t() + b.double()).float()
    assert (sd3.linear_f32(x, w, b) - ref).abs().max().item() < 1e-4
    g = sd3.linear_f32(x, w, b, act=sd3.ACT_GELU_TANH)
    assert (g - torch.nn.functional.gelu(ref, approximate="tanh")).abs().max().item() < 1e-4


def test_gate_residual(sd3):
    torch.manual_seed(2)
    B, T, N, K = 3, 200, 1536, 512
    x = torch.randn(B * T, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    b = torch.randn(N, device="cuda")
    mod = torch.randn(B, 5 * N, device="cuda")
    gate = mod[:, N:2 * N]
    resid = torch.randn(B * T, N, device="cuda")
    r0 = resid.clone()
    sd3.check(sd3.lib().sd3_linear_gate_residual(
        sd3.ptr(x), sd3.ptr(w), sd3.ptr(b), gate.data_ptr(), mod.stride(0), T, sd3.ptr(resid),
        B * T, N, K, sd3.stream_ptr()))
    ref = r0 + ((x.float() @ w.float().t() + b).view(B, T, N) * gate[:, None, :]).view(B * T, N)
    assert rel_l2(resid, ref) < 1e-4


@pytest.mark.parametrize("E,B,Tin,Tt,off", [(192, 2, 100, 150, 50), (1536, 2, 77, 333, 0), (128, 1, 130, 130, 0)])
def test_qkv_project_norm_and_concat(sd3, E, B, Tin, Tt, off):
    torch.manual_seed(3)
    x = torch.randn(B * Tin, E, device="cuda").bfloat16()
    w = (torch.randn(3 * E, E, device="cuda") * 0.1).bfloat16()
    b = torch.randn(3 * E, device="cuda")
    wq = torch.randn(64, device="cuda")
    wk = torch.randn(64, device="cuda")
    qkv = torch.zeros(B, Tt, 3 * E, device="cuda", dtype=torch.bfloat16)
    sd3.qkv_project(x, w, b, wq, wk, 1e-6, qkv, B, Tin, Tt, off, E)
    y = (x.float() @ w.float().t() + b).view(B, Tin, 3, E // 64, 64)

    def rms(v, wt):
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-6) * wt

    ref = torch.stack([rms(y[:, :, 0], wq), rms(y[:, :, 1], wk), y[:, :, 2]], 2).reshape(B, Tin, 3 * E)
    assert rel_l2(qkv[:, off:off + Tin], ref) < 1e-2
    # rows outside [off, off+Tin) are not touched
    assert qkv[:, :off].abs().max().item() == 0 if off else True
    assert qkv[:, off + Tin:].abs().max().item() == 0 if off + Tin < Tt else True


@pytest.mark.parametrize("B,T,NH,Tc", [(1, 128, 1, 0), (1, 1, 1, 0), (1, 333, 2, 77), (2, 1357, 3, 333),
                                       (1, 640, 24, 128), (1, 4429, 2, 333), (3, 129, 1, 129)])
def test_attention_bf16(sd3, B, T, NH, Tc):
    torch.manual_seed(T)
    E = NH * 64
    qkv = torch.randn(B, T, 3 * E, device="cuda").bfloat16()
    if Tc == T:
        pytest.skip("all-context split has no image rows")
    oc, ox = sd3.attention(qkv, B, T, NH, Tc, 0.125)
    q, k, v = [t.view(B, T, NH, 64).transpose(1, 2).float() for t in qkv.chunk(3, -1)]
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, T, E)
    got = torch.cat([oc, ox], 1) if oc is not None else ox
    assert rel_l2(got, ref) < 1e-2
    # dropping the context rows must not change the image rows
    _, ox2 = sd3.attention(qkv, B, T, NH, Tc, 0.125, want_context=False)
    assert torch.equal(ox, ox2)


def test_attention_large_scores_stay_finite(sd3):
    # peaked softmax: exercises the running-max update / O rescale path
    torch.manual_seed(5)
    B, T, NH = 1, 700, 2
    qkv = (torch.randn(B, T, 3 * NH * 64, device="cuda") * 6).bfloat16()
    _, ox = sd3.attention(qkv, B, T, NH, 0, 0.125)
    q, k, v = [t.view(B, T, NH, 64).transpose(1, 2).float() for t in qkv.chunk(3, -1)]
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, T, -1)
    assert torch.isfinite(ox.float()).all()
    assert rel_l2(ox, ref) < 2e-2


@pytest.mark.parametrize("B,T,NH,D", [(2, 333, 24, 64), (1, 100, 2, 128), (2, 50, 3, 32), (1, 7, 1, 16)])
def test_attention_generic_f32(sd3, B, T, NH, D):
    torch.manual_seed(6)
    q, k, v = [torch.randn(B, T, NH * D, device="cuda") for _ in range(3)]
    o = sd3.attention_generic(q, k, v, NH)
    qq, kk, vv = [t.view(B, T, NH, D).transpose(1, 2).double() for t in (q, k, v)]
    ref = torch.nn.functional.scaled_dot_product_attention(qq, kk, vv).transpose(1, 2).reshape(B, T, NH * D)
    assert (o - ref.float()).abs().max().item() < 1e-4


@pytest.mark.parametrize("B,T,E", [(2, 77, 1536), (1, 5, 256), (3, 33, 768), (1, 2, 64), (1, 3, 2048)])
def test_layernorm_modulate(sd3, B, T, E):
    torch.manual_seed(7)
    x = torch.randn(B * T, E, device="cuda") * 2 + 0.3
    mod = torch.randn(B, 9 * E, device="cuda") * 0.3
    o1, o2 = sd3.layernorm_modulate(x, B, T, E, 1e-6, mod[:, 0:E], mod[:, E:2 * E],
                                    mod[:, 6 * E:7 * E], mod[:, 7 * E:8 * E], out_dtype=torch.float32)
    ln = torch.nn.functional.layer_norm(x, (E,), eps=1e-6).view(B, T, E)
    r1 = (ln * (1 + mod[:, None, E:2 * E]) + mod[:, None, 0:E]).view(B * T, E)
    r2 = (ln * (1 + mod[:, None, 7 * E:8 * E]) + mod[:, None, 6 * E:7 * E]).view(B * T, E)
    assert (o1 - r1).abs().max().item() < 1e-4
    assert (o2 - r2).abs().max().item() < 1e-4
    b1, _ = sd3.layernorm_modulate(x, B, T, E, 1e-6, mod[:, 0:E], mod[:, E:2 * E])
    assert rel_l2(b1, r1) < 1e-2


@pytest.mark.parametrize("B,N,K", [(2, 1536, 256), (8, 27652, 1536), (11, 1536, 2048), (1, 3, 8)])
def test_skinny_linear(sd3, B, N, K):
    torch.manual_seed(8)
    inp = torch.randn(B, K, device="cuda")
    w = torch.randn(N, K, device="cuda") * 0.05
    b = torch.randn(N, device="cuda")
    add = torch.randn(B, N, device="cuda")
    o = sd3.skinny_linear(inp, w, b, add, act=1)
    ref = torch.nn.functional.silu(inp.double() @ w.double().t() + b + add).float()
    assert (o - ref).abs().max().item() < 1e-4
    o = sd3.skinny_linear(inp, w.bfloat16(), b)
    ref = (inp.double() @ w.bfloat16().double().t() + b).float()
    assert (o - ref).abs().max().item() < 1e-4


def test_sinusoidal_and_pos_table(sd3):
    from oracle import mmdit_oracle as O
    t = torch.tensor([0.0, 0.5, 500.0, 999.0, 37.25], device="cuda")
    o = sd3.sinusoidal_embedding(t, 256)
    assert (o.cpu() - O.sinusoidal_embedding(t.cpu(), 256)).abs().max().item() < 1e-4
    for (h, w, E, pmax, base) in [(64, 64, 1536, 384, 64), (6, 10, 128, 24, 8), (1, 1, 64, 16, 8)]:
        tab = sd3.pos_embed_table(h, w, E, pmax, base)
        assert (tab.cpu() - O.pos_embed_cropped(E, h, w, pmax, base)).abs().max().item() < 1e-6


def test_patch_embed(sd3):
    torch.manual_seed(9)
    lat = torch.randn(2, 16, 8, 12, device="cuda").bfloat16().float()
    w = (torch.randn(64, 16, 2, 2, device="cuda") * 0.1).bfloat16()
    b = torch.randn(64, device="cuda")
    pt = sd3.pos_embed_table(4, 6, 64, 16, 8)
    o = sd3.patch_embed(lat, w.view(64, 64).contiguous(), b, pt, 2, 64)
    ref = torch.nn.functional.conv2d(lat, w.float(), b, stride=2).flatten(2).transpose(1, 2) + pt
    assert (o.view(2, 24, 64) - ref).abs().max().item() < 1e-4


def test_pack_weight_and_cast(sd3):
    w = torch.randn(70, 33, device="cuda")
    p = sd3.pack_weight(w, torch.float32)
    assert torch.equal(p, w.t().contiguous())
    p16 = sd3.pack_weight(w)
    assert torch.equal(p16, w.t().contiguous().bfloat16())
    assert torch.equal(sd3.cast(w, torch.bfloat16), w.bfloat16())
    assert torch.equal(sd3.cast(w.bfloat16(), torch.float32), w.bfloat16().float())


def test_rmsnorm_heads(sd3):
    torch.manual_seed(10)
    x = torch.randn(10, 3 * 96, device="cuda")
    w = torch.randn(32, device="cuda")
    ref = x.clone().view(10, 9, 32)
    ref[:, 3:6] = ref[:, 3:6] * torch.rsqrt(ref[:, 3:6].pow(2).mean(-1, keepdim=True) + 1e-6) * w
    sd3.rmsnorm_heads(x, 96, 3, 32, w, 1e-6)
    assert (x.view(10, 9, 32) - ref).abs().max().item() < 1e-5


@pytest.mark.parametrize("M,N,K,act", [(512, 768, 1536, 0), (333, 1536, 6144, 1), (129, 192, 1552, 0),
                                       (4096, 4608, 1536, 0), (64, 64, 128, 0)])
def test_linear_e4m3_matches_the_same_contraction_in_fp32(sd3, M, N, K, act):
    """FP8 GEMM (tcgen05 kind::f8f6f4): quantise both operands with per-tensor
    scales, then compare with the fp32 product of the very same e4m3 values, so
    the only difference left is the accumulation order."""
    gen = torch.Generator(device="cuda").manual_seed(M + N + K)
    x = torch.randn(M, K, generator=gen, device="cuda")
    w = torch.randn(N, K, generator=gen, device="cuda") * 0.02
    bias = torch.randn(N, generator=gen, device="cuda") * 0.1
    sx = x.abs().max().item() / 448.0
    sw = w.abs().max().item() / 448.0
    x8 = torch.empty(M, K, device="cuda", dtype=torch.uint8)
    w8 = torch.empty(N, K, device="cuda", dtype=torch.uint8)
    sd3.check(sd3.lib().sd3_quantize_e4m3(sd3.ptr(x), sd3.DTYPE_F32, sd3.ptr(x8), M * K, sx, sd3.stream_ptr()))
    sd3.check(sd3.lib().sd3_quantize_e4m3(sd3.ptr(w.bfloat16()), sd3.DTYPE_BF16, sd3.ptr(w8), N * K, sw,
                                          sd3.stream_ptr()))
    # the quantiser rounds to nearest even like torch's conversion
    assert torch.equal(x8.view(torch.float8_e4m3fn).float(), (x / sx).to(torch.float8_e4m3fn).float())
    assert torch.equal(w8.view(torch.float8_e4m3fn).float(),
                       (w.bfloat16().float() / sw).to(torch.float8_e4m3fn).float())
    out = torch.empty(M, N, device="cuda", dtype=torch.float32)
    sd3.check(sd3.lib().sd3_linear_e4m3(sd3.ptr(x8), sd3.ptr(w8), sd3.ptr(bias), sd3.ptr(out), sd3.DTYPE_F32,
                                        M, N, K, sx * sw, act, sd3.stream_ptr()))
    torch.cuda.synchronize()
    assert sd3.device_status() == 0
    ref = (x8.view(torch.float8_e4m3fn).double() @ w8.view(torch.float8_e4m3fn).double().t()) * (sx * sw) + bias.double()
    if act:
        ref = torch.nn.functional.gelu(ref, approximate="tanh")
    err = (out.double() - ref).abs().max().item()
    assert err < 2e-3 * max(1.0, ref.abs().max().item()), err


@pytest.mark.parametrize("M,N,K,act", [(512, 256, 256, 0), (1024, 4608, 1536, 0), (333, 1536, 6144, 1)])
def test_linear_e4m3_cta_pair_kernel_bf16_output(sd3, M, N, K, act):
    """bf16 output with N % 256 == 0 and M >= 256 takes the CTA-pair e4m3 kernel."""
    gen = torch.Generator(device="cuda").manual_seed(M + N + K)
    x = torch.randn(M, K, generator=gen, device="cuda")
    w = torch.randn(N, K, generator=gen, device="cuda") * 0.02
    bias = torch.randn(N, generator=gen, device="cuda") * 0.1
    sx, sw = x.abs().max().item() / 448.0, w.abs().max().item() / 448.0
    x8, w8 = (x / sx).to(torch.float8_e4m3fn), (w / sw).to(torch.float8_e4m3fn)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    sd3.check(sd3.lib().sd3_linear_e4m3(sd3.ptr(x8.view(torch.uint8)), sd3.ptr(w8.view(torch.uint8)),
                                        sd3.ptr(bias), sd3.ptr(out), sd3.DTYPE_BF16, M, N, K, sx * sw, act,
                                        sd3.stream_ptr()))
    torch.cuda.synchronize()
    assert sd3.device_status() == 0
    ref = (x8.double() @ w8.double().t()) * (sx * sw) + bias.double()
    if act:
        ref = torch.nn.functional.gelu(ref, approximate="tanh")
    assert ((out.double() - ref).norm() / ref.norm()).item() < 4e-3  # bf16 rounding of the output


@pytest.mark.parametrize("T", [63, 64, 65, 127, 128, 129, 191, 192, 193, 255, 256, 257, 320, 321])
def test_attention_bf16_around_tile_boundaries(sd3, T):
    """One to six 64-key sub-tiles, ragged and exact, through the three-buffer score ring."""
    torch.manual_seed(T)
    B, NH = 2, 2
    Tc = T // 3
    E = NH * 64
    qkv = torch.randn(B, T, 3 * E, device="cuda").bfloat16()
    oc, ox = sd3.attention(qkv, B, T, NH, Tc, 0.125)
    q, k, v = [t.view(B, T, NH, 64).transpose(1, 2).float() for t in qkv.chunk(3, -1)]
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, T, E)
    assert rel_l2(torch.cat([oc, ox], 1), ref) < 1e-2
    assert sd3.device_status() == 0


def test_attention_rising_scores_rescale_every_sub_tile(sd3):
    """Scores that grow steadily along the keys move the running maximum by more
    than 2^8 (exp2 domain) in every sub-tile, so O is rescaled each time."""
    B, T, NH = 1, 512, 1
    q = torch.zeros(B, T, 64, device="cuda")
    q[..., 0] = 8.0
    k = torch.zeros(B, T, 64, device="cuda")
    k[..., 0] = torch.arange(T, device="cuda", dtype=torch.float32) * 0.25  # score*scale rises 0.25 per key
    gen = torch.Generator(device="cuda").manual_seed(9)
    v = torch.randn(B, T, 64, generator=gen, device="cuda")
    qkv = torch.cat([q, k, v], -1).bfloat16()
    _, ox = sd3.attention(qkv, B, T, NH, 0, 0.125)
    qf, kf, vf = [t.float().view(B, T, 1, 64).transpose(1, 2) for t in qkv.chunk(3, -1)]
    ref = torch.nn.functional.scaled_dot_product_attention(qf, kf, vf).transpose(1, 2).reshape(B, T, 64)
    assert torch.isfinite(ox.float()).all()
    assert rel_l2(ox, ref) < 1e-2
    assert sd3.device_status() == 0


@pytest.mark.parametrize("B,T,NH,Tc,amp", [(1, 4429, 3, 333, 1.0), (1, 2100, 2, 0, 4.0), (1, 16717, 3, 333, 1.0),
                                           (2, 2500, 1, 77, 1.0)])
def test_attention_key_split_matches_unsplit(sd3, B, T, NH, Tc, amp):
    """sd3_attention_ws: launches with too few CTAs for the GPU split the keys of each query
    tile over several CTAs and merge (maximum, row sum, unnormalised rows); same result as the
    one-CTA-per-tile path and as the fp32 reference."""
    torch.manual_seed(T + NH)
    E = NH * 64
    qkv = (torch.randn(B, T, 3 * E, device="cuda") * amp).bfloat16()
    scratch = sd3.attention_scratch(B, T, NH)
    assert scratch is not None  # these shapes are chosen to need the split
    oc0, ox0 = sd3.attention(qkv, B, T, NH, Tc, 0.125)
    oc1, ox1 = sd3.attention(qkv, B, T, NH, Tc, 0.125, scratch=scratch)
    torch.cuda.synchronize()
    assert sd3.device_status() == 0
    q, k, v = [t.view(B, T, NH, 64).transpose(1, 2).float() for t in qkv.chunk(3, -1)]
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, T, E)
    got = torch.cat([oc1, ox1], 1) if oc1 is not None else ox1
    assert rel_l2(got, ref) < 1e-2
    assert rel_l2(ox1, ox0) < 5e-3  # the two paths differ by bf16 rounding of differently ordered sums
    # a shape that fills the GPU needs no scratch, and a null scratch falls back to the unsplit path
    assert sd3.attention_scratch(8, 4429, 24) is None


def _normed_qkv(B, T, NH, wq, wk, seed, amp=1.0):
    """q and k per-head RMS-normed with weights wq, wk (as the QKV epilogue leaves them), v random."""
    gen = torch.Generator(device="cuda").manual_seed(seed)
    raw = torch.randn(B, T, 3, NH, 64, device="cuda", generator=gen) * amp

    def rms(t, w):
        return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + 1e-6) * w

    q, k, v = rms(raw[:, :, 0], wq), rms(raw[:, :, 1], wk), raw[:, :, 2]
    return torch.stack([q, k, v], 2).reshape(B, T, 3 * NH * 64).bfloat16()


@pytest.mark.parametrize("B,T,NH,Tc,wamp", [(2, 1357, 3, 333, 1.0), (1, 128, 1, 0, 1.0), (2, 129, 2, 65, 2.0),
                                            (1, 640, 2, 0, 2.5), (2, 4429, 2, 333, 1.0), (1, 1, 1, 0, 1.0),
                                            (3, 77, 4, 13, 0.3)])
def test_attention_bounded_matches_online(sd3, B, T, NH, Tc, wamp):
    """sd3_attention_bounded: with a valid bound on |q . k| the softmax runs without a running
    maximum; same result as the online softmax and the fp32 reference, ragged last tiles and
    context/image split included.  wamp 2.5 gives scores up to 64 * 6.25 / 8 * log2(e) = 72 in
    the exp2 domain, near the 80 the mode accepts."""
    gen = torch.Generator(device="cuda").manual_seed(T)
    wq = wamp * (1.0 + 0.2 * torch.rand(64, device="cuda", generator=gen) - 0.2)
    wk = wamp * (1.0 + 0.2 * torch.rand(64, device="cuda", generator=gen) - 0.2)
    qkv = _normed_qkv(B, T, NH, wq, wk, seed=T + 1)
    bound = sd3.qk_norm_score_bound(wq, wk)
    assert bound * 0.125 * 1.4426950408889634 <= 80.0  # the bounded kernel really runs
    oc0, ox0 = sd3.attention(qkv, B, T, NH, Tc, 0.125)
    oc1, ox1 = sd3.attention(qkv, B, T, NH, Tc, 0.125, score_bound=bound)
    torch.cuda.synchronize()
    assert sd3.device_status() == 0
    E = NH * 64
    q, k, v = [t.view(B, T, NH, 64).transpose(1, 2).float() for t in qkv.chunk(3, -1)]
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, T, E)
    got = torch.cat([oc1, ox1], 1) if oc1 is not None else ox1
    assert torch.isfinite(got.float()).all()
    assert rel_l2(got, ref) < 1e-2
    assert rel_l2(ox1, ox0) < 6e-3
    # the actual scores respect the bound the weights promise
    assert (q @ k.transpose(-1, -2)).abs().max().item() <= bound


def test_attention_bounded_with_key_split(sd3):
    """Bounded softmax together with the key split: the partial results carry maximum 0."""
    B, T, NH, Tc = 1, 4429, 3, 333
    wq = torch.full((64,), 1.3, device="cuda")
    wk = torch.full((64,), 0.9, device="cuda")
    qkv = _normed_qkv(B, T, NH, wq, wk, seed=3)
    scratch = sd3.attention_scratch(B, T, NH)
    assert scratch is not None
    bound = sd3.qk_norm_score_bound(wq, wk)
    oc0, ox0 = sd3.attention(qkv, B, T, NH, Tc, 0.125)
    oc1, ox1 = sd3.attention(qkv, B, T, NH, Tc, 0.125, scratch=scratch, score_bound=bound)
    torch.cuda.synchronize()
    assert sd3.device_status() == 0
    assert rel_l2(ox1, ox0) < 6e-3 and rel_l2(oc1, oc0) < 6e-3


def test_attention_bound_above_limit_uses_online_softmax(sd3):
    """A bound above 80 / (scale log2 e), or none, selects the online softmax: large scores stay
    finite (the bounded arithmetic would overflow on these inputs)."""
    torch.manual_seed(5)
    B, T, NH = 1, 700, 2
    qkv = (torch.randn(B, T, 3 * NH * 64, device="cuda") * 6).bfloat16()
    q, k, v = [t.view(B, T, NH, 64).transpose(1, 2).float() for t in qkv.chunk(3, -1)]
    bound = (q @ k.transpose(-1, -2)).abs().max().item() * 1.01
    assert bound * 0.125 * 1.4426950408889634 > 80.0
    _, ox = sd3.attention(qkv, B, T, NH, 0, 0.125, score_bound=bound)
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, T, -1)
    assert torch.isfinite(ox.float()).all()
    assert rel_l2(ox, ref) < 2e-2
    assert sd3.device_status() == 0


@pytest.mark.parametrize("B,T,NH,Tc", [(2, 1357, 3, 333), (1, 4429, 2, 333), (2, 130, 2, 0)])
def test_attention_prescaled_queries(sd3, B, T, NH, Tc):
    """scale == 0: the queries carry softmax_scale * log2(e) already (the engine folds the factor
    into the RMSNorm weight of q), the scores are exp2 arguments; bounded and online softmax."""
    c = 0.125 * 1.4426950408889634
    wq = torch.full((64,), 1.2, device="cuda")
    wk = torch.full((64,), 0.8, device="cuda")
    qkv = _normed_qkv(B, T, NH, wq, wk, seed=T + 2)
    E = NH * 64
    pre = qkv.clone()
    pre[..., :E] = (qkv[..., :E].float() * c).bfloat16()
    bound = sd3.qk_norm_score_bound(wq, wk) * c
    oc0, ox0 = sd3.attention(qkv, B, T, NH, Tc, 0.125)
    oc1, ox1 = sd3.attention(pre, B, T, NH, Tc, 0.0, score_bound=bound)  # bounded, unit scale
    oc2, ox2 = sd3.attention(pre, B, T, NH, Tc, 0.0)                     # online softmax, unit scale
    torch.cuda.synchronize()
    assert sd3.device_status() == 0
    q, k, v = [t.view(B, T, NH, 64).transpose(1, 2).float() for t in qkv.chunk(3, -1)]
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, T, E)
    for oc, ox in ((oc1, ox1), (oc2, ox2)):
        got = torch.cat([oc, ox], 1) if oc is not None else ox
        assert rel_l2(got, ref) < 1e-2
        assert rel_l2(ox, ox0) < 8e-3


@pytest.mark.parametrize("M0,M1,N,K,act", [(4096, 333, 1536, 1536, 0), (2048, 333, 6144, 1536, 1), (512, 77, 256, 256, 0),
                                           (300, 300, 1536, 6144, 0)])
def test_linear_pair_equals_two_linears(sd3, M0, M1, N, K, act):
    """sd3_linear_pair / sd3_linear_gate_residual_pair: two GEMMs of one shape class in one
    launch give what the two single calls give."""
    from ctypes import c_void_p
    gen = torch.Generator(device="cuda").manual_seed(M0 + M1 + N)
    xs = [torch.randn(m, K, device="cuda", generator=gen).bfloat16() for m in (M0, M1)]
    ws = [(torch.randn(N, K, device="cuda", generator=gen) * 0.03).bfloat16() for _ in range(2)]
    bs = [torch.randn(N, device="cuda", generator=gen) * 0.1 for _ in range(2)]
    ref = [sd3.linear(xs[i], ws[i], bs[i], act=act) for i in range(2)]
    outs = [torch.empty_like(r) for r in ref]
    sd3.check(sd3.lib().sd3_linear_pair(sd3.ptr(xs[0]), sd3.ptr(ws[0]), sd3.ptr(bs[0]), sd3.ptr(outs[0]), M0,
                                        sd3.ptr(xs[1]), sd3.ptr(ws[1]), sd3.ptr(bs[1]), sd3.ptr(outs[1]), M1,
                                        sd3.dtype_tag(outs[0]), N, K, act, sd3.stream_ptr()), "sd3_linear_pair")
    torch.cuda.synchronize()
    for o, r in zip(outs, ref):
        assert rel_l2(o, r) < 1e-5
    # gate + residual form
    gates = [torch.randn(1, N, device="cuda", generator=gen) for _ in range(2)]
    res0 = [torch.randn(m, N, device="cuda", generator=gen) for m in (M0, M1)]
    want = [sd3.linear_gate_residual(xs[i], ws[i], bs[i], gates[i], xs[i].shape[0], res0[i].clone()) for i in range(2)]
    got = [r.clone() for r in res0]
    sd3.check(sd3.lib().sd3_linear_gate_residual_pair(
        sd3.ptr(xs[0]), sd3.ptr(ws[0]), sd3.ptr(bs[0]), sd3.ptr(gates[0]), M0, sd3.ptr(got[0]), M0,
        sd3.ptr(xs[1]), sd3.ptr(ws[1]), sd3.ptr(bs[1]), sd3.ptr(gates[1]), M1, sd3.ptr(got[1]), M1,
        0, N, K, sd3.stream_ptr()), "sd3_linear_gate_residual_pair")
    torch.cuda.synchronize()
    assert sd3.device_status() == 0
    for o, r in zip(got, want):
        assert rel_l2(o, r) < 1e-5
