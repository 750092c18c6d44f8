"""sd3_patch_embed_static: the allocation-free variant of the patch-embedding
operator, for callers that cannot call cudaMalloc where they run it
(allocator-free serving loops, fixed memory budgets).  Its scratch is a fixed
array inside the library, shared by all calls on a device.

This file is collected last on purpose: a run that stops at the first failure
has then already executed every other test.  The test passes on its own in a
fresh process and after the rest of the suite."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(seed, B, C, H, W, E, patch, sd3):
    g = torch.Generator(device="cuda").manual_seed(seed)
    lat = torch.randn(B, C, H, W, device="cuda", generator=g).bfloat16()
    w = (torch.randn(E, C * patch * patch, device="cuda", generator=g) * 0.1).bfloat16()
    b = torch.randn(E, device="cuda", generator=g)
    pt = sd3.pos_embed_table(H // patch, W // patch, E, 96, 32)
    return lat, w, b, pt


def test_static_scratch_matches_caller_scratch_twice_in_a_row(sd3):
    # two different problems back to back: the second call finds the first
    # call's patches still in the shared array and must not be affected by them
    for seed, (B, C, H, W, E) in enumerate([(2, 16, 32, 48, 256), (3, 16, 16, 16, 128)]):
        lat, w, b, pt = _inputs(seed, B, C, H, W, E, 2, sd3)
        ref = sd3.patch_embed(lat, w, b, pt, 2, E)          # existing entry point, caller scratch
        out = torch.empty_like(ref)
        got = sd3.patch_embed_static(lat, w, b, pt, 2, E, out=out)
        torch.cuda.synchronize()
        # same kernels on the same data: identical bits (the suite's fp32-out bound is 1e-4)
        assert (got - ref).abs().max().item() <= 1e-4
        assert torch.equal(got, ref)
    assert sd3.device_status() == 0


def test_static_scratch_rejects_oversized_problems(sd3):
    # 8 * 512 * 512 * 64 elements > SD3_STATIC_PATCH_ELEMS: rejected before any launch
    B, C, H, W, E = 8, 16, 1024, 1024, 128
    assert B * (H // 2) * (W // 2) * C * 4 > sd3.STATIC_PATCH_ELEMS
    lat = torch.empty(1, device="cuda", dtype=torch.bfloat16)  # never dereferenced
    w = torch.empty(E, C * 4, device="cuda", dtype=torch.bfloat16)
    b = torch.zeros(E, device="cuda")
    pt = torch.zeros(8, device="cuda")
    out = torch.empty(8, device="cuda")
    rc = sd3.lib().sd3_patch_embed_static(sd3.ptr(lat), sd3.DTYPE_BF16, sd3.ptr(w), sd3.ptr(b), sd3.ptr(pt),
                                          sd3.ptr(out), B, C, H, W, 2, E, sd3.stream_ptr())
    assert rc == -2
    assert b"built-in scratch" in sd3.lib().sd3_last_error()


def test_static_call_allocates_nothing_once_warm(sd3):
    # after one warm call (symbol addresses, kernel attributes and the tensor-map entry
    # point resolved) a call with a preallocated output leaves the allocator untouched
    lat, w, b, pt = _inputs(7, 2, 16, 32, 32, 256, 2, sd3)
    out = torch.empty(2 * 16 * 16, 256, device="cuda")
    sd3.patch_embed_static(lat, w, b, pt, 2, 256, out=out)
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    alloc0 = torch.cuda.memory_allocated()
    sd3.patch_embed_static(lat, w, b, pt, 2, 256, out=out)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == alloc0
    assert torch.cuda.mem_get_info()[0] == free0  # the driver's view: nothing was allocated or freed
    assert torch.equal(out, sd3.patch_embed(lat, w, b, pt, 2, 256))


def test_static_binding_validates_tensors(sd3):
    lat, w, b, pt = _inputs(8, 1, 16, 16, 16, 128, 2, sd3)
    with pytest.raises(sd3.Sd3Error):  # output too small
        sd3.patch_embed_static(lat, w, b, pt, 2, 128, out=torch.empty(10, 128, device="cuda"))
    with pytest.raises(sd3.Sd3Error):  # wrong dtype
        sd3.patch_embed_static(lat, w, b, pt, 2, 128, out=torch.empty(64, 128, device="cuda", dtype=torch.bfloat16))
    with pytest.raises(sd3.Sd3Error):  # weight of the wrong shape
        sd3.patch_embed_static(lat, w[:, :32].contiguous(), b, pt, 2, 128)
