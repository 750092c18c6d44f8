"""Sequence sharding around attention (Ulysses): the re-layout math on CPU with
emulated ranks, and the full sharded forward on 2 GPUs (NCCL) against the
golden toy model."""
import importlib.util
import os
import sys

import pytest
import torch

from conftest import REPO, golden, load_binding
from oracle import mmdit_oracle as O


def load_ulysses():
    name = "sd3_ulysses"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, os.path.join(REPO, "sd3.c_b200", "ulysses.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("P,NH,Tc,Tl", [(2, 4, 5, 6), (4, 8, 3, 2), (8, 24, 7, 3), (1, 2, 4, 9)])
def test_relayout_with_emulated_ranks_equals_unsharded_attention(P, NH, Tc, Tl):
    U = load_ulysses()
    torch.manual_seed(P * 100 + NH)
    D = 8
    E = NH * D
    Tx = P * Tl
    ctx = torch.randn(Tc, 3 * E)
    img = torch.randn(Tx, 3 * E)
    # unsharded reference: context rows first
    full = torch.cat([ctx, img], 0)
    q, k, v = (t.reshape(1, Tc + Tx, NH, D) for t in full.chunk(3, -1))
    ref = O.attention(q, k, v)[0]  # (T, E)
    # every rank prepares its slabs; the all-to-all is emulated by indexing
    send = [U.split_heads_for_send(img[r * Tl:(r + 1) * Tl].contiguous(), P) for r in range(P)]
    o_ctx_parts, o_img_send = [], []
    for r in range(P):
        recv = torch.stack([send[s][r] for s in range(P)], 0)  # slab from every source rank
        att_in = U.assemble_attention_input(ctx, recv, r, P)   # (1, T, 3E/P)
        qq, kk, vv = (t.reshape(1, Tc + Tx, NH // P, D) for t in att_in.chunk(3, -1))
        o = O.attention(qq, kk, vv)[0]                         # (T, E/P): my heads
        o_ctx_parts.append(o[:Tc])
        o_img_send.append(U.split_tokens_for_send(o[Tc:].contiguous(), P))
    for r in range(P):
        recv = torch.stack([o_img_send[s][r] for s in range(P)], 0)
        rows = U.assemble_rows(recv)                           # (Tl, E)
        assert torch.allclose(rows, ref[Tc + r * Tl:Tc + (r + 1) * Tl], atol=1e-5)
    o_ctx = U.assemble_rows(torch.stack(o_ctx_parts, 0))
    assert torch.allclose(o_ctx, ref[:Tc], atol=1e-5)


def _gpu_worker(rank, world, port, ret):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        sys.path.insert(0, REPO)
        sd3 = load_binding()
        U = load_ulysses()
        g = golden("model_toy.pt")
        cfg = g["config"]
        pm = U.PackedModel(sd3, g["params"], cfg)
        comm = U.DistComm()
        outs = []
        for b in range(g["latent"].shape[0]):  # one sample at a time
            out = U.dit_forward_sharded(pm, g["pooled"][b:b + 1].cuda(), g["captions"][b:b + 1].cuda(),
                                        g["latent"][b:b + 1].cuda(), g["timesteps"][b:b + 1].cuda(), comm)
            outs.append(out)
        torch.cuda.synchronize()
        assert sd3.device_status() == 0
        ret[rank] = torch.cat(outs, 0).cpu()
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
def test_sharded_forward_two_gpus_matches_golden():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    g = golden("model_toy.pt")
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29600 + (os.getpid() % 1000)
    mp.spawn(_gpu_worker, args=(2, port, ret), nprocs=2, join=True)
    for r in range(2):
        rel = ((ret[r] - g["out"]).norm() / g["out"].norm()).item()
        assert rel < 1e-2, rel
    assert torch.equal(ret[0], ret[1])


@pytest.mark.gpu
def test_sharded_forward_one_rank_matches_golden():
    """The sharded forward with the one-rank communicator (every exchange is a copy): the
    whole sequence-parallel code path on a single GPU against the golden toy model."""
    sd3 = load_binding()
    U = load_ulysses()
    g = golden("model_toy.pt")
    pm = U.PackedModel(sd3, g["params"], g["config"])
    comm = U.LocalComm()
    outs = [U.dit_forward_sharded(pm, g["pooled"][b:b + 1].cuda(), g["captions"][b:b + 1].cuda(),
                                  g["latent"][b:b + 1].cuda(), g["timesteps"][b:b + 1].cuda(), comm)
            for b in range(g["latent"].shape[0])]
    torch.cuda.synchronize()
    assert sd3.device_status() == 0
    out = torch.cat(outs, 0).cpu()
    assert ((out - g["out"]).norm() / g["out"].norm()).item() < 1e-2


@pytest.mark.gpu
@pytest.mark.parametrize("rows,E,K,G", [(300, 256, 256, 2), (512, 512, 256, 4), (77, 192, 1536, 1), (1024, 1536, 1536, 8)])
def test_qkv_project_head_group_layout(rows, E, K, G):
    """sd3_qkv_project_groups writes (groups, rows, 3, E/groups): the all-to-all send layout,
    equal to re-laying the plain (rows, 3E) projection with split_heads_for_send."""
    sd3 = load_binding()
    U = load_ulysses()
    gen = torch.Generator(device="cuda").manual_seed(rows + G)
    x = torch.randn(rows, K, device="cuda", generator=gen).bfloat16()
    w = (torch.randn(3 * E, K, device="cuda", generator=gen) * 0.05).bfloat16()
    b = torch.randn(3 * E, device="cuda", generator=gen) * 0.1
    wq = 1.0 + 0.2 * torch.randn(64, device="cuda", generator=gen)
    wk = 1.0 + 0.2 * torch.randn(64, device="cuda", generator=gen)
    out = torch.empty(G, rows, 3, E // G, device="cuda", dtype=torch.bfloat16)
    sd3.qkv_project_groups(x, w, b, wq, wk, 1e-6, out, E, G)
    # reference: fp32 linear + per-head RMSNorm on q and k, then the re-layout
    y = x.float() @ w.float().t() + b
    q, k, v = y.split(E, dim=-1)

    def rms(t, wt):
        t = t.view(rows, E // 64, 64)
        return (t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + 1e-6) * wt).view(rows, E)

    ref = torch.cat([rms(q, wq), rms(k, wk), v], -1)
    ref = U.split_heads_for_send(ref.contiguous(), G)
    torch.cuda.synchronize()
    assert sd3.device_status() == 0
    assert ((out.float() - ref).norm() / ref.norm()).item() < 1e-2


def _gloo_worker(rank, world, port, ret):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        U = load_ulysses()
        comm = U.DistComm()
        torch.manual_seed(7)  # same tensors on every rank
        NH, D, Tc, Tl = 4, 8, 3, 5
        E, P = NH * D, world
        Eh = E // P
        ctx = torch.randn(Tc, 3 * E)
        img = torch.randn(P * Tl, 3 * E)
        mine = img[rank * Tl:(rank + 1) * Tl].contiguous()
        send = U.split_heads_for_send(mine, P)                     # (P, Tl, 3, Eh)
        recv = torch.empty_like(send)
        h = comm.all_to_all_start(recv, send)                       # asynchronous form
        recv2 = torch.empty_like(send)
        comm.all_to_all_into(recv2, send)                           # blocking form
        h.wait()
        assert torch.equal(recv, recv2)
        att_in = U.assemble_attention_input(ctx, recv, rank, P)     # (1, T, 3 Eh)
        q, k, v = (t.reshape(1, Tc + P * Tl, NH // P, D) for t in att_in.chunk(3, -1))
        o = O.attention(q, k, v)[0]                                 # my heads, all rows
        back = torch.empty(P, Tl, Eh)
        comm.all_to_all_into(back, U.split_tokens_for_send(o[Tc:].contiguous(), P))
        rows = U.assemble_rows(back)                                # my rows, all heads
        gath = torch.empty(P, Tc, Eh)
        comm.all_gather_into(gath, o[:Tc].contiguous())
        ret[rank] = (rows, U.assemble_rows(gath))
    finally:
        dist.destroy_process_group()


def test_exchanges_through_dist_comm_two_gloo_ranks():
    """The communicator's three calls (blocking and asynchronous all-to-all, all-gather) on two
    gloo ranks on the CPU: sharded attention equals the unsharded one."""
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29700 + (os.getpid() % 1000)
    mp.spawn(_gloo_worker, args=(2, port, ret), nprocs=2, join=True)
    torch.manual_seed(7)
    NH, D, Tc, Tl, P = 4, 8, 3, 5, 2
    E = NH * D
    ctx = torch.randn(Tc, 3 * E)
    img = torch.randn(P * Tl, 3 * E)
    full = torch.cat([ctx, img], 0)
    q, k, v = (t.reshape(1, Tc + P * Tl, NH, D) for t in full.chunk(3, -1))
    ref = O.attention(q, k, v)[0]
    for r in range(P):
        rows, ctx_rows = ret[r]
        assert torch.allclose(rows, ref[Tc + r * Tl:Tc + (r + 1) * Tl], atol=1e-5)
        assert torch.allclose(ctx_rows, ref[:Tc], atol=1e-5)
