"""Batch sharding across ranks (the multi-GPU mode has no data-path
collective): world_size-2 gloo processes on CPU each take their contiguous
slice of the batch, run the per-sample computation (the CPU oracle stands in
for the device here), and the gathered result must equal the unsharded run
bit for bit, because samples never interact."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import REPO, golden, load_binding
from oracle import mmdit_oracle as O


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sys.path.insert(0, REPO)
        s = load_binding()
        g = golden("model_toy.pt")
        cfg = g["config"]
        p = {k: v.float() for k, v in g["params"].items()}
        B = g["latent"].shape[0]
        lo, hi = s.shard_range(B, world, rank)
        out = O.dit_forward(g["pooled"].float()[lo:hi], g["captions"].float()[lo:hi],
                            g["latent"].float()[lo:hi], g["timesteps"][lo:hi], p, cfg["num_layers"],
                            cfg["dual_attention_layers"], cfg["attn_heads"], cfg["patch_size"],
                            cfg["pos_embed_max_size"], cfg["base_height"], True)
        gathered = [None] * world
        dist.all_gather_object(gathered, (lo, hi, out))
        # max-over-ranks timing reduction used by the benchmark
        t = torch.tensor([float(rank + 1)])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            full = torch.cat([o for _, _, o in sorted(gathered, key=lambda x: x[0])], 0)
            ret["out"] = full
            ret["tmax"] = t.item()
            ret["ranges"] = [(a, b) for a, b, _ in gathered]
    finally:
        dist.destroy_process_group()


def test_batch_sharding_two_ranks_matches_single():
    g = golden("model_toy.pt")
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    assert ret["tmax"] == 2.0
    assert sorted(ret["ranges"]) == [(0, 1), (1, 2)]
    assert (ret["out"] - g["out"]).abs().max().item() < 1e-5
    cfg = g["config"]
    p = {k: v.float() for k, v in g["params"].items()}
    single = O.dit_forward(g["pooled"].float(), g["captions"].float(), g["latent"].float(),
                           g["timesteps"], p, cfg["num_layers"], cfg["dual_attention_layers"],
                           cfg["attn_heads"], cfg["patch_size"], cfg["pos_embed_max_size"],
                           cfg["base_height"], True)
    # per-sample results do not depend on which rank computed them
    assert torch.allclose(ret["out"], single, atol=1e-6, rtol=0)


def test_shard_range_covers_batch_without_overlap():
    s = load_binding()
    for n in (1, 2, 7, 8, 32):
        for world in (1, 2, 3, 4, 8):
            spans = [s.shard_range(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for (a, b), (c, d) in zip(spans, spans[1:]):
                assert b == c and a <= b
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
