"""Shard planning on CPU: slices are exact, and a 2-rank gloo run (each rank evaluating its shard with the
oracle, then the boundary all-gather) reproduces the un-sharded oracle bit for bit."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from helpers import make_block, to_np
from oracle import hyena_oracle as O
from vortex_b200 import sharding


def test_ranges_cover_everything():
    for D, G, W in ((4096, 256, 8), (768, 48, 4), (96, 6, 4), (64, 4, 3)):
        got = [sharding.channel_range(D, G, W, r) for r in range(W)]
        assert got[0][0] == 0 and got[-1][1] == D
        assert all(a[1] == b[0] for a, b in zip(got, got[1:]))
        assert all((hi - lo) % (D // G) == 0 and hi > lo for lo, hi in got)
    assert [sharding.batch_range(64, 8, r) for r in (0, 7)] == [(0, 8), (56, 64)]
    with pytest.raises(ValueError):
        sharding.channel_range(64, 4, 8, 0)


@pytest.mark.parametrize("layout,heads", [("interleaved", 1), ("split", 1), ("column_split", 4)])
def test_packed_columns_match_the_channel_maps(layout, heads):
    D, d0, d1 = 64, 16, 48
    cols = sharding.packed_columns(D, d0, d1, layout, heads).numpy()
    q, k, v = O.qkv_index(D, layout, heads)
    qs, ks, vs = O.qkv_index(d1 - d0, layout, max(1, heads * (d1 - d0) // D))
    # column i of the shard's packed tensor must be the column of the full tensor that feeds the same role
    for full, part in ((q, qs), (k, ks), (v, vs)):
        assert np.array_equal(cols[part], full[d0:d1])


def _worker(rank, world, port, layout, K, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    B, L, D, G = 2, 150, 64, 4
    p = make_block(77, B, L, D, G, K, "f32")              # same seed on every rank: identical full problem
    sh = sharding.shard_block(p, D, G, world, rank, layout=layout, num_heads=2)
    d0, d1 = sharding.channel_range(D, G, world, rank)
    y, _, _ = O.hyena_fused(to_np(sh["u"]), to_np(sh["w3"]), to_np(sh["h"]), None if sh["Dp"] is None else to_np(sh["Dp"]),
                            d1 - d0, K, io="f32", layout=layout, num_heads=1 if layout != "column_split" else 1)
    full = sharding.gather_channels(torch.from_numpy(y))
    if rank == 0:
        ref, _, _ = O.hyena_fused(to_np(p["u"]), to_np(p["w3"]), to_np(p["h"]), None if p["Dp"] is None else to_np(p["Dp"]),
                                  D, K, io="f32", layout=layout, num_heads=2)
        out.put(bool(np.array_equal(full.numpy(), ref)))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("layout,K", [("interleaved", 7), ("split", 128), ("column_split", 7)])
def test_two_rank_channel_sharding_equals_unsharded(layout, K):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, layout, K, out)) for r in range(2)]
    for pr in procs:
        pr.start()
    ok = out.get(timeout=120)
    for pr in procs:
        pr.join(timeout=60)
        assert pr.exitcode == 0
    assert ok


def _uneven_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    B, L, D, G = 2, 5, 64, 4                                   # 4 groups on 3 ranks: 1, 1 and 2 groups
    full = torch.arange(B * L * D, dtype=torch.float32).reshape(B, L, D)
    d0, d1 = sharding.channel_range(D, G, world, rank)
    widths = [b - a for a, b in (sharding.channel_range(D, G, world, r) for r in range(world))]
    ok = torch.equal(sharding.gather_channels(full[..., d0:d1]), full)                     # widths exchanged
    ok = ok and torch.equal(sharding.gather_channels(full[..., d0:d1], widths=widths), full)   # widths given
    try:
        sharding.gather_channels(full[..., d0:d1], widths=[D // world] * world)
        ok = False
    except ValueError:
        pass
    out.put((rank, bool(ok), widths))
    dist.barrier()
    dist.destroy_process_group()


def test_gather_of_uneven_channel_shards():
    """channel_range hands out whole filter groups, so 4 groups on 3 ranks give shards of 16, 16 and 32 channels:
    the boundary all-gather pads to the widest shard for the exchange and returns the exact concatenation."""
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_uneven_worker, args=(r, 3, port, out)) for r in range(3)]
    for pr in procs:
        pr.start()
    got = [out.get(timeout=120) for _ in range(3)]
    for pr in procs:
        pr.join(timeout=60)
        assert pr.exitcode == 0
    assert all(ok for _, ok, _ in got), got
    assert got[0][2] == [16, 16, 32]
