"""Channel shards on real GPUs: two ranks, each running the CUDA kernels on its half of the hidden channels of one
seeded problem and all-gathering the block output over NCCL, reproduce the un-sharded CUDA output bit for bit.
Needs two CUDA devices (skipped otherwise); plain NCCL on local buffers, NVLS off."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, kind, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", NCCL_DEBUG="WARN")
    import torch.distributed as dist
    from helpers import cuda, make_block
    from vortex_b200 import hyena_ops, ops, sharding
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    B, L, D, G = 2, 1500, 512, 32
    K = {"se": 7, "mr": 128}[kind]
    p = make_block(91, B, L, D, G, K, "bf16")              # the same seed on every rank: one problem

    def block(q):
        q = cuda(q)
        if K >= 128:
            return hyena_ops.hyena_mr_fwd(q["u"].contiguous(), q["w3"], None, q["h"], q["Dp"], want_state=True)
        return hyena_ops.hyena_se_fwd(q["u"].contiguous(), q["w3"], None, q["h"], want_state=True)

    sh = sharding.shard_block(p, D, G, world, rank, layout="interleaved")
    y, fs, st = block(sh)
    ops.device_status()
    widths = [b - a for a, b in (sharding.channel_range(D, G, world, r) for r in range(world))]
    full = sharding.gather_channels(y, widths=widths)
    stacked = sharding.gather_channels(y, widths=widths, concat=False)
    ok = True
    if rank == 0:
        y1, fs1, st1 = block(p)                            # the whole problem on one GPU
        d0, d1 = sharding.channel_range(D, G, world, rank)
        ok = torch.equal(full, y1) and torch.equal(st, st1[:, d0:d1]) and torch.equal(fs, fs1[:, 3 * d0:3 * d1])
        ok = ok and all(torch.equal(stacked[r], y1[..., sum(widths[:r]):sum(widths[:r + 1])]) for r in range(world))
    out.put((rank, bool(ok)))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("kind", ["mr", "se"])
def test_two_gpu_channel_shards_gathered_equal_one_gpu(kind):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, kind, out)) for r in range(2)]
    for pr in procs:
        pr.start()
    got = [out.get(timeout=300) for _ in range(2)]
    for pr in procs:
        pr.join(timeout=120)
        assert pr.exitcode == 0
    assert all(ok for _, ok in got), got
